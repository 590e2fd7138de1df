"""Training-step helpers around the causal LM: a fixed-denominator chunked linear +
cross-entropy loss, FP32 master weights behind the BF16 model weights, gradient
averaging over a process group, and a fixed-shape training step replayed from a CUDA graph.

Counterparts upstream: ``causallsso/graph_linear_cross_entropy.py:29-209``
(``fixed_dense_linear_cross_entropy``), ``causallsso/bf16_shadow.py:60-180``
(``BF16ShadowWeights``) and ``causallsso/cuda_graph.py:75-331``
(``SolveDeltaGraphedTrainingStep``).  The division of labour is the same (the optimizer
and the collectives stay outside the captured graph, one instance per batch shape, the
loss denominator is a constant so nothing inside the graph depends on data), the
mechanics differ: here the model's own parameters are the BF16 copies and the FP32
masters live beside them, and forward and backward are captured as one graph.
"""
from __future__ import annotations

import ctypes
from contextlib import contextmanager
from typing import Any, Iterable, List, Optional

import torch
import torch.distributed as dist
from torch import nn

from . import _lib


def _ce_rows(logits: torch.Tensor, labels: torch.Tensor, ignore_index: int):
    """Per row of BF16 CUDA logits ``[N, V]``: log-sum-exp and -log softmax(label) (0 where ignored), one kernel."""
    lib = _lib.load()
    rows, vocab = logits.shape
    with torch.cuda.device(logits.device):
        lse = torch.empty(rows, dtype=torch.float32, device=logits.device)
        row_loss = torch.empty(rows, dtype=torch.float32, device=logits.device)
        a = _lib.CrossEntropyArgs(rows, vocab, logits.data_ptr(), labels.data_ptr(), int(ignore_index),
                                  lse.data_ptr(), row_loss.data_ptr(), None, None)
        stream = ctypes.c_void_p(torch.cuda.current_stream(logits.device).cuda_stream)
        _lib.check(lib.sd_cross_entropy_forward(ctypes.byref(a), stream))
    return lse, row_loss


def _ce_grad(logits: torch.Tensor, labels: torch.Tensor, lse: torch.Tensor, coef: torch.Tensor, ignore_index: int):
    """d logits = (softmax - onehot(label)) * coef in BF16 (zeros where ignored); ``coef`` an FP32 device scalar."""
    lib = _lib.load()
    rows, vocab = logits.shape
    with torch.cuda.device(logits.device):
        dlogits = torch.empty_like(logits)
        a = _lib.CrossEntropyArgs(rows, vocab, logits.data_ptr(), labels.data_ptr(), int(ignore_index),
                                  lse.data_ptr(), None, coef.data_ptr(), dlogits.data_ptr())
        stream = ctypes.c_void_p(torch.cuda.current_stream(logits.device).cuda_stream)
        _lib.check(lib.sd_cross_entropy_backward(ctypes.byref(a), stream))
    return dlogits


class _FixedDenseLinearCrossEntropy(torch.autograd.Function):
    """loss = sum over valid tokens of CE(x W^T + b, target) / total, evaluated in token
    chunks so that the [tokens, vocab] logits never exist at once.  The gradients with
    respect to x, W and b are formed in the forward pass (while each chunk's logits are
    at hand) and scaled by the incoming cotangent in backward."""

    @staticmethod
    def forward(ctx, x, target, weight, bias, ignore_index, total, num_chunks):
        lead = x.shape[:-1]
        x2 = x.reshape(-1, x.shape[-1])
        t = target.reshape(-1)
        tokens = x2.shape[0]
        need = [ctx.needs_input_grad[0], ctx.needs_input_grad[2], bias is not None and ctx.needs_input_grad[3]]
        dx = torch.empty_like(x2) if need[0] else None
        dw = torch.zeros_like(weight, dtype=torch.float32) if need[1] else None
        db = torch.zeros_like(bias, dtype=torch.float32) if need[2] else None
        loss = torch.zeros((), dtype=torch.float32, device=x.device)
        step = -(-tokens // max(1, num_chunks))
        # a tensor denominator (the count of valid labels, taken on the device) stays on the device: no host sync
        scale = (1.0 / total.to(torch.float32)) if torch.is_tensor(total) else 1.0 / float(total)
        on_kernels = x2.is_cuda and x2.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and t.dtype == torch.long
        if on_kernels:   # the loss kernels work on the BF16 logits of a chunk as the projection leaves them
            coef = (scale if torch.is_tensor(scale) else torch.full((), scale, device=x.device)).reshape(1).float()
        for lo in range(0, tokens, step):
            xs, ts = x2[lo:lo + step], t[lo:lo + step]
            if on_kernels:
                logits = torch.nn.functional.linear(xs, weight, bias)
                ts = ts.contiguous()
                lse, row_loss = _ce_rows(logits, ts, ignore_index)
                loss = loss + row_loss.sum() * scale
                if need[0] or need[1] or need[2]:
                    g = _ce_grad(logits, ts, lse, coef, ignore_index)
                    if need[0]:
                        dx[lo:lo + step] = g @ weight
                    if need[1]:
                        dw.add_((g.t() @ xs).float())
                    if need[2]:
                        db.add_(g.float().sum(0))
                continue
            logits = torch.nn.functional.linear(xs, weight, bias).float()
            valid = ts != ignore_index
            safe = torch.where(valid, ts, torch.zeros_like(ts))
            logz = torch.logsumexp(logits, dim=-1)
            picked = logits.gather(1, safe.unsqueeze(1)).squeeze(1)
            loss = loss + torch.where(valid, logz - picked, torch.zeros_like(logz)).sum() * scale
            if need[0] or need[1] or need[2]:
                g = torch.softmax(logits, dim=-1)
                g.scatter_add_(1, safe.unsqueeze(1), -torch.ones_like(picked).unsqueeze(1))
                g = (g * (valid.unsqueeze(1).float() * scale)).to(x.dtype)
                if need[0]:
                    dx[lo:lo + step] = g @ weight
                if need[1]:
                    dw.add_((g.t() @ xs).float())
                if need[2]:
                    db.add_(g.float().sum(0))
        ctx.lead = lead
        ctx.save_for_backward(*(v for v in (dx, dw, db) if v is not None))
        ctx.have = [v is not None for v in (dx, dw, db)]
        ctx.dtypes = (weight.dtype, None if bias is None else bias.dtype)
        return loss

    @staticmethod
    def backward(ctx, grad_loss):
        saved = list(ctx.saved_tensors)
        dx = saved.pop(0) if ctx.have[0] else None
        dw = saved.pop(0) if ctx.have[1] else None
        db = saved.pop(0) if ctx.have[2] else None
        if dx is not None:
            dx = (dx * grad_loss.to(dx.dtype)).reshape(*ctx.lead, dx.shape[-1])
        if dw is not None:
            dw = (dw * grad_loss).to(ctx.dtypes[0])
        if db is not None:
            db = (db * grad_loss).to(ctx.dtypes[1])
        return dx, None, dw, db, None, None, None


def fixed_dense_linear_cross_entropy(x: torch.Tensor, target: torch.Tensor, weight: torch.Tensor,
                                     bias: Optional[torch.Tensor] = None, *, ignore_index: int = -100,
                                     total, num_chunks: int = 8) -> torch.Tensor:
    """Linear layer and cross entropy in one pass over token chunks, divided by the CONSTANT
    ``total`` (the number of valid labels of the fixed batch shape) instead of a count taken
    from the data, so a captured graph holds no data-dependent scalar (upstream
    graph_linear_cross_entropy.py:186-209).  ``total`` may also be a 0-dim tensor on the device of
    ``x`` (e.g. the count of valid labels): the mean then matches ``F.cross_entropy`` without a host read."""
    if torch.is_tensor(total):
        if total.ndim != 0 or total.device != x.device:
            raise ValueError("a tensor total must be a scalar on the device of x")
    elif not isinstance(total, int) or isinstance(total, bool) or total <= 0:
        raise ValueError("total must be a positive int")
    if x.shape[:-1] != target.shape:
        raise ValueError("target must have the leading shape of x")
    if weight.ndim != 2 or weight.shape[1] != x.shape[-1]:
        raise ValueError("weight must have shape [vocab, hidden]")
    return _FixedDenseLinearCrossEntropy.apply(x, target, weight, bias, ignore_index, total, num_chunks)


class _FusedCrossEntropy(torch.autograd.Function):
    """Mean cross entropy over BF16 logits in two kernels: the forward reads every row once (log-sum-exp and the
    label's term), the reverse writes d logits = (softmax - onehot) * cotangent / count in BF16.  The FP32 copy of the
    [tokens, vocab] logits that ``F.cross_entropy(logits.float(), ...)`` makes never exists."""

    @staticmethod
    def forward(ctx, logits, labels, ignore_index, count):
        lse, row_loss = _ce_rows(logits, labels, ignore_index)
        ctx.save_for_backward(logits, labels, lse, count)
        ctx.ignore_index = int(ignore_index)
        return row_loss.sum() / count

    @staticmethod
    def backward(ctx, gout):
        logits, labels, lse, count = ctx.saved_tensors
        coef = (gout.float() / count).reshape(1).contiguous()
        return _ce_grad(logits, labels, lse, coef, ctx.ignore_index), None, None, None


def fused_cross_entropy(logits: torch.Tensor, labels: torch.Tensor, *, ignore_index: int = -100) -> torch.Tensor:
    """``F.cross_entropy(logits.float(), labels, ignore_index=...)`` (mean over the counted tokens) for BF16 CUDA
    logits ``[..., V]`` and ``torch.long`` labels ``[...]``, the role of upstream's ``FusedCrossEntropyLoss``
    (``modeling_solvedelta.py:469-470``).  The token count is taken on the device (no host synchronisation); with no
    counted token the loss is 0 where PyTorch returns NaN."""
    if logits.device.type != "cuda" or logits.dtype != torch.bfloat16:
        raise TypeError("logits must be a BF16 CUDA tensor")
    if labels.dtype != torch.long:
        raise TypeError("labels must be torch.long")
    if labels.shape != logits.shape[:-1]:
        raise ValueError("labels must have the shape of logits without its last axis")
    flat = logits.reshape(-1, logits.shape[-1]).contiguous()
    target = labels.reshape(-1).to(logits.device).contiguous()
    count = (target != ignore_index).sum().clamp_min(1).to(torch.float32)
    return _FusedCrossEntropy.apply(flat, target, ignore_index, count)


class BF16ShadowWeights:
    """FP32 master weights for a model whose own parameters are the BF16 copies the kernels read.

    ``optimizer_factory(masters)`` builds the optimizer over the FP32 masters, which own the
    update and the checkpoint.  A pre-step hook hands each parameter's gradient to its master in
    FP32, a post-step hook copies the updated masters back into the model (one cast per optimizer
    step, not per micro-batch, as upstream bf16_shadow.py:147-165) and clears the gradients."""

    def __init__(self, model: nn.Module, optimizer_factory) -> None:
        self.params: List[torch.Tensor] = [p for p in model.parameters() if p.requires_grad]
        self.masters: List[torch.Tensor] = [p.detach().float().clone().requires_grad_() for p in self.params]
        self.optimizer: torch.optim.Optimizer = optimizer_factory(self.masters)
        self._current = True
        self.optimizer.register_step_pre_hook(self._pre_step)
        self.optimizer.register_step_post_hook(self._post_step)

    def _pre_step(self, optimizer, args, kwargs) -> None:
        for master, param in zip(self.masters, self.params):
            if param.grad is None:
                master.grad = None
            elif master.grad is None:
                master.grad = param.grad.float()
            else:
                master.grad.copy_(param.grad)
        self._current = False

    def _post_step(self, optimizer, args, kwargs) -> None:
        self.refresh()
        for param in self.params:
            if param.grad is not None:
                param.grad.zero_()   # in place: a captured backward accumulates into this storage

    @torch.no_grad()
    def refresh(self) -> None:
        """Copy the masters into the model's parameters (after any change to the masters)."""
        for master, param in zip(self.masters, self.params):
            param.copy_(master)
        self._current = True

    def assert_current(self) -> None:
        if not self._current:
            raise RuntimeError("BF16 weights are stale: the optimizer stepped without a refresh")

    @property
    def nbytes(self) -> int:
        return sum(m.numel() * m.element_size() for m in self.masters)


@torch.no_grad()
def allreduce_gradients(params: Iterable[torch.Tensor], group: Any = None) -> int:
    """Average the gradients over the process group, one flat bucket per dtype (the whole model
    fits one bucket: NVSwitch makes launch count, not link count, the cost).  Returns the number of
    collectives issued.  Parameters without a gradient are skipped on every rank alike."""
    if not dist.is_available() or not dist.is_initialized():
        return 0
    world = dist.get_world_size(group)
    if world == 1:
        return 0
    buckets = {}
    for p in params:
        if p.grad is not None:
            buckets.setdefault(p.grad.dtype, []).append(p.grad)
    issued = 0
    for dtype in sorted(buckets, key=str):
        grads = buckets[dtype]
        flat = torch._utils._flatten_dense_tensors(grads)
        dist.all_reduce(flat, op=dist.ReduceOp.SUM, group=group)
        flat.div_(world)
        for g, piece in zip(grads, torch._utils._unflatten_dense_tensors(flat, grads)):
            g.copy_(piece)
        issued += 1
    return issued


class BucketedGradientAverager:
    """Gradient averaging overlapped with the backward pass (the role torch DDP plays upstream with
    ``gradient_as_bucket_view=True``, causallsso/cuda_graph.py:250-262).

    Parameters are grouped, last registered first (roughly the order backward produces gradients),
    into flat buckets of about ``bucket_bytes`` per gradient dtype.  Every parameter's ``.grad`` is a view
    of its bucket, so backward accumulates straight into the bucket and nothing is copied.  A
    post-accumulate hook counts the gradients of a bucket; when the last one arrives the bucket's
    all-reduce is launched asynchronously, on the communication stream of the process group, while
    backward carries on with earlier layers.  ``finish()`` waits for the collectives and divides by the
    world size; ``zero_grad()`` clears the buckets and keeps the views.  Parameters that receive no
    gradient in a step would stall their bucket, so ``finish()`` launches whatever is still pending
    (with whatever those buckets hold); every rank must skip the same parameters.

    The graph-replayed step cannot use it (hooks do not run during a replay): it keeps the single flat
    all-reduce after the replay.
    """

    def __init__(self, params: Iterable[torch.Tensor], group: Any = None, bucket_bytes: int = 64 << 20) -> None:
        self.group = group
        self.enabled = dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1
        self.world = dist.get_world_size(group) if self.enabled else 1
        self.params = [p for p in params if p.requires_grad]
        self.buckets: List[dict] = []
        self._hooks = []
        self._sync = True
        open_bucket: dict = {}
        for p in reversed(self.params):
            key = (p.dtype, p.device)
            b = open_bucket.get(key)
            if b is None or b["bytes"] >= bucket_bytes:
                b = {"params": [], "bytes": 0, "dtype": p.dtype, "device": p.device}
                open_bucket[key] = b
                self.buckets.append(b)
            b["params"].append(p)
            b["bytes"] += p.numel() * p.element_size()
        for index, b in enumerate(self.buckets):
            b["flat"] = torch.zeros(sum(p.numel() for p in b["params"]), dtype=b["dtype"], device=b["device"])
            offset = 0
            for p in b["params"]:
                p.grad = b["flat"][offset:offset + p.numel()].view_as(p)
                offset += p.numel()
                self._hooks.append(p.register_post_accumulate_grad_hook(self._make_hook(index)))
            b["arrived"], b["handle"] = 0, None

    def _make_hook(self, index: int):
        def hook(param):
            b = self.buckets[index]
            b["arrived"] += 1
            if b["arrived"] == len(b["params"]):
                self._launch(b)
        return hook

    def _launch(self, b: dict) -> None:
        if self.enabled and self._sync and b["handle"] is None:
            b["handle"] = dist.all_reduce(b["flat"], op=dist.ReduceOp.SUM, group=self.group, async_op=True)

    @torch.no_grad()
    def finish(self) -> int:
        """Call after backward: returns the number of collectives of this step."""
        issued = 0
        for b in self.buckets:
            if self.enabled and self._sync:
                self._launch(b)
                b["handle"].wait()
                b["flat"].div_(self.world)
                issued += 1
            b["arrived"], b["handle"] = 0, None
        return issued

    @torch.no_grad()
    def zero_grad(self) -> None:
        for b in self.buckets:
            b["flat"].zero_()
            offset = 0
            for p in b["params"]:
                if p.grad is None or p.grad.data_ptr() != b["flat"].data_ptr() + offset * b["flat"].element_size():
                    p.grad = b["flat"][offset:offset + p.numel()].view_as(p)
                offset += p.numel()

    @contextmanager
    def no_sync(self):
        """Gradient accumulation: backward passes inside add to the buckets without any collective."""
        previous, self._sync = self._sync, False
        try:
            yield
        finally:
            self._sync = previous

    def remove(self) -> None:
        for h in self._hooks:
            h.remove()
        self._hooks = []


def causal_lm_loss(model, input_ids: torch.Tensor, labels: torch.Tensor, *, total: int,
                   num_chunks: int = 8) -> torch.Tensor:
    """The model's shifted-label loss through the chunked fixed-denominator head (same value as
    ``model(input_ids, labels=labels).loss`` when ``total`` is the number of valid shifted labels)."""
    hidden = model.model(input_ids=input_ids, use_cache=False).last_hidden_state
    shifted = torch.cat((labels[..., 1:], torch.full_like(labels[:, :1], model.ignore_index)), dim=1)
    return fixed_dense_linear_cross_entropy(hidden, shifted, model.lm_head.weight, model.lm_head.bias,
                                            ignore_index=model.ignore_index, total=total, num_chunks=num_chunks)


class SolveDeltaGraphedTrainingStep:
    """Forward, loss and backward of the causal LM for ONE batch shape, captured as a CUDA graph.

    ``step(input_ids, labels)`` copies the batch into the static buffers, replays the graph and
    returns the loss (a static scalar: read it before the next replay).  When it returns, every
    parameter's ``.grad`` has this micro-batch ADDED to it (the captured backward accumulates in
    place), so gradient accumulation is repeated calls, and the optimizer, any clipping and the
    gradient all-reduce stay outside the graph, under the training loop's control, as upstream
    (cuda_graph.py:125-150).  With ``distributed=True`` the call ends with ``allreduce_gradients``
    over ``process_group`` unless made inside ``no_sync()``.

    Build it before any eager backward of the same model, or after every tensor that still holds such
    a backward's graph (a kept loss) has been freed: gradient accumulators created on another stream
    and kept alive by an old graph break the capture (upstream cuda_graph.py:133-137 captures before
    wrapping in DDP for the same reason).

    Limits, as upstream's: CUDA token ids and labels of one fixed shape, no masks, resets or cache,
    model in training mode, replay on the stream that built the helper; labels carry no ignored
    positions beyond the shift (the loss denominator is the constant B*(T-1))."""

    def __init__(self, model, sample_input_ids: torch.Tensor, sample_labels: torch.Tensor, *,
                 num_warmup_iters: int = 3, distributed: bool = False, process_group: Any = None,
                 num_chunks: int = 8) -> None:
        self._validate_pair(sample_input_ids, sample_labels)
        if not model.training:
            raise RuntimeError("the captured model must be in training mode")
        self.model = model
        self.device = sample_input_ids.device
        self.batch_size, self.sequence_length = sample_input_ids.shape
        if self.sequence_length < 2:
            raise ValueError("a training step needs at least two tokens per row")
        self.total = self.batch_size * (self.sequence_length - 1)
        self.num_chunks = num_chunks
        self.distributed = distributed
        self.process_group = process_group
        self._sync = True
        # opt-in: read the device fault word after every replay (costs a device synchronisation per step)
        self.check_faults = False
        self._input_dtype, self._label_dtype = sample_input_ids.dtype, sample_labels.dtype
        self._ids = sample_input_ids.clone()
        self._labels = sample_labels.clone()
        self._replay_stream = torch.cuda.current_stream(self.device)
        self.params = [p for p in model.parameters() if p.requires_grad]
        # gradients the caller already holds survive warm-up and capture untouched
        held = [None if p.grad is None else p.grad.clone() for p in self.params]
        side = torch.cuda.Stream(device=self.device)
        side.wait_stream(self._replay_stream)
        with torch.cuda.stream(side):
            for _ in range(max(1, num_warmup_iters)):   # lazy initialisation and allocator warm-up
                self._forward_backward()
        self._replay_stream.wait_stream(side)
        for p in self.params:                            # static gradient storage for the capture
            if p.grad is None:
                p.grad = torch.zeros_like(p)
        self.graph = torch.cuda.CUDAGraph()
        try:
            with torch.cuda.graph(self.graph):
                self.loss = self._forward_backward()
        except RuntimeError as error:
            raise RuntimeError(
                "capturing the training step failed.  The usual cause: an autograd graph from an earlier "
                "backward on another stream is still alive (a loss or output tensor that was kept), so the "
                "parameters' gradient accumulators still belong to that stream; free it (del loss) before "
                "building this helper") from error
        with torch.no_grad():
            for p, g in zip(self.params, held):
                if g is None:
                    p.grad.zero_()
                else:
                    p.grad.copy_(g)

    def _forward_backward(self) -> torch.Tensor:
        loss = causal_lm_loss(self.model, self._ids, self._labels, total=self.total, num_chunks=self.num_chunks)
        loss.backward()
        return loss.detach()

    @staticmethod
    def _validate_pair(input_ids: torch.Tensor, labels: torch.Tensor) -> None:
        if input_ids.ndim != 2 or labels.shape != input_ids.shape:
            raise ValueError("input_ids and labels must share one shape [B,T]")
        if input_ids.device.type != "cuda" or labels.device != input_ids.device:
            raise ValueError("input_ids and labels must live on one CUDA device")
        # as upstream (causallsso/cuda_graph.py:279-280): the loss gathers and scatters with the labels
        if input_ids.dtype != torch.long or labels.dtype != torch.long:
            raise TypeError("input_ids and labels must be torch.long tensors")

    def __call__(self, input_ids: torch.Tensor, labels: torch.Tensor) -> torch.Tensor:
        self._validate_pair(input_ids, labels)
        expected = (self.batch_size, self.sequence_length)
        if tuple(input_ids.shape) != expected:
            raise ValueError(f"this CUDA Graph requires input shape {expected}, got {tuple(input_ids.shape)}")
        if input_ids.dtype != self._input_dtype or labels.dtype != self._label_dtype:
            raise TypeError("input dtypes must match the captured sample dtypes")
        if input_ids.device != self.device:
            raise ValueError("input device must match the captured CUDA device")
        if torch.cuda.current_stream(self.device).cuda_stream != self._replay_stream.cuda_stream:
            raise RuntimeError("CUDA Graph replay must use the stream that constructed this helper")
        if not self.model.training:
            raise RuntimeError("the captured model must remain in training mode")
        self._ids.copy_(input_ids)
        self._labels.copy_(labels)
        self.graph.replay()
        if self.distributed and self._sync:
            allreduce_gradients(self.params, self.process_group)
        if self.check_faults:
            _lib.check_device_fault()   # waits for the device: a bounded wait inside a kernel that ran out raises here
        return self.loss

    step = __call__

    @contextmanager
    def no_sync(self):
        """Skip the gradient all-reduce for the replays inside (gradient accumulation)."""
        previous, self._sync = self._sync, False
        try:
            yield
        finally:
            self._sync = previous


__all__ = ["BF16ShadowWeights", "BucketedGradientAverager", "SolveDeltaGraphedTrainingStep", "allreduce_gradients",
           "causal_lm_loss",
           "fixed_dense_linear_cross_entropy", "fused_cross_entropy"]
