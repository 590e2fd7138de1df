"""Autograd wrappers of the mixer glue kernels (conv4 + SiLU, decay gate,
sigmoid-gated RMSNorm).  BF16 CUDA activations, FP32 parameters; arithmetic
is in the CUDA library (include/solvedelta_b200.h), there is no fallback.

Upstream counterparts: causallsso/model.py:110-164 (_packed_conv),
model.py:375-390 (decay gate), causallsso/ops/norm_gate.py:19-43,162-217.
"""
from __future__ import annotations

import ctypes
from typing import Optional, Tuple

import torch
import torch.nn.functional as F

from . import _lib


def _stream(device):
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def _scratch(nbytes, device):
    return torch.empty(max(int(nbytes), 16), dtype=torch.uint8, device=device)


def _require_bf16_cuda(name, t):
    if t.device.type != "cuda" or t.dtype != torch.bfloat16:
        raise TypeError(f"{name} must be a BF16 CUDA tensor")


class _Conv4Silu(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, initial_state, want_state, valid=None, reset=None, inplace=False):
        lib = _lib.load()
        B, T, D = x.shape
        w32 = weight.detach().float().contiguous()
        init = None if initial_state is None else initial_state.detach().to(torch.bfloat16).contiguous()
        with torch.cuda.device(x.device):
            y = torch.empty(B, T, D, dtype=torch.bfloat16, device=x.device)
            # in place: a thread reads the three state entries of its channels before it writes them (one tile)
            fin = (init if inplace else torch.empty(B, D, 3, dtype=torch.bfloat16, device=x.device)) if want_state else None
            a = _lib.Conv4ForwardArgs(B, T, D, x.data_ptr(), x.stride(0), x.stride(1), w32.data_ptr(),
                                      None if init is None else init.data_ptr(), y.data_ptr(),
                                      None if fin is None else fin.data_ptr(),
                                      None if valid is None else valid.data_ptr(),
                                      None if reset is None else reset.data_ptr())
            _lib.check(lib.sd_conv4_silu_forward(ctypes.byref(a), _stream(x.device)))
        ctx.save_for_backward(x, w32, init if init is not None else x.new_empty(0))
        ctx.masks = (valid, reset)
        ctx.has_init = init is not None
        ctx.weight_dtype = weight.dtype
        ctx.set_materialize_grads(False)
        if fin is not None:
            ctx.mark_non_differentiable(fin)
        return y, fin

    @staticmethod
    def backward(ctx, dy, _dfin):
        lib = _lib.load()
        x, w32, init = ctx.saved_tensors
        B, T, D = x.shape
        if dy is None:
            return (torch.zeros_like(x), torch.zeros(D, 4, dtype=ctx.weight_dtype, device=x.device), None, None,
                    None, None, None)
        dy = dy.to(torch.bfloat16).contiguous()
        valid, reset = ctx.masks
        with torch.cuda.device(x.device):
            dx = torch.empty(B, T, D, dtype=torch.bfloat16, device=x.device)
            dw = torch.empty(D, 4, dtype=torch.float32, device=x.device)
            dinit = torch.empty(B, D, 3, dtype=torch.bfloat16, device=x.device) if ctx.has_init else None
            scratch = _scratch(lib.sd_conv4_backward_scratch_bytes(B, T, D), x.device)
            a = _lib.Conv4BackwardArgs(B, T, D, x.data_ptr(), x.stride(0), x.stride(1), w32.data_ptr(),
                                       init.data_ptr() if ctx.has_init else None, dy.data_ptr(), dx.data_ptr(),
                                       dw.data_ptr(), None if dinit is None else dinit.data_ptr(),
                                       scratch.data_ptr(), scratch.numel(),
                                       None if valid is None else valid.data_ptr(),
                                       None if reset is None else reset.data_ptr())
            _lib.check(lib.sd_conv4_silu_backward(ctypes.byref(a), _stream(x.device)))
        return dx, dw.to(ctx.weight_dtype), dinit, None, None, None, None


def _conv_mask(name: str, mask: Optional[torch.Tensor], x: torch.Tensor) -> Optional[torch.Tensor]:
    """bool [B,T] on the activation device -> its bytes as uint8 (no copy when contiguous)."""
    if mask is None:
        return None
    if mask.dtype != torch.bool or mask.shape != x.shape[:2]:
        raise ValueError(f"{name} must be bool [B,T]")
    if mask.device != x.device:
        raise ValueError("masks must share the activation device")
    return mask.contiguous().view(torch.uint8)


def conv4_silu(x: torch.Tensor, weight: torch.Tensor, initial_state: Optional[torch.Tensor] = None,
               return_final_state: bool = False, valid_mask: Optional[torch.Tensor] = None,
               reset_mask: Optional[torch.Tensor] = None, _inplace_state: bool = False
               ) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    """Depthwise causal conv (4 taps, tap 3 = current token) + SiLU over [B,T,D] BF16 rows
    (any batch/token strides, unit channel stride) with a carried [B,D,3] state.

    With masks (bool [B,T]) it is the masked token loop of causallsso/model.py:146-164, run inside
    the kernel on the padded batch: an invalid token gives zero output and leaves the state
    untouched, a reset on a valid token starts from the zero state, and the returned state of a
    row holds its last three valid inputs since the last reset (older slots show the carried state
    or zeros through).  No repacking and no host synchronisation (upstream's CUDA branch gathers
    segments around causal_conv1d instead, model.py:166-273)."""
    _require_bf16_cuda("x", x)
    if x.ndim != 3 or x.stride(-1) != 1:
        raise ValueError("x must be [B,T,D] with unit channel stride")
    if weight.shape != (x.shape[-1], 4):
        raise ValueError("conv weight must have shape [D,4]")
    if initial_state is not None and initial_state.shape != (x.shape[0], x.shape[2], 3):
        raise ValueError("conv initial state must have shape [B,D,3]")
    valid, reset = _conv_mask("valid_mask", valid_mask, x), _conv_mask("reset_mask", reset_mask, x)
    if x.shape[1] == 0:
        fin = None
        if return_final_state:
            fin = (initial_state.to(torch.bfloat16) if initial_state is not None
                   else x.new_zeros(x.shape[0], x.shape[2], 3))
        return x.new_zeros(x.shape), fin
    # a cache that owns its state may have a single-token no-grad step update it in place
    inplace = (_inplace_state and return_final_state and initial_state is not None and x.shape[1] == 1
               and not torch.is_grad_enabled() and valid is None and reset is None
               and initial_state.dtype == torch.bfloat16 and initial_state.is_contiguous())
    return _Conv4Silu.apply(x, weight, initial_state, return_final_state, valid, reset, inplace)


def conv4_silu_segmented(x: torch.Tensor, weight: torch.Tensor, plan, initial_state: Optional[torch.Tensor] = None,
                         return_final_state: bool = False) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    """``conv4_silu`` with the masks of a segment plan from ``build_packed_segments`` (the plan is only
    checked against the input; the kernel works on the padded batch in place)."""
    if (plan.batch, plan.length) != tuple(x.shape[:2]):
        raise ValueError("packed segment plan does not match the conv input")
    return conv4_silu(x, weight, initial_state, return_final_state, plan.valid_mask, plan.reset_mask)


@torch.no_grad()
def mixer_decode_step(u: torch.Tensor, h: torch.Tensor, erase_raw: torch.Tensor, write_raw: torch.Tensor,
                      qkv: torch.Tensor, conv_weight: torch.Tensor, conv_state: torch.Tensor,
                      decay_raw: torch.Tensor, log_rate: torch.Tensor, decay_bias: torch.Tensor,
                      geometry_raw: torch.Tensor, geometry_bias: torch.Tensor,
                      predictor: torch.Tensor, memory: torch.Tensor, *, output_gate: Optional[torch.Tensor] = None,
                      norm_weight: Optional[torch.Tensor] = None, norm_eps: float = 1e-6,
                      gate_projections: Optional[tuple] = None) -> torch.Tensor:
    """One cached token of the mixer between its projections, in ONE launch: conv4 + SiLU of the q | k | v slice
    against ``conv_state`` (advanced in place), the decay gate, the geometry rate and the recurrent step on
    ``predictor`` / ``memory`` (updated in place).  ``u, h`` are ``[B,1,H,r]`` and ``erase_raw, write_raw``
    ``[B,1,H,r|V]`` views of the projection row, ``qkv`` ``[B,1,D]``, ``decay_raw`` ``[B,1,H,r]``, ``geometry_raw``
    ``[B,1,H]``; FP32 ``conv_weight [D,4]``, ``log_rate [H]``, ``decay_bias [H*r]``, ``geometry_bias [H]``.
    Returns the output row ``[B,1,H,V]`` (BF16).  Same arithmetic as ``conv4_silu`` + ``kda_decay_gate`` +
    ``sigmoid`` + the T = 1 branch of ``solvedelta_native``; with ``output_gate`` ``[B,1,H,V]`` and FP32
    ``norm_weight [V]`` the row also passes through ``rms_norm_gated``.  ``gate_projections`` =
    ``(decay_hidden [B,1,G], decay_proj.weight [H*r,G], gate_hidden [B,1,G], output_gate_proj.weight [H*V,G],
    output_gate_proj.bias [H*V] | None)``, all BF16, moves the two small projections in front of the gates into the
    kernel as well (``decay_raw`` and ``output_gate`` may then be None; needs ``norm_weight``)."""
    lib = _lib.load()
    B, T, H, r = u.shape
    V = write_raw.shape[-1]
    if T != 1:
        raise ValueError("mixer_decode_step takes exactly one token")
    for name, t in (("u", u), ("h", h), ("erase_raw", erase_raw), ("write_raw", write_raw), ("qkv", qkv),
                    ("geometry_raw", geometry_raw), ("conv_state", conv_state)):
        _require_bf16_cuda(name, t)
    if gate_projections is None:
        _require_bf16_cuda("decay_raw", decay_raw)
    for name, t in (("conv_weight", conv_weight), ("log_rate", log_rate), ("decay_bias", decay_bias),
                    ("geometry_bias", geometry_bias), ("predictor", predictor), ("memory", memory)):
        if t.dtype != torch.float32 or not t.is_contiguous():
            raise TypeError(f"{name} must be contiguous FP32")
    D = 2 * H * r + H * V
    if qkv.shape != (B, 1, D) or conv_state.shape != (B, D, 3) or not conv_state.is_contiguous():
        raise ValueError("qkv must be [B,1,D] and conv_state contiguous [B,D,3] with D = 2*H*r + H*V")
    if qkv.stride(-1) != 1 or geometry_raw.stride(-1) != 1 or (decay_raw is not None and decay_raw.stride(-1) != 1):
        raise ValueError("row operands require unit innermost stride")

    def operand(t):
        return _lib.Operand(t.data_ptr(), t.stride(0), t.stride(1), t.stride(2))

    with torch.cuda.device(u.device):
        y = torch.empty(B, 1, H, V, dtype=torch.bfloat16, device=u.device)
        a = _lib.MixerDecodeArgs()
        a.shape = _lib.Shape(B, 1, H, r, V)
        a.u, a.h = operand(u), operand(h)
        a.erase_raw, a.write_raw = operand(erase_raw), operand(write_raw)
        a.qkv, a.qkv_stride_b = qkv.data_ptr(), qkv.stride(0)
        a.conv_weight, a.conv_state = conv_weight.data_ptr(), conv_state.data_ptr()
        if decay_raw is not None:
            decay2 = decay_raw.reshape(B, H * r) if decay_raw.is_contiguous() else decay_raw.contiguous().view(B, H * r)
            a.decay_raw, a.decay_stride_b = decay2.data_ptr(), decay2.stride(0)
        a.log_rate, a.decay_bias = log_rate.data_ptr(), decay_bias.data_ptr()
        a.geometry_raw, a.geometry_stride_b = geometry_raw.data_ptr(), geometry_raw.stride(0)
        a.geometry_bias = geometry_bias.data_ptr()
        a.C, a.S, a.y = predictor.data_ptr(), memory.data_ptr(), y.data_ptr()
        if gate_projections is not None:
            decay_hidden, decay_w, gate_hidden, gate_w, gate_b = gate_projections
            G = decay_hidden.shape[-1]
            for name, t in (("decay_hidden", decay_hidden), ("decay_proj.weight", decay_w),
                            ("gate_hidden", gate_hidden), ("output_gate_proj.weight", gate_w)):
                _require_bf16_cuda(name, t)
            if (decay_w.shape != (H * r, G) or gate_w.shape != (H * V, G) or not decay_w.is_contiguous()
                    or not gate_w.is_contiguous() or G % 8 or G > 128 or norm_weight is None):
                raise ValueError("fused gate projections: weights [H*r,G] / [H*V,G] contiguous, G a multiple of 8, "
                                 "at most 128, and the fused norm")
            a.gate_rank = G
            a.decay_hidden, a.decay_hidden_stride_b = decay_hidden.data_ptr(), decay_hidden.stride(0)
            a.gate_hidden, a.gate_hidden_stride_b = gate_hidden.data_ptr(), gate_hidden.stride(0)
            a.decay_proj_weight, a.gate_proj_weight = decay_w.data_ptr(), gate_w.data_ptr()
            a.gate_proj_bias = None if gate_b is None else gate_b.data_ptr()
        if norm_weight is not None:
            if gate_projections is None and (output_gate is None or output_gate.dtype != torch.bfloat16
                                             or not output_gate.is_contiguous()):
                raise ValueError("the fused norm needs a contiguous BF16 output_gate [B,1,H,V]")
            if norm_weight.dtype != torch.float32 or norm_weight.shape != (V,):
                raise TypeError("norm_weight must be FP32 [V]")
            a.norm_weight, a.norm_eps = norm_weight.data_ptr(), float(norm_eps)
            if output_gate is not None:
                a.output_gate, a.output_gate_stride_b = output_gate.data_ptr(), H * V
        _lib.check(lib.sd_mixer_decode_step(ctypes.byref(a), _stream(u.device)))
    return y


@torch.no_grad()
def add_rmsnorm_reverse_supported(width: int) -> bool:
    """Row widths the reverse pass of :func:`add_rmsnorm` is built for (whole groups of 256 channels, up to 2048)."""
    return width % 256 == 0 and 0 < width <= 2048


def _add_rmsnorm_forward(xc, dc, w, eps):
    lib = _lib.load()
    D = xc.shape[-1]
    with torch.cuda.device(xc.device):
        normed = torch.empty_like(xc)
        total = torch.empty_like(xc) if dc is not None else xc
        a = _lib.AddRmsnormArgs(xc.numel() // D, D, float(eps), xc.data_ptr(), dc.data_ptr() if dc is not None else None,
                                w.data_ptr(), total.data_ptr() if dc is not None else None, normed.data_ptr())
        _lib.check(lib.sd_add_rmsnorm(ctypes.byref(a), _stream(xc.device)))
    return total, normed


class _AddRmsNorm(torch.autograd.Function):
    """``(x + delta, RMSNorm(x + delta) * weight)`` with one reverse kernel: the cotangents of both outputs become
    the single gradient that ``x`` and ``delta`` share, plus the weight gradient.  Only the sum is saved."""

    @staticmethod
    def forward(ctx, x, delta, weight, eps):
        xc = x.contiguous()
        dc = delta.contiguous() if delta is not None else None
        w = weight.detach().float().contiguous()
        total, normed = _add_rmsnorm_forward(xc, dc, w, eps)
        ctx.save_for_backward(total, w)
        ctx.eps, ctx.has_delta, ctx.weight_dtype = float(eps), delta is not None, weight.dtype
        ctx.set_materialize_grads(False)
        if delta is None:   # the sum is x itself: the caller keeps using x, this output is a placeholder
            total = xc.new_empty(0)
            ctx.mark_non_differentiable(total)
        return total, normed

    @staticmethod
    def backward(ctx, dtotal, dnormed):
        lib = _lib.load()
        total, w = ctx.saved_tensors
        if dnormed is None:
            return dtotal, (dtotal if ctx.has_delta else None), None, None
        D = total.shape[-1]
        rows = total.numel() // D
        dn = dnormed.to(torch.bfloat16).contiguous()
        dt = dtotal.to(torch.bfloat16).contiguous() if dtotal is not None else None
        with torch.cuda.device(total.device):
            dx = torch.empty_like(total)
            dw = torch.empty(D, dtype=torch.float32, device=total.device)
            scratch = _scratch(lib.sd_add_rmsnorm_backward_scratch_bytes(rows, D), total.device)
            a = _lib.AddRmsnormBackwardArgs(rows, D, ctx.eps, total.data_ptr(), w.data_ptr(),
                                            dt.data_ptr() if dt is not None else None, dn.data_ptr(), dx.data_ptr(),
                                            dw.data_ptr(), scratch.data_ptr(), scratch.numel())
            _lib.check(lib.sd_add_rmsnorm_backward(ctypes.byref(a), _stream(total.device)))
        return dx, (dx if ctx.has_delta else None), dw.to(ctx.weight_dtype), None


def add_rmsnorm(x: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, eps: float):
    """``s = x + delta`` and ``RMSNorm(s) * weight`` in one pass: returns ``(s, normed)``, both BF16 with the shape
    of ``x`` (``delta=None``: the norm alone, ``s`` is ``x``).  ``weight`` ``[D]``, FP32 without autograd; with
    autograd any floating dtype, and ``D`` must satisfy :func:`add_rmsnorm_reverse_supported`."""
    _require_bf16_cuda("x", x)
    if delta is not None:
        _require_bf16_cuda("delta", delta)
        if x.shape != delta.shape:
            raise ValueError("x and delta must share a shape [...,D]")
    if weight.shape != (x.shape[-1],):
        raise ValueError("weight must be [D]")
    needs_grad = torch.is_grad_enabled() and (x.requires_grad or weight.requires_grad
                                              or (delta is not None and delta.requires_grad))
    if needs_grad:
        if not add_rmsnorm_reverse_supported(x.shape[-1]):
            raise ValueError("the reverse pass takes rows of 256, 512, ..., 2048 channels")
        total, normed = _AddRmsNorm.apply(x, delta, weight, eps)
        return (x if delta is None else total), normed
    if weight.dtype != torch.float32:
        raise ValueError("weight must be FP32 [D]")
    if delta is None and not add_rmsnorm_reverse_supported(x.shape[-1]):
        raise ValueError("the norm alone takes rows of 256, 512, ..., 2048 channels")
    return _add_rmsnorm_forward(x.contiguous(), delta.contiguous() if delta is not None else None,
                                weight.detach().contiguous(), eps)


class _Swiglu(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gate_value):
        gv = gate_value.contiguous()
        ctx.save_for_backward(gv)
        return _swiglu_forward(gv)

    @staticmethod
    def backward(ctx, dout):
        lib = _lib.load()
        (gv,) = ctx.saved_tensors
        width = gv.shape[-1] // 2
        do = dout.to(torch.bfloat16).contiguous()
        with torch.cuda.device(gv.device):
            dgv = torch.empty_like(gv)
            a = _lib.SwigluArgs(gv.numel() // (2 * width), width, gv.data_ptr(), None, do.data_ptr(), dgv.data_ptr())
            _lib.check(lib.sd_swiglu_backward(ctypes.byref(a), _stream(gv.device)))
        return dgv


def _swiglu_forward(gv):
    lib = _lib.load()
    width = gv.shape[-1] // 2
    with torch.cuda.device(gv.device):
        out = torch.empty(*gv.shape[:-1], width, dtype=torch.bfloat16, device=gv.device)
        a = _lib.SwigluArgs(gv.numel() // (2 * width), width, gv.data_ptr(), out.data_ptr(), None, None)
        _lib.check(lib.sd_swiglu(ctypes.byref(a), _stream(gv.device)))
    return out


def swiglu(gate_value: torch.Tensor) -> torch.Tensor:
    """``silu(gate) * value`` for rows ``[gate | value]``: ``[..., 2 I]`` -> ``[..., I]`` BF16, with a reverse pass
    that writes the gradient row ``[d gate | d value]`` in one kernel."""
    _require_bf16_cuda("gate_value", gate_value)
    if gate_value.shape[-1] % 2:
        raise ValueError("the last axis must hold gate and value halves")
    if torch.is_grad_enabled() and gate_value.requires_grad:
        return _Swiglu.apply(gate_value)
    return _swiglu_forward(gate_value.contiguous())


def small_linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None, *,
                 swiglu: bool = False) -> Optional[torch.Tensor]:
    """``F.linear(x, weight, bias)`` for the one to four rows of a cached single-token step (inference only), one warp
    per output column; with ``swiglu`` the result is ``silu(y[..., :N/2]) * y[..., N/2:]``.  Returns ``None`` when the
    call is not one the kernel takes (gradients recorded, more rows, not BF16 CUDA, unaligned), and the caller runs
    its library projection."""
    if torch.is_grad_enabled() and (x.requires_grad or weight.requires_grad):
        return None
    K = x.shape[-1]
    if (x.device.type != "cuda" or x.dtype != torch.bfloat16 or weight.dtype != torch.bfloat16 or weight.ndim != 2
            or weight.shape[1] != K or not weight.is_contiguous() or weight.device != x.device or K % 8
            or (bias is not None and (bias.dtype != torch.bfloat16 or not bias.is_contiguous()))):
        return None
    rows = x.numel() // K
    if rows < 1 or rows > _lib.GEMV_MAX_ROWS or x.stride(-1) != 1:
        return None
    x2 = x.reshape(rows, K)   # a view for the layouts a decode step produces; a copy of a few KB otherwise
    stride = x2.stride(0) if rows > 1 else K
    N = weight.shape[0]
    if stride % 8 or x2.data_ptr() % 16 or weight.data_ptr() % 16 or (swiglu and N % 2):
        return None
    lib = _lib.load()
    width = N // 2 if swiglu else N
    with torch.cuda.device(x.device):
        out = torch.empty(*x.shape[:-1], width, dtype=torch.bfloat16, device=x.device)
        a = _lib.GemvArgs(rows, N, K, 1 if swiglu else 0, x2.data_ptr(), stride, weight.data_ptr(),
                          bias.data_ptr() if bias is not None else None, out.data_ptr(), width)
        _lib.check(lib.sd_gemv(ctypes.byref(a), _stream(x.device)))
    return out


def pack_rows(pieces, widths, row_shape, device) -> Optional[torch.Tensor]:
    """One BF16 row-shaped tensor ``[..., P]`` holding ``pieces`` side by side (``None``: zeros; columns past the
    last piece: zeros), written by one kernel; ``None`` when the layout is not one the kernel takes (widths in whole
    groups of eight channels, at most twelve pieces, BF16 CUDA) and the caller has to assemble the row itself."""
    P = row_shape[-1]
    if (device.type != "cuda" or len(widths) > _lib.PACK_MAX_PIECES or P % 8 or any(w % 8 for w in widths)
            or any(g is not None and g.dtype != torch.bfloat16 for g in pieces)):
        return None
    lib = _lib.load()
    held = [g.contiguous() if g is not None else None for g in pieces]
    with torch.cuda.device(device):
        out = torch.empty(row_shape, dtype=torch.bfloat16, device=device)
        a = _lib.PackRowsArgs()
        a.rows, a.pieces, a.row_width, a.dst = out.numel() // P, len(widths), P, out.data_ptr()
        for k, (g, w) in enumerate(zip(held, widths)):
            a.piece[k].src = g.data_ptr() if g is not None else None
            a.piece[k].width = w
        _lib.check(lib.sd_pack_rows(ctypes.byref(a), _stream(device)))
    return out


class _KdaGate(torch.autograd.Function):
    @staticmethod
    def forward(ctx, raw, log_rate, bias):
        lib = _lib.load()
        H, r = raw.shape[-2], raw.shape[-1]
        rows = raw.numel() // (H * r)
        rawc = raw.contiguous()
        A = log_rate.detach().float().contiguous()
        b = bias.detach().float().reshape(H, r).contiguous()
        with torch.cuda.device(raw.device):
            out = torch.empty(raw.shape, dtype=torch.float32, device=raw.device)
            a = _lib.KdaGateArgs(rows, H, r, rawc.data_ptr(), A.data_ptr(), b.data_ptr(), out.data_ptr())
            _lib.check(lib.sd_kda_gate_forward(ctypes.byref(a), _stream(raw.device)))
        ctx.save_for_backward(rawc, A, b)
        ctx.param_shapes = (log_rate.shape, bias.shape, log_rate.dtype, bias.dtype)
        return out

    @staticmethod
    def backward(ctx, dout):
        lib = _lib.load()
        rawc, A, b = ctx.saved_tensors
        H, r = b.shape
        rows = rawc.numel() // (H * r)
        dout = dout.float().contiguous()
        with torch.cuda.device(rawc.device):
            draw = torch.empty_like(rawc)
            dA = torch.empty(H, dtype=torch.float32, device=rawc.device)
            db = torch.empty(H, r, dtype=torch.float32, device=rawc.device)
            scratch = _scratch(lib.sd_kda_gate_backward_scratch_bytes(rows, H, r), rawc.device)
            a = _lib.KdaGateArgs(rows, H, r, rawc.data_ptr(), A.data_ptr(), b.data_ptr(), None, dout.data_ptr(),
                                 draw.data_ptr(), dA.data_ptr(), db.data_ptr(), scratch.data_ptr(), scratch.numel())
            _lib.check(lib.sd_kda_gate_backward(ctypes.byref(a), _stream(rawc.device)))
        sa, sb, da, dbt = ctx.param_shapes
        return draw, dA.reshape(sa).to(da), db.reshape(sb).to(dbt)


def kda_decay_gate(raw: torch.Tensor, log_rate: torch.Tensor, bias: torch.Tensor) -> torch.Tensor:
    """log_decay = -exp(log_rate[h]) * softplus(raw + bias[h,c]); raw BF16 [...,H,r] -> FP32."""
    _require_bf16_cuda("raw", raw)
    H, r = raw.shape[-2], raw.shape[-1]
    if log_rate.numel() != H or bias.numel() != H * r:
        raise ValueError("log_rate must have H entries and bias H*r entries")
    return _KdaGate.apply(raw, log_rate, bias)


class _NormGate(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, gate, weight, eps):
        lib = _lib.load()
        V = x.shape[-1]
        rows = x.numel() // V
        xc, gc = x.contiguous(), gate.contiguous()
        w = weight.detach().float().contiguous()
        with torch.cuda.device(x.device):
            y = torch.empty(x.shape, dtype=torch.bfloat16, device=x.device)
            a = _lib.NormGateArgs(rows, V, float(eps), xc.data_ptr(), gc.data_ptr(), w.data_ptr(), y.data_ptr())
            _lib.check(lib.sd_norm_gate_forward(ctypes.byref(a), _stream(x.device)))
        ctx.save_for_backward(xc, gc, w)
        ctx.eps = float(eps)
        ctx.weight_dtype = weight.dtype
        return y

    @staticmethod
    def backward(ctx, dy):
        lib = _lib.load()
        xc, gc, w = ctx.saved_tensors
        V = xc.shape[-1]
        rows = xc.numel() // V
        dy = dy.to(torch.bfloat16).contiguous()
        with torch.cuda.device(xc.device):
            dx, dg = torch.empty_like(xc), torch.empty_like(gc)
            dw = torch.empty(V, dtype=torch.float32, device=xc.device)
            scratch = _scratch(lib.sd_norm_gate_backward_scratch_bytes(rows, V), xc.device)
            a = _lib.NormGateArgs(rows, V, ctx.eps, xc.data_ptr(), gc.data_ptr(), w.data_ptr(), None, dy.data_ptr(),
                                  dx.data_ptr(), dg.data_ptr(), dw.data_ptr(), scratch.data_ptr(), scratch.numel())
            _lib.check(lib.sd_norm_gate_backward(ctypes.byref(a), _stream(xc.device)))
        return dx, dg, dw.to(ctx.weight_dtype), None


def _norm_gate_forward(xc, gc, w, eps):
    lib = _lib.load()
    V = xc.shape[-1]
    with torch.cuda.device(xc.device):
        y = torch.empty(xc.shape, dtype=torch.bfloat16, device=xc.device)
        a = _lib.NormGateArgs(xc.numel() // V, V, float(eps), xc.data_ptr(), gc.data_ptr(), w.data_ptr(), y.data_ptr())
        _lib.check(lib.sd_norm_gate_forward(ctypes.byref(a), _stream(xc.device)))
    return y


class _NormGateLinear(torch.autograd.Function):
    """Gated RMSNorm followed by a Linear over the flattened [H*D] rows, without keeping the normalised
    panel for the reverse pass: it is produced again from x and gate there (one more pass of the norm
    kernel instead of a saved [..., H*D] BF16 tensor per layer).  causallsso/ops/norm_gate.py:46-159."""

    @staticmethod
    def forward(ctx, x, gate, norm_weight, linear_weight, linear_bias, eps):
        xc, gc = x.contiguous(), gate.contiguous()
        w = norm_weight.detach().float().contiguous()
        y = _norm_gate_forward(xc, gc, w, eps)
        packed_weight = linear_weight.detach().to(torch.bfloat16)
        packed_bias = None if linear_bias is None else linear_bias.detach().to(torch.bfloat16)
        out = F.linear(y.reshape(*x.shape[:-2], -1), packed_weight, packed_bias)
        ctx.save_for_backward(xc, gc, w, packed_weight)
        ctx.eps = float(eps)
        ctx.dtypes = (norm_weight.dtype, linear_weight.dtype, None if linear_bias is None else linear_bias.dtype)
        ctx.set_materialize_grads(False)
        return out

    @staticmethod
    def backward(ctx, dout):
        if dout is None:
            return (None,) * 6
        lib = _lib.load()
        xc, gc, w, packed_weight = ctx.saved_tensors
        V = xc.shape[-1]
        rows = xc.numel() // V
        dout2 = dout.to(torch.bfloat16).reshape(-1, dout.shape[-1])
        y = _norm_gate_forward(xc, gc, w, ctx.eps)           # regenerated, not saved
        dlinear = torch.mm(dout2.t(), y.reshape(dout2.shape[0], -1))
        dy = torch.mm(dout2, packed_weight).reshape(xc.shape).contiguous()
        del y
        with torch.cuda.device(xc.device):
            dx, dg = torch.empty_like(xc), torch.empty_like(gc)
            dw = torch.empty(V, dtype=torch.float32, device=xc.device)
            scratch = _scratch(lib.sd_norm_gate_backward_scratch_bytes(rows, V), xc.device)
            a = _lib.NormGateArgs(rows, V, ctx.eps, xc.data_ptr(), gc.data_ptr(), w.data_ptr(), None, dy.data_ptr(),
                                  dx.data_ptr(), dg.data_ptr(), dw.data_ptr(), scratch.data_ptr(), scratch.numel())
            _lib.check(lib.sd_norm_gate_backward(ctypes.byref(a), _stream(xc.device)))
        norm_dtype, weight_dtype, bias_dtype = ctx.dtypes
        dbias = None if bias_dtype is None else dout2.float().sum(dim=0).to(bias_dtype)
        return dx, dg, dw.to(norm_dtype), dlinear.to(weight_dtype), dbias, None


def rms_norm_gated_linear(x: torch.Tensor, gate: torch.Tensor, norm_weight: torch.Tensor, linear_weight: torch.Tensor,
                          linear_bias: Optional[torch.Tensor], eps: float) -> torch.Tensor:
    """``F.linear(rms_norm_gated(x, gate, norm_weight, eps).flatten(-2), linear_weight, linear_bias)`` in BF16,
    with the normalised panel recomputed in the reverse pass (upstream ``RMSNormGated.forward_linear``)."""
    _require_bf16_cuda("x", x)
    _require_bf16_cuda("gate", gate)
    if x.shape != gate.shape or x.ndim < 2:
        raise ValueError("x and gate must have the same [...,H,D] shape")
    if norm_weight.shape != (x.shape[-1],):
        raise ValueError("weight must have shape [D]")
    if linear_weight.ndim != 2 or linear_weight.shape[1] != x.shape[-2] * x.shape[-1]:
        raise ValueError("the linear layer must take the flattened [H*D] rows")
    return _NormGateLinear.apply(x, gate, norm_weight, linear_weight, linear_bias, eps)


def rms_norm_gated(x: torch.Tensor, gate: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """y = x * rsqrt(mean(x^2) + eps) * weight * sigmoid(gate) over the last axis (<= 128)."""
    _require_bf16_cuda("x", x)
    _require_bf16_cuda("gate", gate)
    if x.shape != gate.shape or x.ndim < 2:
        raise ValueError("x and gate must have the same [...,H,D] shape")
    if weight.shape != (x.shape[-1],):
        raise ValueError("weight must have shape [D]")
    return _NormGate.apply(x, gate, weight, eps)


__all__ = ["add_rmsnorm", "conv4_silu", "conv4_silu_segmented", "kda_decay_gate", "mixer_decode_step", "rms_norm_gated",
           "swiglu",
           "rms_norm_gated_linear"]
