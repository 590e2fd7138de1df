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
    def forward(ctx, x, weight, initial_state, want_state):
        lib = _lib.load()
        B, T, D = x.shape
        w32 = weight.detach().float().contiguous()
        init = None if initial_state is None else initial_state.detach().to(torch.bfloat16).contiguous()
        with torch.cuda.device(x.device):
            y = torch.empty(B, T, D, dtype=torch.bfloat16, device=x.device)
            fin = torch.empty(B, D, 3, dtype=torch.bfloat16, device=x.device) if want_state else None
            a = _lib.Conv4ForwardArgs(B, T, D, x.data_ptr(), x.stride(0), x.stride(1), w32.data_ptr(),
                                      None if init is None else init.data_ptr(), y.data_ptr(),
                                      None if fin is None else fin.data_ptr())
            _lib.check(lib.sd_conv4_silu_forward(ctypes.byref(a), _stream(x.device)))
        ctx.save_for_backward(x, w32, init if init is not None else x.new_empty(0))
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
            return torch.zeros_like(x), torch.zeros(D, 4, dtype=ctx.weight_dtype, device=x.device), None, None
        dy = dy.to(torch.bfloat16).contiguous()
        with torch.cuda.device(x.device):
            dx = torch.empty(B, T, D, dtype=torch.bfloat16, device=x.device)
            dw = torch.empty(D, 4, dtype=torch.float32, device=x.device)
            dinit = torch.empty(B, D, 3, dtype=torch.bfloat16, device=x.device) if ctx.has_init else None
            scratch = _scratch(lib.sd_conv4_backward_scratch_bytes(B, T, D), x.device)
            a = _lib.Conv4BackwardArgs(B, T, D, x.data_ptr(), x.stride(0), x.stride(1), w32.data_ptr(),
                                       init.data_ptr() if ctx.has_init else None, dy.data_ptr(), dx.data_ptr(),
                                       dw.data_ptr(), None if dinit is None else dinit.data_ptr(),
                                       scratch.data_ptr(), scratch.numel())
            _lib.check(lib.sd_conv4_silu_backward(ctypes.byref(a), _stream(x.device)))
        return dx, dw.to(ctx.weight_dtype), dinit, None


def conv4_silu(x: torch.Tensor, weight: torch.Tensor, initial_state: Optional[torch.Tensor] = None,
               return_final_state: bool = False) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    """Depthwise causal conv (4 taps, tap 3 = current token) + SiLU over [B,T,D] BF16 rows
    (any batch/token strides, unit channel stride) with a carried [B,D,3] state."""
    _require_bf16_cuda("x", x)
    if x.ndim != 3 or x.stride(-1) != 1:
        raise ValueError("x must be [B,T,D] with unit channel stride")
    if weight.shape != (x.shape[-1], 4):
        raise ValueError("conv weight must have shape [D,4]")
    if initial_state is not None and initial_state.shape != (x.shape[0], x.shape[2], 3):
        raise ValueError("conv initial state must have shape [B,D,3]")
    return _Conv4Silu.apply(x, weight, initial_state, return_final_state)


def conv4_silu_segmented(x: torch.Tensor, weight: torch.Tensor, plan, initial_state: Optional[torch.Tensor] = None,
                         return_final_state: bool = False) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    """Masked / reset batches: the conv of causallsso/model.py:146-164 with masks, run as one batch
    of reset-free segments (plan from ``build_packed_segments``).  Invalid tokens give zero output and
    leave the state untouched, a reset token starts from the zero state, the first segment of a batch
    row continues ``initial_state`` unless it opens with a reset; the returned state of a row holds its
    last three valid inputs since the last reset (older slots show the carried state or zeros through).
    Host-side index plumbing around ``conv4_silu`` (upstream does the same around causal_conv1d,
    model.py:166-273)."""
    from .packing import pack_tokens, unpack_tokens

    _require_bf16_cuda("x", x)
    batch, length, channels = x.shape
    if (plan.batch, plan.length) != (batch, length):
        raise ValueError("packed segment plan does not match the conv input")
    if initial_state is not None and initial_state.shape != (batch, channels, 3):
        raise ValueError("conv initial state must have shape [B,D,3]")
    if plan.num_tokens == 0:
        output = x.new_zeros(batch, length, channels)
        if not return_final_state:
            return output, None
        return output, (initial_state if initial_state is not None else x.new_zeros(batch, channels, 3))
    padded = plan.max_seqlen
    position = torch.arange(plan.num_tokens, dtype=torch.long, device=x.device) - plan.cu_seqlens[plan.segment_ids]
    destination = plan.segment_ids * padded + position
    tokens = pack_tokens(x, plan).squeeze(0)
    rows = tokens.new_zeros(plan.num_segments * padded, channels).index_copy(0, destination, tokens)
    rows = rows.view(plan.num_segments, padded, channels)
    segment_initial = None
    if initial_state is not None:
        carried = initial_state.to(torch.bfloat16).index_select(0, plan.segment_batch)
        segment_initial = torch.where(plan.use_initial[:, None, None], carried, torch.zeros_like(carried))
    segment_out, _ = conv4_silu(rows, weight, segment_initial, False)
    flat = segment_out.reshape(plan.num_segments * padded, channels)
    output = unpack_tokens(flat.index_select(0, destination).unsqueeze(0), plan)
    if not return_final_state:
        return output, None
    with torch.no_grad():
        # state of a segment = the three inputs before position len in [carried state | segment tokens]
        start = segment_initial if segment_initial is not None else rows.new_zeros(plan.num_segments, channels, 3)
        extended = torch.cat((start.transpose(1, 2), rows.detach()), dim=1)            # [S, 3 + padded, D]
        take = plan.segment_lengths.long()[:, None] + torch.arange(3, device=x.device)[None, :]
        final = extended.gather(1, take[:, :, None].expand(-1, -1, channels)).transpose(1, 2)  # [S, D, 3]
        chosen = final.index_select(0, plan.last_segment.clamp_min(0))
        base = initial_state.to(torch.bfloat16) if initial_state is not None else torch.zeros_like(chosen)
        state = torch.where((plan.last_segment >= 0)[:, None, None], chosen, base).contiguous()
    return output, state


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


def rms_norm_gated(x: torch.Tensor, gate: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """y = x * rsqrt(mean(x^2) + eps) * weight * sigmoid(gate) over the last axis (<= 128)."""
    _require_bf16_cuda("x", x)
    _require_bf16_cuda("gate", gate)
    if x.shape != gate.shape or x.ndim < 2:
        raise ValueError("x and gate must have the same [...,H,D] shape")
    if weight.shape != (x.shape[-1],):
        raise ValueError("weight must have shape [D]")
    return _NormGate.apply(x, gate, weight, eps)


__all__ = ["conv4_silu", "conv4_silu_segmented", "kda_decay_gate", "rms_norm_gated"]
