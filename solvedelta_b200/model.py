"""SolveDelta mixer: fused input projection, conv4 + SiLU, decay / geometry
gates, the chunked recurrence, sigmoid-gated RMSNorm and output projection.

Same parameter names, projection layout and call signature as upstream's
``SolveDelta`` (causallsso/model.py:27-474), so upstream state dicts load:
``in_proj`` packs (q, k, v, u, h, erase_raw, write_raw, geometry_raw,
decay_hidden, output_gate_hidden) and is padded to a multiple of 64 columns
(model.py:39-60); q/k/v go through the conv, the other slices are read in
place as strided views of the projection row; decay and geometry gates are
evaluated in FP32.  The module-level name ``solvedelta_native`` is the call
site upstream's tests patch (tests/model/test_modeling_solvedelta.py:343).

GEMMs run through torch (cuBLAS); everything else is this package's CUDA
library.  Inputs must be BF16 CUDA tensors: there is no CPU path here
(upstream's CPU branch is model.py:430-462).
"""
from __future__ import annotations

import math
from typing import NamedTuple, Optional

import torch
import torch.nn.functional as F
from torch import nn

from .config import SolveDeltaConfig
from .mixer_ops import (conv4_silu, kda_decay_gate, mixer_decode_step, pack_rows, rms_norm_gated,
                        rms_norm_gated_linear, small_linear)
from .ops import SolveDeltaState, solvedelta_masked_native, solvedelta_native


class SolveDeltaLayerState(NamedTuple):
    operator: SolveDeltaState
    conv: Optional[torch.Tensor]


class _SplitRow(torch.autograd.Function):
    """Slices of the fused projection row as views (no copy), with a backward that writes every
    slice gradient once into one row-shaped buffer.  Plain slicing would make autograd allocate and
    add one zero-filled full row per slice (ten rows of 7488 columns per token for the mixer)."""

    @staticmethod
    def forward(ctx, row, sizes):
        ctx.sizes = sizes
        ctx.row_shape, ctx.row_dtype, ctx.row_device = row.shape, row.dtype, row.device
        ctx.set_materialize_grads(False)
        pieces, start = [], 0
        for size in sizes:
            pieces.append(row[..., start:start + size])
            start += size
        return tuple(pieces)

    @staticmethod
    def backward(ctx, *grads):
        if all(g is None for g in grads):
            return None, None
        if ctx.row_dtype == torch.bfloat16:
            packed = pack_rows(grads, ctx.sizes, ctx.row_shape, ctx.row_device)   # one kernel for the whole row
            if packed is not None:
                return packed, None
        drow = torch.empty(ctx.row_shape, dtype=ctx.row_dtype, device=ctx.row_device)
        start = 0
        for size, grad in zip(ctx.sizes, grads):
            target = drow[..., start:start + size]
            if grad is None:
                target.zero_()
            else:
                target.copy_(grad)
            start += size
        if start < ctx.row_shape[-1]:
            drow[..., start:].zero_()   # padding columns of the projection
        return drow, None


class RMSNormGated(nn.Module):
    """y = RMSNorm(x) * weight * sigmoid(gate) (causallsso/ops/norm_gate.py:162-217)."""

    def __init__(self, hidden_size: int, eps: float = 1e-6) -> None:
        super().__init__()
        self.hidden_size = hidden_size
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(hidden_size))

    def forward(self, x: torch.Tensor, gate: torch.Tensor) -> torch.Tensor:
        return rms_norm_gated(x, gate, self.weight, self.eps)

    def forward_linear(self, x: torch.Tensor, gate: torch.Tensor, linear: nn.Linear) -> torch.Tensor:
        """The following projection without saving the normalised panel (norm_gate.py:195-217)."""
        return rms_norm_gated_linear(x, gate, self.weight, linear.weight, linear.bias, self.eps)


class SolveDelta(nn.Module):
    def __init__(self, config: SolveDeltaConfig) -> None:
        super().__init__()
        self.config = config
        heads = config.num_heads
        width = config.resolved_head_k_dim
        value_width = config.resolved_head_v_dim
        gate_rank = value_width
        self.projection_sizes = (
            heads * width, heads * width, heads * value_width,   # q, k, v (through the conv)
            heads * width, heads * width,                         # u, h
            heads * width, heads * value_width,                   # erase_raw, write_raw
            heads, gate_rank, gate_rank)                          # geometry_raw, decay_hidden, gate_hidden
        self.projection_width = sum(self.projection_sizes)
        self.projection_padding = (-self.projection_width) % 64
        self.in_proj = nn.Linear(config.hidden_size, self.projection_width + self.projection_padding,
                                 bias=config.bias)
        self.output_proj = nn.Linear(heads * value_width, config.hidden_size, bias=config.bias)
        self.decay_proj = nn.Linear(gate_rank, heads * width, bias=False)
        self.output_gate_proj = nn.Linear(gate_rank, heads * value_width, bias=True)
        self.output_norm = RMSNormGated(value_width, eps=config.norm_eps)
        if config.use_short_conv:
            self.conv_weight = nn.Parameter(torch.empty(sum(self.projection_sizes[:3]), 4))
            nn.init.kaiming_uniform_(self.conv_weight, a=5 ** 0.5)
        self.geometry_write_bias = nn.Parameter(torch.full((heads,), math.log(9.0), dtype=torch.float32))
        rate = torch.empty(heads, dtype=torch.float32).uniform_(1, 16)
        self.associative_log_rate = nn.Parameter(rate.log())
        step = torch.exp(torch.rand(heads, width, dtype=torch.float32) * (math.log(0.1) - math.log(0.001))
                         + math.log(0.001)).clamp_min_(1e-4)
        self.associative_decay_bias = nn.Parameter(step + torch.log(-torch.expm1(-step)))
        for parameter in (self.geometry_write_bias, self.associative_log_rate, self.associative_decay_bias):
            parameter._no_weight_decay = True

    @staticmethod
    def _linear(layer: nn.Linear, x: torch.Tensor) -> torch.Tensor:
        weight = layer.weight.to(x.dtype)
        small = small_linear(x, weight, None if layer.bias is None else layer.bias.to(x.dtype))
        if small is not None:   # the few rows of a cached single-token step
            return small
        if layer.bias is None:
            return F.linear(x, weight)
        # one GEMM with the bias in its epilogue: on a strided slice of the projection row F.linear would run the
        # product and a separate element-wise add
        rows = x.reshape(-1, x.shape[-1])
        return torch.addmm(layer.bias.to(x.dtype), rows, weight.t()).view(*x.shape[:-1], weight.shape[0])

    def _fp32_copy(self, name: str) -> torch.Tensor:
        """Contiguous FP32 copy of a parameter for the fused decode kernel, refreshed when the parameter changes."""
        parameter = getattr(self, name)
        if parameter.dtype == torch.float32 and parameter.is_contiguous():
            return parameter.detach()
        cache = self.__dict__.setdefault("_fp32_copies", {})
        key = (parameter.data_ptr(), parameter._version)
        hit = cache.get(name)
        if hit is None or hit[0] != key:
            hit = (key, parameter.detach().float().contiguous())
            cache[name] = hit
        return hit[1]

    def _fp32_norm_weight(self) -> torch.Tensor:
        weight = self.output_norm.weight
        if weight.dtype == torch.float32 and weight.is_contiguous():
            return weight.detach()
        cache = self.__dict__.setdefault("_fp32_copies", {})
        key = (weight.data_ptr(), weight._version)
        hit = cache.get("output_norm.weight")
        if hit is None or hit[0] != key:
            hit = (key, weight.detach().float().contiguous())
            cache["output_norm.weight"] = hit
        return hit[1]

    def _fused_decode_applies(self, inplace_state, masked, length, initial_state, geometry_enabled,
                              associative_decay_enabled, return_final_state) -> bool:
        if not (inplace_state and return_final_state and not masked and length == 1 and self.config.use_short_conv
                and geometry_enabled and associative_decay_enabled and not torch.is_grad_enabled()):
            return False
        if initial_state is None or initial_state.conv is None or initial_state.operator is None:
            return False
        conv, (C, S) = initial_state.conv, initial_state.operator
        return (conv.dtype == torch.bfloat16 and conv.is_contiguous() and C.dtype == torch.float32
                and S.dtype == torch.float32 and C.is_contiguous() and S.is_contiguous())

    def forward(self, hidden_states: torch.Tensor, *, initial_state: Optional[SolveDeltaLayerState] = None,
                valid_mask: Optional[torch.Tensor] = None, reset_mask: Optional[torch.Tensor] = None,
                geometry_enabled: bool = True, associative_decay_enabled: bool = True,
                return_final_state: bool = False, inplace_state: bool = False):
        if hidden_states.ndim != 3:
            raise ValueError("hidden_states must have shape [B,T,hidden_size]")
        batch, length, hidden_width = hidden_states.shape
        if hidden_width != self.config.hidden_size:
            raise ValueError("hidden state width does not match the configuration")
        if hidden_states.device.type != "cuda" or hidden_states.dtype != torch.bfloat16:
            raise TypeError("the B200 mixer requires BF16 CUDA hidden states (no CPU path)")
        masked = valid_mask is not None or reset_mask is not None
        if masked:
            # masks and resets are applied inside the conv and operator kernels on the padded batch: no segment
            # plan, no host synchronisation (upstream repacks into reset-free segments, causallsso/model.py:302-316)
            for name, mask in (("valid_mask", valid_mask), ("reset_mask", reset_mask)):
                if mask is None:
                    continue
                if mask.dtype != torch.bool or mask.shape != (batch, length):
                    raise ValueError(f"{name} must be bool [B,T]")
                if mask.device != hidden_states.device:
                    raise ValueError("masks must share the activation device")
        heads = self.config.num_heads
        width = self.config.resolved_head_k_dim
        value_width = self.config.resolved_head_v_dim
        sizes = self.projection_sizes
        row = self._linear(self.in_proj, hidden_states)          # [B,T,P] BF16, slices stay views
        conv_state = initial_state.conv if initial_state is not None else None
        if self.config.use_short_conv:
            # q | k | v stay one slice: the conv reads it in place
            split = _SplitRow.apply(row, (sum(sizes[:3]),) + tuple(sizes[3:]))
            qkv_in = split[0]
            pieces = (None, None, None) + tuple(split[1:])
        else:
            pieces = _SplitRow.apply(row, tuple(sizes))
        piece = lambda i: pieces[i]
        view = lambda x, size: x.unflatten(-1, (heads, size))  # stays a view of the projection row
        if self._fused_decode_applies(inplace_state, masked, length, initial_state, geometry_enabled,
                                      associative_decay_enabled, return_final_state):
            # cached single-token step: conv, decay gate, geometry rate and the recurrent step in one launch, the
            # cache's conv window and operator states updated in place
            dw, gw, gb = self.decay_proj.weight, self.output_gate_proj.weight, self.output_gate_proj.bias
            in_kernel = (dw.dtype == gw.dtype == torch.bfloat16 and dw.is_contiguous() and gw.is_contiguous()
                         and gb.dtype == torch.bfloat16 and dw.shape[1] % 16 == 0 and dw.shape[1] <= 128)
            if in_kernel:   # the two small projections in front of the gates run inside the kernel too
                associative_raw = output_gate = None
                projections = (piece(8), dw.detach(), piece(9), gw.detach(), gb.detach())
            else:
                associative_raw = self._linear(self.decay_proj, piece(8)).view(batch, length, heads, width)
                output_gate = self._linear(self.output_gate_proj, piece(9)).view(batch, length, heads, value_width)
                projections = None
            operator = initial_state.operator
            output = mixer_decode_step(
                view(piece(3), width), view(piece(4), width), view(piece(5), width), view(piece(6), value_width),
                qkv_in, self._fp32_copy("conv_weight"), initial_state.conv, associative_raw,
                self._fp32_copy("associative_log_rate"), self._fp32_copy("associative_decay_bias").reshape(-1),
                piece(7), self._fp32_copy("geometry_write_bias"), operator.predictor, operator.S,
                output_gate=output_gate, norm_weight=self._fp32_norm_weight(), norm_eps=self.output_norm.eps,
                gate_projections=projections)
            result = self._linear(self.output_proj, output.reshape(batch, length, heads * value_width))
            return result, SolveDeltaLayerState(SolveDeltaState(operator.predictor, operator.S), initial_state.conv)
        if self.config.use_short_conv:
            qkv, final_conv = conv4_silu(qkv_in, self.conv_weight, conv_state, return_final_state,
                                         valid_mask, reset_mask, _inplace_state=inplace_state)
            q_raw, key_raw, value_raw = qkv.split(sizes[:3], dim=-1)
        else:
            q_raw, key_raw, value_raw = (F.silu(piece(i)) for i in range(3))
            final_conv = None
        u, h = view(piece(3), width), view(piece(4), width)
        q = view(q_raw, width)
        keys = view(key_raw, width).unsqueeze(-2)
        values = view(value_raw, value_width).unsqueeze(-2)
        erase_raw = view(piece(5), width).unsqueeze(-2)
        write_raw = view(piece(6), value_width).unsqueeze(-2)
        associative_raw = self._linear(self.decay_proj, piece(8)).view(batch, length, heads, width)
        output_gate = self._linear(self.output_gate_proj, piece(9)).view(batch, length, heads, value_width)
        log_decay = kda_decay_gate(associative_raw, self.associative_log_rate, self.associative_decay_bias)
        geometry_write = torch.sigmoid(piece(7).float() + self.geometry_write_bias.float().view(1, 1, heads))
        if not geometry_enabled:
            geometry_write = torch.zeros_like(geometry_write)
        if not associative_decay_enabled:
            log_decay = torch.zeros_like(log_decay)
        operator_initial = initial_state.operator if initial_state is not None else None
        if not masked:
            extra = {"_inplace_state": True} if inplace_state else {}   # the public signature is upstream's
            output, operator_state = solvedelta_native(
                u, h, q, keys, values, log_decay, erase_raw, write_raw, geometry_write,
                initial_state=operator_initial, return_final_state=return_final_state, **extra)
        else:
            output, operator_state = solvedelta_masked_native(
                u, h, q, keys, values, log_decay, erase_raw, write_raw, geometry_write,
                valid_mask=valid_mask, reset_mask=reset_mask,
                initial_state=operator_initial, return_final_state=return_final_state)
        result = self.output_norm.forward_linear(output, output_gate, self.output_proj)
        if not return_final_state:
            return result
        if operator_state is None:
            raise RuntimeError("operator did not return the requested final state")
        return result, SolveDeltaLayerState(operator_state, final_conv)


__all__ = ["RMSNormGated", "SolveDelta", "SolveDeltaLayerState"]
