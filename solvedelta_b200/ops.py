"""Operator entry points with the upstream names, signatures and errors.

Mirrors causallsso/ops/operator.py:13-55 (``solvedelta_native``) and
causallsso/ops/residual_frame/operator.py:154-304
(``solvedelta_residual_frame_native``): BF16 CUDA activations with unit
innermost stride and arbitrary outer strides, FP32 ``associative_log_decay``
and ``geometry_write`` ([H], [1,H] or [B,T,H]), FP32 continuation states
``SolveDeltaState(predictor=C [B,H,r,r], S [B,H,r,V])``.  One
``torch.autograd.Function`` covers the whole operator; ``None`` incoming
gradients are legal (``set_materialize_grads(False)``), gradients are returned
for the nine tensor operands and for both initial states.

PyTorch is used for device memory and the current stream only; all arithmetic
is in the CUDA library behind ``include/solvedelta_b200.h``.  There is no CPU
or eager fallback.
"""
from __future__ import annotations

import ctypes
from typing import NamedTuple, Optional, Tuple

import torch

from . import _lib
from .packing import PackedSegments


class SolveDeltaState(NamedTuple):
    """Continuation state; same field names as causallsso/reference.py:14-16."""

    predictor: torch.Tensor
    S: torch.Tensor


def solvedelta_zero_state(batch: int, heads: int, rank: int, value_dim: int, *,
                          dtype: torch.dtype, device: torch.device) -> SolveDeltaState:
    return SolveDeltaState(
        predictor=torch.zeros(batch, heads, rank, rank, dtype=dtype, device=device),
        S=torch.zeros(batch, heads, rank, value_dim, dtype=dtype, device=device),
    )


def _operand(t: torch.Tensor) -> _lib.Operand:
    """[B,T,H,w] tensor (any outer strides, unit inner stride) -> C operand."""
    sb, st, sh = t.stride(0), t.stride(1), t.stride(2)
    return _lib.Operand(t.data_ptr(), sb, st, sh)


def _gamma_operand(t: torch.Tensor) -> _lib.Operand:
    return _lib.Operand(t.data_ptr(), t.stride(0), t.stride(1), t.stride(2))


def _shape(u: torch.Tensor, value_dim: int) -> _lib.Shape:
    B, T, H, r = u.shape
    return _lib.Shape(B, T, H, r, value_dim)


def _stream_ptr(device) -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def _buffer(nbytes: int, device) -> torch.Tensor:
    return torch.empty(max(int(nbytes), 16), dtype=torch.uint8, device=device)


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


def _fill_operands(args, tensors):
    names = ("u", "h", "q", "keys", "values", "erase_raw", "write_raw", "log_decay")
    u, h, q, k, v, ld, er, wr, gam = tensors
    for name, t in zip(names, (u, h, q, k, v, er, wr, ld)):
        setattr(args, name, _operand(t))
    args.gamma = _gamma_operand(gam)


def _mask_bytes(mask: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
    """bool [B,T] -> the same bytes as uint8 (a view, no copy when contiguous)."""
    if mask is None:
        return None
    return mask.contiguous().view(torch.uint8)


class _SolveDeltaFunction(torch.autograd.Function):
    """forward(u,h,q,k,v,log_decay,erase_raw,write_raw,gamma[B,T,H],C0|None,S0|None,valid|None,reset|None)
    -> (y, C_T, S_T); k,v,erase_raw,write_raw are the 4-D views without the edit axis; valid / reset
    are uint8 [B,T] token masks applied inside the kernels."""

    @staticmethod
    def forward(ctx, u, h, q, k, v, log_decay, erase_raw, write_raw, gamma, C0, S0, valid=None, reset=None):
        lib = _lib.load()
        device = u.device
        B, T, H, r = u.shape
        V = v.shape[-1]
        shape = _shape(u, V)
        with torch.cuda.device(device):
            y = torch.empty(B, T, H, V, dtype=torch.bfloat16, device=device)
            C_T = torch.empty(B, H, r, r, dtype=torch.float32, device=device)
            S_T = torch.empty(B, H, r, V, dtype=torch.float32, device=device)
            saved = _buffer(lib.sd_saved_bytes(ctypes.byref(shape)), device)
            scratch = _buffer(lib.sd_forward_scratch_bytes(ctypes.byref(shape)), device)
            C0c = None if C0 is None else C0.contiguous()
            S0c = None if S0 is None else S0.contiguous()
            args = _lib.ForwardArgs()
            args.shape = shape
            _fill_operands(args, (u, h, q, k, v, log_decay, erase_raw, write_raw, gamma))
            args.C0, args.S0 = _ptr(C0c), _ptr(S0c)
            args.y, args.C_T, args.S_T = y.data_ptr(), C_T.data_ptr(), S_T.data_ptr()
            args.saved, args.saved_bytes = saved.data_ptr(), saved.numel()
            args.scratch, args.scratch_bytes = scratch.data_ptr(), scratch.numel()
            args.valid_mask, args.reset_mask = _ptr(valid), _ptr(reset)
            _lib.check(lib.sd_forward(ctypes.byref(args), _stream_ptr(device)))
        ctx.set_materialize_grads(False)
        ctx.has_state = (C0 is not None, S0 is not None)
        ctx.masks = (valid, reset)
        ctx.save_for_backward(u, h, q, k, v, log_decay, erase_raw, write_raw, gamma, saved)
        return y, C_T, S_T

    @staticmethod
    def backward(ctx, dy, dC_T, dS_T):
        lib = _lib.load()
        u, h, q, k, v, log_decay, erase_raw, write_raw, gamma, saved = ctx.saved_tensors
        device = u.device
        B, T, H, r = u.shape
        V = v.shape[-1]
        shape = _shape(u, V)
        with torch.cuda.device(device):
            if dy is None:
                dy = torch.zeros(B, T, H, V, dtype=torch.bfloat16, device=device)
            elif dy.dtype != torch.bfloat16 or dy.stride(-1) != 1:
                dy = dy.to(torch.bfloat16).contiguous()
            dC_T = None if dC_T is None else dC_T.float().contiguous()
            dS_T = None if dS_T is None else dS_T.float().contiguous()
            bf = dict(dtype=torch.bfloat16, device=device)
            du = torch.empty(B, T, H, r, **bf)
            dh = torch.empty(B, T, H, r, **bf)
            dq = torch.empty(B, T, H, r, **bf)
            dk = torch.empty(B, T, H, r, **bf)
            dv = torch.empty(B, T, H, V, **bf)
            der = torch.empty(B, T, H, r, **bf)
            dwr = torch.empty(B, T, H, V, **bf)
            dld = torch.empty(B, T, H, r, dtype=torch.float32, device=device)
            dgam = torch.empty(B, T, H, dtype=torch.float32, device=device)
            dC0 = torch.empty(B, H, r, r, dtype=torch.float32, device=device)
            dS0 = torch.empty(B, H, r, V, dtype=torch.float32, device=device)
            scratch = _buffer(lib.sd_backward_scratch_bytes(ctypes.byref(shape)), device)
            args = _lib.BackwardArgs()
            args.shape = shape
            _fill_operands(args, (u, h, q, k, v, log_decay, erase_raw, write_raw, gamma))
            args.dy = _operand(dy)
            args.dC_T, args.dS_T = _ptr(dC_T), _ptr(dS_T)
            args.saved, args.saved_bytes = saved.data_ptr(), saved.numel()
            args.scratch, args.scratch_bytes = scratch.data_ptr(), scratch.numel()
            args.du, args.dh, args.dq = du.data_ptr(), dh.data_ptr(), dq.data_ptr()
            args.dkeys, args.dvalues = dk.data_ptr(), dv.data_ptr()
            args.derase_raw, args.dwrite_raw = der.data_ptr(), dwr.data_ptr()
            args.dlog_decay, args.dgamma = dld.data_ptr(), dgam.data_ptr()
            args.dC0, args.dS0 = dC0.data_ptr(), dS0.data_ptr()
            valid, reset = ctx.masks
            args.valid_mask, args.reset_mask = _ptr(valid), _ptr(reset)
            _lib.check(lib.sd_backward(ctypes.byref(args), _stream_ptr(device)))
        has_C0, has_S0 = ctx.has_state
        return (du, dh, dq, dk, dv, dld, der, dwr, dgam,
                dC0 if has_C0 else None, dS0 if has_S0 else None, None, None)


class _OjaResidual(torch.autograd.Function):
    """forward(target, source, beta[B,T,H], log_decay, query, C0|None) -> (frame_action, update, C_T)."""

    @staticmethod
    def forward(ctx, target, source, beta, log_decay, query, C0):
        lib = _lib.load()
        device = target.device
        B, T, H, r = target.shape
        shape = _shape(target, r)
        with torch.cuda.device(device):
            action = torch.empty(B, T, H, r, dtype=torch.bfloat16, device=device)
            update = torch.empty(B, T, H, r, dtype=torch.bfloat16, device=device)
            C_T = torch.empty(B, H, r, r, dtype=torch.float32, device=device)
            saved = _buffer(lib.sd_saved_bytes(ctypes.byref(shape)), device)
            scratch = _buffer(lib.sd_forward_scratch_bytes(ctypes.byref(shape)), device)
            C0c = None if C0 is None else C0.contiguous()
            args = _lib.PredictorForwardArgs()
            args.shape = shape
            args.target, args.source, args.query = _operand(target), _operand(source), _operand(query)
            args.beta, args.log_decay = _gamma_operand(beta), _operand(log_decay)
            args.C0 = _ptr(C0c)
            args.frame_action, args.update, args.C_T = action.data_ptr(), update.data_ptr(), C_T.data_ptr()
            args.saved, args.saved_bytes = saved.data_ptr(), saved.numel()
            args.scratch, args.scratch_bytes = scratch.data_ptr(), scratch.numel()
            _lib.check(lib.sd_predictor_forward(ctypes.byref(args), _stream_ptr(device)))
        ctx.set_materialize_grads(False)
        ctx.has_state = C0 is not None
        ctx.save_for_backward(target, source, beta, log_decay, query, saved, action)
        return action, update, C_T

    @staticmethod
    def backward(ctx, d_action, d_update, dC_T):
        lib = _lib.load()
        target, source, beta, log_decay, query, saved, action = ctx.saved_tensors
        device = target.device
        B, T, H, r = target.shape
        shape = _shape(target, r)
        with torch.cuda.device(device):
            d_action = None if d_action is None else d_action.to(torch.bfloat16).contiguous()
            d_update = None if d_update is None else d_update.to(torch.bfloat16).contiguous()
            dC_T = None if dC_T is None else dC_T.float().contiguous()
            bf = dict(dtype=torch.bfloat16, device=device)
            dtarget, dsource, dquery = (torch.empty(B, T, H, r, **bf) for _ in range(3))
            dld = torch.empty(B, T, H, r, dtype=torch.float32, device=device)
            dbeta = torch.empty(B, T, H, dtype=torch.float32, device=device)
            dC0 = torch.empty(B, H, r, r, dtype=torch.float32, device=device)
            scratch = _buffer(lib.sd_backward_scratch_bytes(ctypes.byref(shape)), device)
            args = _lib.PredictorBackwardArgs()
            args.shape = shape
            args.target, args.source, args.query = _operand(target), _operand(source), _operand(query)
            args.beta, args.log_decay = _gamma_operand(beta), _operand(log_decay)
            args.frame_action = action.data_ptr()
            args.d_frame_action, args.d_update, args.dC_T = _ptr(d_action), _ptr(d_update), _ptr(dC_T)
            args.saved, args.saved_bytes = saved.data_ptr(), saved.numel()
            args.scratch, args.scratch_bytes = scratch.data_ptr(), scratch.numel()
            args.dtarget, args.dsource, args.dquery = dtarget.data_ptr(), dsource.data_ptr(), dquery.data_ptr()
            args.dbeta, args.dlog_decay, args.dC0 = dbeta.data_ptr(), dld.data_ptr(), dC0.data_ptr()
            _lib.check(lib.sd_predictor_backward(ctypes.byref(args), _stream_ptr(device)))
        return dtarget, dsource, dbeta, dld, dquery, dC0 if ctx.has_state else None


def oja_residual(target: torch.Tensor, source: torch.Tensor, beta: torch.Tensor, log_decay: torch.Tensor,
                 query: torch.Tensor, initial_state: Optional[torch.Tensor], *, chunk_size: int = 32,
                 output_final_state: bool = True):
    """The predictor sub-owner of causallsso/ops/residual_frame/predictor.py:285-305, same arguments and
    returns: ``(frame_action, update, final_state)`` with ``frame_action = C_t^T query`` accumulated through
    the sequence (what the operator adds to the normalised key to form the primal address), ``update``
    the residual step Delta of the NLMS solve, and ``final_state`` the predictor state ``C`` ``[B,H,r,r]`` (None
    unless requested).  ``source`` and ``query`` are used as given (upstream passes the L2-normalised panels)
    and receive the gradients of the rows themselves.  ``chunk_size`` is accepted for signature compatibility;
    the kernels work on 64-token chunks and the result does not depend on it."""
    for name, t in (("target", target), ("source", source), ("query", query)):
        if t.device.type != "cuda" or t.dtype != torch.bfloat16:
            raise TypeError(f"{name} must be a BF16 CUDA tensor")
        if t.ndim != 4 or t.shape != target.shape:
            raise ValueError(f"{name} must have shape [B,T,H,r]")
        if t.stride(-1) != 1:
            raise ValueError("native vector operands require unit innermost stride")
    batch, length, heads, rank = target.shape
    if rank > 128:
        raise ValueError("head width above 128 is not supported")
    if log_decay.dtype != torch.float32 or log_decay.shape != target.shape:
        raise TypeError("log_decay must be FP32 [B,T,H,r]")
    if beta.dtype != torch.float32 or beta.shape != (batch, length, heads):
        raise TypeError("beta must be FP32 [B,T,H]")
    if initial_state is not None and (initial_state.dtype != torch.float32
                                      or initial_state.shape != (batch, heads, rank, rank)):
        raise ValueError("initial_state must be FP32 [B,H,r,r]")
    if log_decay.stride(-1) != 1:
        log_decay = log_decay.contiguous()
    if length == 0:
        empty = target.new_zeros(target.shape)
        final = None
        if output_final_state:
            final = (initial_state.clone() if initial_state is not None
                     else torch.zeros(batch, heads, rank, rank, dtype=torch.float32, device=target.device))
        return empty, empty.clone(), final
    action, update, final = _OjaResidual.apply(target, source, beta, log_decay, query, initial_state)
    return action, update, (final if output_final_state else None)


def _decode_step(u, h, q, k, v, log_decay, erase_raw, write_raw, gamma, C0, S0, inplace=False):
    lib = _lib.load()
    device = u.device
    B, T, H, r = u.shape
    V = v.shape[-1]
    with torch.cuda.device(device):
        # the kernel updates the cache in place; by default it works on copies, as upstream returns new tensors
        keep = inplace and C0 is not None and S0 is not None and C0.is_contiguous() and S0.is_contiguous()
        C = (torch.zeros(B, H, r, r, dtype=torch.float32, device=device) if C0 is None
             else (C0.detach() if keep else C0.detach().clone(memory_format=torch.contiguous_format)))
        S = (torch.zeros(B, H, r, V, dtype=torch.float32, device=device) if S0 is None
             else (S0.detach() if keep else S0.detach().clone(memory_format=torch.contiguous_format)))
        y = torch.empty(B, 1, H, V, dtype=torch.bfloat16, device=device)
        args = _lib.DecodeArgs()
        args.shape = _shape(u, V)
        _fill_operands(args, (u, h, q, k, v, log_decay, erase_raw, write_raw, gamma))
        args.C, args.S, args.y = C.data_ptr(), S.data_ptr(), y.data_ptr()
        _lib.check(lib.sd_decode_step(ctypes.byref(args), _stream_ptr(device)))
    return y, C, S


def solvedelta_residual_frame_native(
    u: torch.Tensor,
    h: torch.Tensor,
    q: torch.Tensor,
    keys: torch.Tensor,
    values: torch.Tensor,
    associative_log_decay: torch.Tensor,
    erase_raw: torch.Tensor,
    write_raw: torch.Tensor,
    geometry_write: torch.Tensor,
    *,
    initial_state: Optional[SolveDeltaState] = None,
    return_final_state: bool = True,
    _valid_mask: Optional[torch.Tensor] = None,
    _reset_mask: Optional[torch.Tensor] = None,
    _inplace_state: bool = False,
) -> Tuple[torch.Tensor, Optional[SolveDeltaState]]:
    """Dense BF16 path from raw gate logits.

    Same checks, in the same order and with the same exception types, as
    causallsso/ops/residual_frame/operator.py:169-196 and :247-262.  Any
    sequence length is accepted: a ragged last chunk is completed inside the
    kernels with neutral tokens (the upstream path pads with zero tokens,
    residual_frame/operator.py:218-245, which is the same arithmetic).
    """
    if u.ndim != 4:
        raise ValueError("u must have shape [B,T,H,r]")
    batch, length, heads, rank = u.shape
    if h.shape != u.shape or q.shape != u.shape:
        raise ValueError("h and q must match u")
    if keys.shape != (batch, length, heads, 1, rank):
        raise ValueError("Residual-Frame SolveDelta requires keys [B,T,H,1,r]")
    if values.ndim != 5 or values.shape[:4] != (batch, length, heads, 1):
        raise ValueError("values must have shape [B,T,H,1,d_v]")
    value_dim = values.shape[-1]
    if associative_log_decay.shape != (batch, length, heads, rank):
        raise ValueError("associative_log_decay must have shape [B,T,H,r]")
    if erase_raw.shape != keys.shape or write_raw.shape != values.shape:
        raise ValueError("erase_raw/write_raw shapes must match keys/values")
    if geometry_write.shape not in ((heads,), (1, heads), (batch, length, heads)):
        raise ValueError("geometry_write must have shape [H], [1,H], or [B,T,H]")
    if u.device.type != "cuda" or u.dtype != torch.bfloat16:
        raise TypeError("the production Residual-Frame path requires BF16 CUDA operands")
    if any(x.dtype != u.dtype for x in (h, q, keys, values, erase_raw, write_raw)):
        raise TypeError("all public vector operands must be BF16")
    if associative_log_decay.dtype != torch.float32:
        raise TypeError("associative_log_decay must be FP32")
    if geometry_write.dtype != torch.float32:
        raise TypeError("geometry_write must be FP32")
    if rank > 128 or value_dim > 128:
        raise ValueError("the B200 kernels support head widths up to 128")
    if any(x.stride(-1) != 1 for x in (u, h, q, keys, values, erase_raw, write_raw)):
        raise ValueError("native vector operands require unit innermost stride")
    if associative_log_decay.stride(-1) != 1:
        associative_log_decay = associative_log_decay.contiguous()

    predictor_initial = memory_initial = None
    if initial_state is not None:
        expected = ((batch, heads, rank, rank), (batch, heads, rank, value_dim))
        if any(value.shape != exp for value, exp in zip(initial_state, expected)):
            raise ValueError("initial_state shapes do not match the input geometry")
        if any(value.dtype != torch.float32 for value in initial_state):
            raise TypeError("all continuation states must be FP32")
        predictor_initial, memory_initial = initial_state

    if geometry_write.shape != (batch, length, heads):
        geometry_write = geometry_write.reshape(1, 1, heads).expand(batch, length, heads)

    k4, v4 = keys.squeeze(-2), values.squeeze(-2)
    er4, wr4 = erase_raw.squeeze(-2), write_raw.squeeze(-2)

    if length == 0:
        output = values.new_zeros(batch, 0, heads, value_dim)
        if not return_final_state:
            return output, None
        if initial_state is not None:
            return output, initial_state
        return output, solvedelta_zero_state(batch, heads, rank, value_dim, dtype=torch.float32,
                                             device=u.device)

    masked = _valid_mask is not None or _reset_mask is not None
    if length == 1 and not torch.is_grad_enabled() and not masked:
        # single-token recurrent inference (causallsso/ops/residual_frame/operator.py:198-216)
        y, C, S = _decode_step(u, h, q, k4, v4, associative_log_decay, er4, wr4, geometry_write,
                               predictor_initial, memory_initial, inplace=_inplace_state)
        return y, (SolveDeltaState(C, S) if return_final_state else None)

    y, C_T, S_T = _SolveDeltaFunction.apply(
        u, h, q, k4, v4, associative_log_decay, er4, wr4, geometry_write,
        predictor_initial, memory_initial, _mask_bytes(_valid_mask), _mask_bytes(_reset_mask))
    if not return_final_state:
        return y, None
    return y, SolveDeltaState(predictor=C_T, S=S_T)


def solvedelta_native(
    u: torch.Tensor,
    h: torch.Tensor,
    q: torch.Tensor,
    keys: torch.Tensor,
    values: torch.Tensor,
    associative_log_decay: torch.Tensor,
    erase_raw: torch.Tensor,
    write_raw: torch.Tensor,
    geometry_write: torch.Tensor,
    *,
    initial_state: Optional[SolveDeltaState] = None,
    return_final_state: bool = False,
    _inplace_state: bool = False,
) -> Tuple[torch.Tensor, Optional[SolveDeltaState]]:
    """Execute dense K=1 SolveDelta from raw fused-projection views.

    Same contract as causallsso/ops/operator.py:13-55.  ``_inplace_state`` (no upstream counterpart) lets a
    single-token no-grad step update the tensors of ``initial_state`` in place and return them, for a cache
    that owns its state; by default the step works on copies, as upstream returns new tensors.
    """
    if u.device.type != "cuda" or u.dtype != torch.bfloat16:
        raise TypeError("solvedelta_native requires BF16 CUDA activations")
    if keys.ndim != 5 or keys.shape[-2] != 1:
        raise ValueError("the current production path requires num_edits=1")
    if erase_raw.shape != keys.shape or erase_raw.dtype != torch.bfloat16:
        raise ValueError("erase_raw must be BF16 with the same shape as keys")
    if write_raw.shape != values.shape or write_raw.dtype != torch.bfloat16:
        raise ValueError("write_raw must be BF16 with the same shape as values")
    if any(operand.stride(-1) != 1 for operand in (u, h, q, keys, values, erase_raw, write_raw)):
        raise ValueError("native vector operands require unit innermost stride")
    return solvedelta_residual_frame_native(
        u, h, q, keys, values, associative_log_decay, erase_raw, write_raw, geometry_write,
        initial_state=initial_state, return_final_state=return_final_state, _inplace_state=_inplace_state)


def solvedelta_segmented_native(
    u: torch.Tensor,
    h: torch.Tensor,
    q: torch.Tensor,
    keys: torch.Tensor,
    values: torch.Tensor,
    associative_log_decay: torch.Tensor,
    erase_raw: torch.Tensor,
    write_raw: torch.Tensor,
    geometry_write: torch.Tensor,
    plan: PackedSegments,
    *,
    initial_state: Optional[SolveDeltaState] = None,
    return_final_state: bool = False,
) -> Tuple[torch.Tensor, Optional[SolveDeltaState]]:
    """Masked / reset batches, same contract as causallsso/ops/operator.py:96-193.

    Invalid tokens produce zero output and leave the state untouched, a reset token
    starts from the zero state, the returned state of a batch row is the one after its
    last valid token (its initial state if it has none).  Upstream gathers the valid
    tokens into a padded batch of reset-free segments and scatters the result back;
    here the kernels read the two token masks of ``plan`` themselves (a masked token is
    a neutral token, a reset is extra forgetting that no decay-weighted term survives),
    so the operands stay where they are and the call does no host work.
    """
    batch, length, heads, rank = u.shape
    if (plan.batch, plan.length) != (batch, length):
        raise ValueError("packed segment plan does not match the operator input")
    if plan.valid_mask is None or plan.reset_mask is None:
        raise ValueError("the segment plan carries no token masks (build it with build_packed_segments)")
    return solvedelta_residual_frame_native(
        u, h, q, keys, values, associative_log_decay, erase_raw, write_raw, geometry_write,
        initial_state=initial_state, return_final_state=return_final_state,
        _valid_mask=plan.valid_mask, _reset_mask=plan.reset_mask)


def solvedelta_masked_native(
    u: torch.Tensor,
    h: torch.Tensor,
    q: torch.Tensor,
    keys: torch.Tensor,
    values: torch.Tensor,
    associative_log_decay: torch.Tensor,
    erase_raw: torch.Tensor,
    write_raw: torch.Tensor,
    geometry_write: torch.Tensor,
    *,
    valid_mask: Optional[torch.Tensor] = None,
    reset_mask: Optional[torch.Tensor] = None,
    initial_state: Optional[SolveDeltaState] = None,
    return_final_state: bool = False,
) -> Tuple[torch.Tensor, Optional[SolveDeltaState]]:
    """``solvedelta_segmented_native`` without the plan: the two bool ``[B,T]`` token masks of the
    token loop (causallsso/reference.py:157-164,216-226) go straight to the kernels.  No upstream
    counterpart (upstream needs the plan to gather segments); it exists so that a caller with
    device-side masks never synchronises with the host."""
    batch, length = u.shape[:2]
    for name, mask in (("valid_mask", valid_mask), ("reset_mask", reset_mask)):
        if mask is None:
            continue
        if mask.dtype != torch.bool or mask.shape != (batch, length):
            raise ValueError(f"{name} must be bool [B,T]")
        if mask.device != u.device:
            raise ValueError("masks must share the operand device")
    return solvedelta_residual_frame_native(
        u, h, q, keys, values, associative_log_decay, erase_raw, write_raw, geometry_write,
        initial_state=initial_state, return_final_state=return_final_state,
        _valid_mask=valid_mask, _reset_mask=reset_mask)


__all__ = [
    "SolveDeltaState",
    "oja_residual",
    "solvedelta_native",
    "solvedelta_masked_native",
    "solvedelta_segmented_native",
    "solvedelta_residual_frame_native",
    "solvedelta_zero_state",
]
