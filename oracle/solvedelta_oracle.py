"""ctypes/numpy front end of the FP64 CPU checker.

TEST INFRASTRUCTURE -- not part of the shipped product.  Only the test-suite,
the smoke entry and the benchmark's CPU-baseline leg import this module; the
product package never does.

The C code restates causallsso/reference.py:82-229 (token loop) and its
adjoint.  Argument meaning mirrors ``solvedelta_reference``: ``erase`` and
``write`` are the post-sigmoid gates, ``keys``/``values`` may carry the
singleton edit axis, ``geometry_write`` may be [H], [1,H] or [B,T,H].
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from typing import NamedTuple, Optional

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "_build", "libsdoracle.so")
_lib = None

RELATIVE_FRAME_RADIUS = 5.0 / 8.0


def build(force: bool = False) -> str:
    """Compile the C checker with the Makefile next to this file."""
    src = os.path.join(_HERE, "solvedelta_oracle.c")
    stale = (
        force
        or not os.path.exists(_LIB_PATH)
        or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src)
    )
    if stale:
        subprocess.check_call(["make", "-s", "-C", _HERE, "-B"])
    return _LIB_PATH


def _load():
    global _lib
    if _lib is None:
        build()
        _lib = ctypes.CDLL(_LIB_PATH)
        _lib.sdo_forward.restype = ctypes.c_int
        _lib.sdo_backward.restype = ctypes.c_int
    return _lib


class OracleState(NamedTuple):
    predictor: np.ndarray  # C [B,H,r,r], prediction = C u
    S: np.ndarray  # [B,H,r,V]


def _f64(x) -> np.ndarray:
    return np.ascontiguousarray(np.asarray(x, dtype=np.float64))


def _ptr(x: Optional[np.ndarray]):
    if x is None:
        return ctypes.c_void_p(0)
    return x.ctypes.data_as(ctypes.c_void_p)


def _prepare(u, h, q, keys, values, log_decay, erase, write, geometry_write):
    u = _f64(u)
    if u.ndim != 4:
        raise ValueError("u must have shape [B,T,H,r]")
    B, T, H, r = u.shape
    h, q = _f64(h), _f64(q)
    if h.shape != u.shape or q.shape != u.shape:
        raise ValueError("h and q must match u")
    keys, values = _f64(keys), _f64(values)
    erase, write = _f64(erase), _f64(write)
    if keys.ndim == 5:
        if keys.shape[3] != 1:
            raise ValueError("the current SolveDelta contract requires num_edits=1")
        keys, values = keys[:, :, :, 0], values[:, :, :, 0]
        erase, write = erase[:, :, :, 0], write[:, :, :, 0]
    keys, values = np.ascontiguousarray(keys), np.ascontiguousarray(values)
    erase, write = np.ascontiguousarray(erase), np.ascontiguousarray(write)
    if keys.shape != u.shape or erase.shape != u.shape:
        raise ValueError("keys/erase must have shape [B,T,H,r]")
    V = values.shape[-1]
    if values.shape != (B, T, H, V) or write.shape != values.shape:
        raise ValueError("values/write must have shape [B,T,H,V]")
    log_decay = _f64(log_decay)
    if log_decay.shape != u.shape:
        raise ValueError("associative_log_decay must have shape [B,T,H,r]")
    gamma = _f64(geometry_write)
    if gamma.shape in ((H,), (1, H)):
        gamma = np.ascontiguousarray(np.broadcast_to(gamma.reshape(1, 1, H), (B, T, H)))
    elif gamma.shape != (B, T, H):
        raise ValueError("geometry_write must have shape [H], [1,H], or [B,T,H]")
    return (B, T, H, r, V), (u, h, q, keys, values, log_decay, erase, write, gamma)


def _masks(shape, valid_mask, reset_mask):
    B, T = shape[0], shape[1]
    out = []
    for m in (valid_mask, reset_mask):
        if m is None:
            out.append(None)
        else:
            m = np.ascontiguousarray(np.asarray(m).astype(np.uint8))
            if m.shape != (B, T):
                raise ValueError("masks must be bool [B,T]")
            out.append(m)
    return out


def _states(shape, initial_state):
    B, T, H, r, V = shape
    if initial_state is None:
        return None, None
    C0, S0 = _f64(initial_state[0]), _f64(initial_state[1])
    if C0.shape != (B, H, r, r) or S0.shape != (B, H, r, V):
        raise ValueError("initial_state shapes do not match inputs")
    return C0, S0


def forward(u, h, q, keys, values, log_decay, erase, write, geometry_write, *,
            initial_state=None, valid_mask=None, reset_mask=None):
    """Token-by-token FP64 forward.  Returns (y [B,T,H,V], OracleState)."""
    shape, ops = _prepare(u, h, q, keys, values, log_decay, erase, write, geometry_write)
    B, T, H, r, V = shape
    C0, S0 = _states(shape, initial_state)
    valid, reset = _masks(shape, valid_mask, reset_mask)
    y = np.zeros((B, T, H, V))
    CT = np.zeros((B, H, r, r))
    ST = np.zeros((B, H, r, V))
    rc = _load().sdo_forward(
        B, T, H, r, V, *[_ptr(x) for x in ops], _ptr(C0), _ptr(S0), _ptr(valid),
        _ptr(reset), _ptr(y), _ptr(CT), _ptr(ST))
    if rc != 0:
        raise MemoryError("oracle forward failed")
    return y, OracleState(CT, ST)


def backward(u, h, q, keys, values, log_decay, erase, write, geometry_write, dy, *,
             dC_T=None, dS_T=None, initial_state=None, valid_mask=None,
             reset_mask=None):
    """Full VJP.  Returns a dict of gradients keyed by operand name.

    ``erase``/``write`` gradients are with respect to the post-sigmoid gates;
    ``geometry_write`` gradient is per token [B,T,H] (sum it over B,T for a
    per-head parameter).
    """
    shape, ops = _prepare(u, h, q, keys, values, log_decay, erase, write, geometry_write)
    B, T, H, r, V = shape
    C0, S0 = _states(shape, initial_state)
    valid, reset = _masks(shape, valid_mask, reset_mask)
    dy = _f64(dy)
    if dy.shape != (B, T, H, V):
        raise ValueError("dy must have shape [B,T,H,V]")
    dC_T = None if dC_T is None else _f64(dC_T)
    dS_T = None if dS_T is None else _f64(dS_T)
    names_r = ("u", "h", "q", "keys", "log_decay", "erase")
    grads = {n: np.zeros((B, T, H, r)) for n in names_r}
    grads["values"] = np.zeros((B, T, H, V))
    grads["write"] = np.zeros((B, T, H, V))
    grads["geometry_write"] = np.zeros((B, T, H))
    grads["C0"] = np.zeros((B, H, r, r))
    grads["S0"] = np.zeros((B, H, r, V))
    rc = _load().sdo_backward(
        B, T, H, r, V, *[_ptr(x) for x in ops], _ptr(C0), _ptr(S0), _ptr(valid),
        _ptr(reset), _ptr(dy), _ptr(dC_T), _ptr(dS_T),
        _ptr(grads["u"]), _ptr(grads["h"]), _ptr(grads["q"]), _ptr(grads["keys"]),
        _ptr(grads["values"]), _ptr(grads["log_decay"]), _ptr(grads["erase"]),
        _ptr(grads["write"]), _ptr(grads["geometry_write"]), _ptr(grads["C0"]),
        _ptr(grads["S0"]))
    if rc != 0:
        raise MemoryError("oracle backward failed")
    return grads


def set_threads(n: int) -> None:
    """Limit the OpenMP team used by the C checker (0 = library default)."""
    try:
        omp = ctypes.CDLL("libgomp.so.1")
        omp.omp_set_num_threads(int(n))
    except OSError:
        pass
