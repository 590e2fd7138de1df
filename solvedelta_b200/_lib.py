"""Loader and builder of the CUDA library behind the C ABI.

The shared object is built in-tree (``solvedelta_b200/_build``) with nvcc for
sm_100a and loaded through ctypes; the structures below mirror
``include/solvedelta_b200.h`` field by field.  There is no fallback: if the
library is missing, every entry point raises.
"""
from __future__ import annotations

import ctypes
import os
import shutil
import subprocess

_PKG = os.path.dirname(os.path.abspath(__file__))
_ROOT = os.path.dirname(_PKG)
_SRC = os.path.join(_PKG, "csrc")
_BUILD = os.path.join(_PKG, "_build")
LIB_PATH = os.path.join(_BUILD, "libsolvedelta_b200.so")
# the profiling build: same sources with -DSD_DIAGNOSTICS (phase clock stamps, per-launch events);
# only bench.py's per-kernel breakdown loads it
DIAG_LIB_PATH = os.path.join(_BUILD, "libsolvedelta_b200_diag.so")
HEADER_PATH = os.path.join(_ROOT, "include", "solvedelta_b200.h")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--expt-extended-lambda", "-shared", "-Xcompiler", "-fPIC",
]


def _sources():
    out = [HEADER_PATH]
    for name in sorted(os.listdir(_SRC)):
        if name.endswith((".cu", ".cuh", ".h")):
            out.append(os.path.join(_SRC, name))
    return out


def _nvcc():
    for cand in (shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    return None


def is_stale(path: str = LIB_PATH) -> bool:
    if not os.path.exists(path):
        return True
    built = os.path.getmtime(path)
    return any(os.path.getmtime(s) > built for s in _sources())


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile csrc/*.cu into the in-tree shared libraries (sm_100a only): the product library and
    its profiling twin."""
    nvcc = _nvcc()
    jobs = []
    for path, extra in ((LIB_PATH, []), (DIAG_LIB_PATH, ["-DSD_DIAGNOSTICS"])):
        if not force and not is_stale(path):
            continue
        if nvcc is None:
            raise RuntimeError("nvcc not found: cannot build " + os.path.basename(path))
        os.makedirs(_BUILD, exist_ok=True)
        units = [os.path.join(_SRC, n) for n in sorted(os.listdir(_SRC)) if n.endswith(".cu")]
        cmd = [nvcc, *NVCC_FLAGS, *extra, "-o", path, *units]
        if verbose:
            cmd.insert(1, "-Xptxas")
            cmd.insert(2, "-v")
        jobs.append((cmd, subprocess.Popen(cmd)))   # the two builds run side by side
    for cmd, proc in jobs:
        if proc.wait() != 0:
            raise subprocess.CalledProcessError(proc.returncode, cmd)
    return LIB_PATH


class Shape(ctypes.Structure):
    _fields_ = [("B", ctypes.c_int32), ("T", ctypes.c_int32), ("H", ctypes.c_int32),
                ("r", ctypes.c_int32), ("V", ctypes.c_int32)]


class Operand(ctypes.Structure):
    _fields_ = [("ptr", ctypes.c_void_p), ("stride_b", ctypes.c_int64),
                ("stride_t", ctypes.c_int64), ("stride_h", ctypes.c_int64)]


_OPERANDS = ("u", "h", "q", "keys", "values", "erase_raw", "write_raw", "log_decay", "gamma")


class ForwardArgs(ctypes.Structure):
    _fields_ = ([("shape", Shape)] + [(n, Operand) for n in _OPERANDS] + [
        ("C0", ctypes.c_void_p), ("S0", ctypes.c_void_p), ("y", ctypes.c_void_p),
        ("C_T", ctypes.c_void_p), ("S_T", ctypes.c_void_p),
        ("saved", ctypes.c_void_p), ("saved_bytes", ctypes.c_size_t),
        ("scratch", ctypes.c_void_p), ("scratch_bytes", ctypes.c_size_t),
        ("valid_mask", ctypes.c_void_p), ("reset_mask", ctypes.c_void_p)])


class BackwardArgs(ctypes.Structure):
    _fields_ = ([("shape", Shape)] + [(n, Operand) for n in _OPERANDS] + [
        ("dy", Operand), ("dC_T", ctypes.c_void_p), ("dS_T", ctypes.c_void_p),
        ("saved", ctypes.c_void_p), ("saved_bytes", ctypes.c_size_t),
        ("scratch", ctypes.c_void_p), ("scratch_bytes", ctypes.c_size_t),
        ("du", ctypes.c_void_p), ("dh", ctypes.c_void_p), ("dq", ctypes.c_void_p),
        ("dkeys", ctypes.c_void_p), ("dvalues", ctypes.c_void_p),
        ("derase_raw", ctypes.c_void_p), ("dwrite_raw", ctypes.c_void_p),
        ("dlog_decay", ctypes.c_void_p), ("dgamma", ctypes.c_void_p),
        ("dC0", ctypes.c_void_p), ("dS0", ctypes.c_void_p),
        ("valid_mask", ctypes.c_void_p), ("reset_mask", ctypes.c_void_p)])


class AddRmsnormArgs(ctypes.Structure):
    _fields_ = [("rows", ctypes.c_int64), ("D", ctypes.c_int32), ("eps", ctypes.c_float),
                ("x", ctypes.c_void_p), ("delta", ctypes.c_void_p), ("weight", ctypes.c_void_p),
                ("sum", ctypes.c_void_p), ("normed", ctypes.c_void_p)]


class AddRmsnormBackwardArgs(ctypes.Structure):
    _fields_ = [("rows", ctypes.c_int64), ("D", ctypes.c_int32), ("eps", ctypes.c_float),
                ("sum", ctypes.c_void_p), ("weight", ctypes.c_void_p), ("dsum", ctypes.c_void_p),
                ("dnormed", ctypes.c_void_p), ("dx", ctypes.c_void_p), ("dweight", ctypes.c_void_p),
                ("scratch", ctypes.c_void_p), ("scratch_bytes", ctypes.c_size_t)]


class SwigluArgs(ctypes.Structure):
    _fields_ = [("rows", ctypes.c_int64), ("I", ctypes.c_int32), ("gate_value", ctypes.c_void_p),
                ("out", ctypes.c_void_p), ("dout", ctypes.c_void_p), ("dgate_value", ctypes.c_void_p)]


PACK_MAX_PIECES = 12


class RowPiece(ctypes.Structure):
    _fields_ = [("src", ctypes.c_void_p), ("width", ctypes.c_int32)]


class PackRowsArgs(ctypes.Structure):
    _fields_ = [("rows", ctypes.c_int64), ("pieces", ctypes.c_int32), ("row_width", ctypes.c_int32),
                ("piece", RowPiece * PACK_MAX_PIECES), ("dst", ctypes.c_void_p)]


GEMV_MAX_ROWS = 4


class GemvArgs(ctypes.Structure):
    _fields_ = [("M", ctypes.c_int32), ("N", ctypes.c_int32), ("K", ctypes.c_int32), ("swiglu", ctypes.c_int32),
                ("x", ctypes.c_void_p), ("x_stride", ctypes.c_int64), ("weight", ctypes.c_void_p),
                ("bias", ctypes.c_void_p), ("y", ctypes.c_void_p), ("y_stride", ctypes.c_int64)]


class CrossEntropyArgs(ctypes.Structure):
    _fields_ = [("rows", ctypes.c_int64), ("V", ctypes.c_int32), ("logits", ctypes.c_void_p),
                ("labels", ctypes.c_void_p), ("ignore_index", ctypes.c_int64), ("lse", ctypes.c_void_p),
                ("row_loss", ctypes.c_void_p), ("coef", ctypes.c_void_p), ("dlogits", ctypes.c_void_p)]


class MixerDecodeArgs(ctypes.Structure):
    _fields_ = ([("shape", Shape)] + [(n, Operand) for n in ("u", "h", "erase_raw", "write_raw")] + [
        ("qkv", ctypes.c_void_p), ("qkv_stride_b", ctypes.c_int64), ("conv_weight", ctypes.c_void_p),
        ("conv_state", ctypes.c_void_p), ("decay_raw", ctypes.c_void_p), ("decay_stride_b", ctypes.c_int64),
        ("log_rate", ctypes.c_void_p), ("decay_bias", ctypes.c_void_p), ("geometry_raw", ctypes.c_void_p),
        ("geometry_stride_b", ctypes.c_int64), ("geometry_bias", ctypes.c_void_p),
        ("C", ctypes.c_void_p), ("S", ctypes.c_void_p), ("y", ctypes.c_void_p),
        ("norm_weight", ctypes.c_void_p), ("norm_eps", ctypes.c_float), ("output_gate", ctypes.c_void_p),
        ("output_gate_stride_b", ctypes.c_int64),
        ("gate_rank", ctypes.c_int32), ("decay_hidden", ctypes.c_void_p), ("decay_hidden_stride_b", ctypes.c_int64),
        ("decay_proj_weight", ctypes.c_void_p), ("gate_hidden", ctypes.c_void_p),
        ("gate_hidden_stride_b", ctypes.c_int64), ("gate_proj_weight", ctypes.c_void_p),
        ("gate_proj_bias", ctypes.c_void_p)])


class PredictorForwardArgs(ctypes.Structure):
    _fields_ = ([("shape", Shape)] + [(n, Operand) for n in ("target", "source", "query", "beta", "log_decay")] + [
        ("C0", ctypes.c_void_p), ("frame_action", ctypes.c_void_p), ("update", ctypes.c_void_p),
        ("C_T", ctypes.c_void_p),
        ("saved", ctypes.c_void_p), ("saved_bytes", ctypes.c_size_t),
        ("scratch", ctypes.c_void_p), ("scratch_bytes", ctypes.c_size_t),
        ("valid_mask", ctypes.c_void_p), ("reset_mask", ctypes.c_void_p)])


class PredictorBackwardArgs(ctypes.Structure):
    _fields_ = ([("shape", Shape)] + [(n, Operand) for n in ("target", "source", "query", "beta", "log_decay")] + [
        ("frame_action", ctypes.c_void_p), ("d_frame_action", ctypes.c_void_p), ("d_update", ctypes.c_void_p),
        ("dC_T", ctypes.c_void_p),
        ("saved", ctypes.c_void_p), ("saved_bytes", ctypes.c_size_t),
        ("scratch", ctypes.c_void_p), ("scratch_bytes", ctypes.c_size_t),
        ("dtarget", ctypes.c_void_p), ("dsource", ctypes.c_void_p), ("dquery", ctypes.c_void_p),
        ("dbeta", ctypes.c_void_p), ("dlog_decay", ctypes.c_void_p), ("dC0", ctypes.c_void_p),
        ("valid_mask", ctypes.c_void_p), ("reset_mask", ctypes.c_void_p)])


class DecodeArgs(ctypes.Structure):
    _fields_ = ([("shape", Shape)] + [(n, Operand) for n in _OPERANDS] + [
        ("C", ctypes.c_void_p), ("S", ctypes.c_void_p), ("y", ctypes.c_void_p)])


class Conv4ForwardArgs(ctypes.Structure):
    _fields_ = [("B", ctypes.c_int32), ("T", ctypes.c_int32), ("D", ctypes.c_int32),
                ("x", ctypes.c_void_p), ("x_stride_b", ctypes.c_int64), ("x_stride_t", ctypes.c_int64),
                ("weight", ctypes.c_void_p), ("initial_state", ctypes.c_void_p), ("y", ctypes.c_void_p),
                ("final_state", ctypes.c_void_p), ("valid_mask", ctypes.c_void_p), ("reset_mask", ctypes.c_void_p)]


class Conv4BackwardArgs(ctypes.Structure):
    _fields_ = [("B", ctypes.c_int32), ("T", ctypes.c_int32), ("D", ctypes.c_int32),
                ("x", ctypes.c_void_p), ("x_stride_b", ctypes.c_int64), ("x_stride_t", ctypes.c_int64),
                ("weight", ctypes.c_void_p), ("initial_state", ctypes.c_void_p), ("dy", ctypes.c_void_p),
                ("dx", ctypes.c_void_p), ("dweight", ctypes.c_void_p), ("dinitial_state", ctypes.c_void_p),
                ("scratch", ctypes.c_void_p), ("scratch_bytes", ctypes.c_size_t),
                ("valid_mask", ctypes.c_void_p), ("reset_mask", ctypes.c_void_p)]


class KdaGateArgs(ctypes.Structure):
    _fields_ = [("rows", ctypes.c_int64), ("H", ctypes.c_int32), ("r", ctypes.c_int32),
                ("raw", ctypes.c_void_p), ("log_rate", ctypes.c_void_p), ("bias", ctypes.c_void_p),
                ("log_decay", ctypes.c_void_p), ("dlog_decay", ctypes.c_void_p), ("draw", ctypes.c_void_p),
                ("dlog_rate", ctypes.c_void_p), ("dbias", ctypes.c_void_p), ("scratch", ctypes.c_void_p),
                ("scratch_bytes", ctypes.c_size_t)]


class NormGateArgs(ctypes.Structure):
    _fields_ = [("rows", ctypes.c_int64), ("V", ctypes.c_int32), ("eps", ctypes.c_float),
                ("x", ctypes.c_void_p), ("gate", ctypes.c_void_p), ("weight", ctypes.c_void_p),
                ("y", ctypes.c_void_p), ("dy", ctypes.c_void_p), ("dx", ctypes.c_void_p),
                ("dgate", ctypes.c_void_p), ("dweight", ctypes.c_void_p), ("scratch", ctypes.c_void_p),
                ("scratch_bytes", ctypes.c_size_t)]


EXPORTS = (
    "sd_saved_bytes", "sd_forward_scratch_bytes", "sd_backward_scratch_bytes",
    "sd_forward", "sd_backward", "sd_decode_step", "sd_forward_launches",
    "sd_backward_launches", "sd_panel_info", "sd_status_string", "sd_version",
    "sd_chunk_tokens", "sd_forward_static", "sd_panel_kind", "sd_device_fault", "sd_device_fault_clear",
    "sd_predictor_forward", "sd_predictor_backward", "sd_mixer_decode_step", "sd_add_rmsnorm", "sd_swiglu",
    "sd_add_rmsnorm_backward_scratch_bytes", "sd_add_rmsnorm_backward", "sd_swiglu_backward", "sd_pack_rows",
    "sd_cross_entropy_forward", "sd_cross_entropy_backward", "sd_gemv",
    "sd_conv4_backward_scratch_bytes", "sd_conv4_silu_forward", "sd_conv4_silu_backward",
    "sd_kda_gate_backward_scratch_bytes", "sd_kda_gate_forward", "sd_kda_gate_backward",
    "sd_norm_gate_backward_scratch_bytes", "sd_norm_gate_forward", "sd_norm_gate_backward",
)

_lib = None
_diag = None


def load_diagnostics() -> ctypes.CDLL:
    """The profiling build (-DSD_DIAGNOSTICS): everything the product library exports plus
    sd_profile_step / sd_launch_name / sd_debug_timeline.  Only measurement code loads it."""
    global _diag
    if _diag is None:
        if not os.path.exists(DIAG_LIB_PATH):
            raise RuntimeError(f"{DIAG_LIB_PATH} is missing: run solvedelta_b200.build()")
        _diag = _declare(ctypes.CDLL(DIAG_LIB_PATH))
        _diag.sd_debug_timeline.restype = None
        _diag.sd_debug_timeline.argtypes = [ctypes.c_void_p]
        _diag.sd_profile_step.restype = ctypes.c_int
        _diag.sd_profile_step.argtypes = [ctypes.POINTER(ForwardArgs), ctypes.POINTER(BackwardArgs),
                                          ctypes.c_void_p, ctypes.POINTER(ctypes.c_float), ctypes.c_int,
                                          ctypes.POINTER(ctypes.c_int)]
        _diag.sd_launch_name.restype = ctypes.c_char_p
        _diag.sd_launch_name.argtypes = [ctypes.c_int]
    return _diag


def load() -> ctypes.CDLL:
    """Return the loaded library; raise if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -c 'import solvedelta_b200; "
            "solvedelta_b200.build()'` (needs nvcc); there is no fallback path")
    _lib = _declare(ctypes.CDLL(LIB_PATH))
    return _lib


def _declare(lib: ctypes.CDLL) -> ctypes.CDLL:
    sp = ctypes.POINTER(Shape)
    for name in ("sd_saved_bytes", "sd_forward_scratch_bytes", "sd_backward_scratch_bytes"):
        getattr(lib, name).restype = ctypes.c_size_t
        getattr(lib, name).argtypes = [sp]
    lib.sd_forward.restype = ctypes.c_int
    lib.sd_forward.argtypes = [ctypes.POINTER(ForwardArgs), ctypes.c_void_p]
    lib.sd_forward_static.restype = ctypes.c_int
    lib.sd_forward_static.argtypes = [ctypes.POINTER(ForwardArgs), ctypes.c_void_p]
    lib.sd_backward.restype = ctypes.c_int
    lib.sd_backward.argtypes = [ctypes.POINTER(BackwardArgs), ctypes.c_void_p]
    lib.sd_decode_step.restype = ctypes.c_int
    lib.sd_decode_step.argtypes = [ctypes.POINTER(DecodeArgs), ctypes.c_void_p]
    lib.sd_forward_launches.restype = ctypes.c_int
    lib.sd_forward_launches.argtypes = [sp]
    lib.sd_backward_launches.restype = ctypes.c_int
    lib.sd_backward_launches.argtypes = [sp]
    lib.sd_panel_info.restype = ctypes.c_int
    lib.sd_panel_info.argtypes = [sp, ctypes.c_int, ctypes.c_char_p,
                                  ctypes.POINTER(ctypes.c_size_t), ctypes.POINTER(ctypes.c_size_t)]
    lib.sd_conv4_backward_scratch_bytes.restype = ctypes.c_size_t
    lib.sd_conv4_backward_scratch_bytes.argtypes = [ctypes.c_int32] * 3
    lib.sd_kda_gate_backward_scratch_bytes.restype = ctypes.c_size_t
    lib.sd_kda_gate_backward_scratch_bytes.argtypes = [ctypes.c_int64, ctypes.c_int32, ctypes.c_int32]
    lib.sd_norm_gate_backward_scratch_bytes.restype = ctypes.c_size_t
    lib.sd_norm_gate_backward_scratch_bytes.argtypes = [ctypes.c_int64, ctypes.c_int32]
    lib.sd_add_rmsnorm_backward_scratch_bytes.restype = ctypes.c_size_t
    lib.sd_add_rmsnorm_backward_scratch_bytes.argtypes = [ctypes.c_int64, ctypes.c_int32]
    for name, struct in (("sd_predictor_forward", PredictorForwardArgs), ("sd_predictor_backward", PredictorBackwardArgs),
                         ("sd_mixer_decode_step", MixerDecodeArgs), ("sd_add_rmsnorm", AddRmsnormArgs),
                         ("sd_swiglu", SwigluArgs), ("sd_swiglu_backward", SwigluArgs),
                         ("sd_add_rmsnorm_backward", AddRmsnormBackwardArgs), ("sd_pack_rows", PackRowsArgs),
                         ("sd_cross_entropy_forward", CrossEntropyArgs), ("sd_cross_entropy_backward", CrossEntropyArgs),
                         ("sd_gemv", GemvArgs),
                         ("sd_conv4_silu_forward", Conv4ForwardArgs), ("sd_conv4_silu_backward", Conv4BackwardArgs),
                         ("sd_kda_gate_forward", KdaGateArgs), ("sd_kda_gate_backward", KdaGateArgs),
                         ("sd_norm_gate_forward", NormGateArgs), ("sd_norm_gate_backward", NormGateArgs)):
        getattr(lib, name).restype = ctypes.c_int
        getattr(lib, name).argtypes = [ctypes.POINTER(struct), ctypes.c_void_p]
    lib.sd_device_fault.restype = ctypes.c_int
    lib.sd_device_fault.argtypes = []
    lib.sd_device_fault_clear.restype = ctypes.c_int
    lib.sd_device_fault_clear.argtypes = []
    lib.sd_panel_kind.restype = ctypes.c_int
    lib.sd_panel_kind.argtypes = [sp, ctypes.c_int, ctypes.c_char_p]
    lib.sd_status_string.restype = ctypes.c_char_p
    lib.sd_status_string.argtypes = [ctypes.c_int]
    lib.sd_version.restype = ctypes.c_int
    lib.sd_chunk_tokens.restype = ctypes.c_int
    return lib


def check_device_fault() -> None:
    """Read the device fault word (this waits for the device) and raise if a bounded wait inside a
    kernel ran out: the results of that launch are undefined.  The word is cleared on the way out."""
    lib = load()
    word = lib.sd_device_fault()
    if word != 0:
        lib.sd_device_fault_clear()
        raise RuntimeError(f"solvedelta_b200: device fault word {word} (a bounded wait inside a kernel ran out; "
                           "the results of that launch are undefined)")


def check(status: int) -> None:
    if status != 0:
        msg = load().sd_status_string(status).decode()
        raise RuntimeError(f"solvedelta_b200: {msg} (status {status})")
