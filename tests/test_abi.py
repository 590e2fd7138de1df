"""The C-ABI library builds, loads and exports what include/solvedelta_b200.h
declares; host-side argument checks answer without touching a GPU."""
import ctypes
import os
import re

import pytest

from solvedelta_b200 import _lib


@pytest.fixture(scope="module")
def lib():
    _lib.build()
    return _lib.load()


def _declared_functions():
    text = open(_lib.HEADER_PATH).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(sd_[a-z0-9_]+)\s*\(", text)))


def test_header_and_loader_agree():
    assert _declared_functions() == sorted(_lib.EXPORTS)


def test_library_exports_every_declared_symbol(lib):
    for name in _declared_functions():
        assert hasattr(lib, name), name


def test_struct_sizes_match_header():
    # int32 x5, padded to 8 before the first pointer-bearing operand
    assert ctypes.sizeof(_lib.Shape) == 20
    assert ctypes.sizeof(_lib.Operand) == 32
    assert ctypes.sizeof(_lib.ForwardArgs) == 24 + 9 * 32 + 5 * 8 + 4 * 8 + 2 * 8
    assert ctypes.sizeof(_lib.BackwardArgs) == 24 + 10 * 32 + 2 * 8 + 4 * 8 + 11 * 8 + 2 * 8
    assert ctypes.sizeof(_lib.DecodeArgs) == 24 + 9 * 32 + 3 * 8
    # mixer glue: three int32 (padded to 16) + pointers / strides / sizes of 8 bytes each
    assert ctypes.sizeof(_lib.Conv4ForwardArgs) == 16 + 9 * 8
    assert ctypes.sizeof(_lib.Conv4BackwardArgs) == 16 + 13 * 8
    assert ctypes.sizeof(_lib.KdaGateArgs) == 16 + 10 * 8
    assert ctypes.sizeof(_lib.NormGateArgs) == 16 + 10 * 8
    assert ctypes.sizeof(_lib.AddRmsnormArgs) == 16 + 5 * 8
    assert ctypes.sizeof(_lib.AddRmsnormBackwardArgs) == 16 + 8 * 8
    assert ctypes.sizeof(_lib.SwigluArgs) == 16 + 4 * 8
    assert ctypes.sizeof(_lib.RowPiece) == 16
    assert ctypes.sizeof(_lib.CrossEntropyArgs) == 16 + 7 * 8
    assert ctypes.sizeof(_lib.GemvArgs) == 16 + 6 * 8
    assert ctypes.sizeof(_lib.PackRowsArgs) == 16 + 12 * 16 + 8


def test_workspace_queries_scale_with_chunks(lib):
    L = lib.sd_chunk_tokens()
    assert L == 64
    one = _lib.Shape(1, L, 1, 128, 128)
    two = _lib.Shape(1, 2 * L, 1, 128, 128)
    ragged = _lib.Shape(1, L + 1, 1, 128, 128)
    for fn in (lib.sd_saved_bytes, lib.sd_forward_scratch_bytes, lib.sd_backward_scratch_bytes):
        a, b, c = fn(ctypes.byref(one)), fn(ctypes.byref(two)), fn(ctypes.byref(ragged))
        assert a > 0 and b == 2 * a and c == b
    assert lib.sd_saved_bytes(ctypes.byref(_lib.Shape(1, 8, 1, 129, 16))) == 0
    assert lib.sd_saved_bytes(ctypes.byref(_lib.Shape(0, 8, 1, 16, 16))) == 0


def test_argument_errors_are_status_codes(lib):
    assert lib.sd_forward(None, None) == -1
    assert lib.sd_backward(None, None) == -1
    assert lib.sd_decode_step(None, None) == -1
    args = _lib.ForwardArgs()
    args.shape = _lib.Shape(1, 8, 1, 200, 16)
    assert lib.sd_forward(ctypes.byref(args), None) == -2
    args.shape = _lib.Shape(1, 8, 1, 16, 16)
    assert lib.sd_forward(ctypes.byref(args), None) == -1  # null operands
    dec = _lib.DecodeArgs()
    dec.shape = _lib.Shape(1, 2, 1, 16, 16)
    assert lib.sd_decode_step(ctypes.byref(dec), None) == -1  # T must be 1
    assert lib.sd_conv4_silu_forward(None, None) == -1
    assert lib.sd_conv4_silu_backward(None, None) == -1
    assert lib.sd_kda_gate_forward(None, None) == -1
    assert lib.sd_kda_gate_backward(None, None) == -1
    assert lib.sd_norm_gate_forward(None, None) == -1
    assert lib.sd_norm_gate_backward(None, None) == -1
    assert lib.sd_conv4_silu_forward(ctypes.byref(_lib.Conv4ForwardArgs(1, 4, 8)), None) == -1  # null operands
    assert lib.sd_conv4_backward_scratch_bytes(2, 130, 96) >= 2 * 3 * 96 * 4 * 4
    assert lib.sd_kda_gate_backward_scratch_bytes(0, 2, 16) == 0
    assert lib.sd_norm_gate_backward_scratch_bytes(300, 64) >= 2 * 64 * 4
    assert lib.sd_status_string(0) == b"ok"
    assert b"128" in lib.sd_status_string(-2)
    off, size = ctypes.c_size_t(), ctypes.c_size_t()
    shape = _lib.Shape(1, 64, 1, 16, 16)
    assert lib.sd_panel_info(ctypes.byref(shape), 0, b"Delta", ctypes.byref(off), ctypes.byref(size)) == 0
    assert size.value == 64 * 128 * 4
    assert lib.sd_panel_info(ctypes.byref(shape), 0, b"nope", ctypes.byref(off), ctypes.byref(size)) == -1


def test_entry_points_reject_cpu_tensors_like_upstream():
    import torch
    from solvedelta_b200 import solvedelta_native

    u = torch.zeros(1, 4, 1, 8, dtype=torch.bfloat16)
    k = torch.zeros(1, 4, 1, 1, 8, dtype=torch.bfloat16)
    ld = torch.zeros(1, 4, 1, 8)
    gam = torch.zeros(1)
    with pytest.raises(TypeError, match="BF16 CUDA"):
        solvedelta_native(u, u, u, k, k, ld, k, k, gam)
    with pytest.raises(TypeError, match="BF16 CUDA"):
        solvedelta_native(u.float(), u, u, k, k, ld, k, k, gam)


def test_product_package_never_imports_the_checker():
    pkg = os.path.dirname(_lib.__file__)
    for root, _, files in os.walk(pkg):
        for name in files:
            if name.endswith((".py", ".cu", ".cuh", ".h")):
                text = open(os.path.join(root, name)).read()
                assert "oracle" not in text.replace("checker", ""), name
