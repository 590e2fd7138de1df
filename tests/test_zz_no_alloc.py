"""sd_forward_static: the forward pass for hosts that must not allocate.

Some callers of this library cannot hand it workspace buffers, because they
are not allowed to call cudaMalloc where the operator runs (all device memory
belongs to their own arena, or a stream capture is in progress).  For them the
library keeps a fixed 32 MiB device array of its own.  This test calls that
entry point through the C ABI several times in a row, on different inputs and
shapes (a narrow, ragged shape comes after a wide one, so that whatever the
wide call left in the shared array lies under the narrow call's panels),
and checks each result against sd_forward with caller-provided buffers.  The
two paths run the same kernels on the same data, so the results must be equal
bit for bit, which is well inside the tolerances of the parity tests.

The file sorts last on purpose: if it fails, a run that stops at the first
failure has already exercised every other test.
"""
import ctypes

import pytest
import torch

from solvedelta_b200 import _lib
from solvedelta_b200.ops import _fill_operands
from tests.gpu_harness import RawRun, make_inputs

pytestmark = pytest.mark.gpu


def _forward_static(dev):
    lib = _lib.load()
    u = dev["u"]
    B, T, H, r = u.shape
    V = dev["values"].shape[-1]
    gam = dev["geometry_write"]
    if gam.ndim != 3:
        gam = gam.reshape(1, 1, H).expand(B, T, H)
    sq = lambda x: x.squeeze(-2)
    tensors = (u, dev["h"], dev["q"], sq(dev["keys"]), sq(dev["values"]), dev["log_decay"],
               sq(dev["erase_raw"]), sq(dev["write_raw"]), gam)
    y = torch.empty(B, T, H, V, dtype=torch.bfloat16, device=u.device)
    C_T = torch.empty(B, H, r, r, dtype=torch.float32, device=u.device)
    S_T = torch.empty(B, H, r, V, dtype=torch.float32, device=u.device)
    args = _lib.ForwardArgs()
    args.shape = _lib.Shape(B, T, H, r, V)
    _fill_operands(args, tensors)
    args.C0, args.S0 = dev["C0"].data_ptr(), dev["S0"].data_ptr()
    args.y, args.C_T, args.S_T = y.data_ptr(), C_T.data_ptr(), S_T.data_ptr()
    # saved / scratch stay NULL: the library uses its own array
    stream = ctypes.c_void_p(torch.cuda.current_stream(u.device).cuda_stream)
    status = lib.sd_forward_static(ctypes.byref(args), stream)
    torch.cuda.synchronize()
    return status, y, C_T, S_T


def test_static_workspace_forward_matches_caller_buffers_twice_in_a_row():
    for seed, (B, T, H, r, V) in ((41, (1, 150, 2, 32, 32)), (43, (1, 300, 1, 128, 128)), (47, (2, 70, 1, 16, 24)),
                                  (41, (1, 150, 2, 32, 32))):
        _, dev = make_inputs(B, T, H, r, V, seed=seed)
        status, y, C_T, S_T = _forward_static(dev)
        assert status == 0, _lib.load().sd_status_string(status)
        ref = RawRun(dev)
        assert torch.equal(y, ref.y)
        assert torch.equal(C_T, ref.C_T)
        assert torch.equal(S_T, ref.S_T)


def test_static_workspace_refuses_oversized_shapes():
    lib = _lib.load()
    _, dev = make_inputs(1, 8, 1, 16, 16, seed=1)
    args = _lib.ForwardArgs()
    args.shape = _lib.Shape(8, 4096, 8, 128, 128)  # 4096 chunk tasks, far beyond the limit
    status = lib.sd_forward_static(ctypes.byref(args), None)
    assert status == -6
    assert b"SD_STATIC_WORKSPACE_BYTES" in lib.sd_status_string(status)
