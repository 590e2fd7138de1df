"""The chunk algebra the CUDA kernels implement equals the token recurrence.

Checks tests/chunk_model.py (the stage-by-stage restatement of the CUDA
pipeline) against the FP64 CPU checker on the committed golden inputs, for
several chunk lengths including ones that leave a ragged tail.
"""
import numpy as np
import pytest
import torch

from oracle import solvedelta_oracle as orc
from tests.chunk_model import Model
from tests.helpers import golden_inputs, golden_state, load_golden, rel_l2

CASES = [("seed7_dense", 4), ("seed7_dense", 16), ("benchlike_r16_state", 16),
         ("benchlike_r32_t150_state", 64), ("benchlike_r32_t150_state", 32),
         ("seed7_zero_geometry", 4)]


def _model_inputs(g):
    u, h, q, keys, values, decay, erase, write, gamma = golden_inputs(g)
    B, T, H, r = u.shape
    t = lambda x: torch.from_numpy(np.ascontiguousarray(x))
    logit = lambda p: np.log(p) - np.log1p(-p)
    gam = gamma if gamma.ndim == 3 else np.broadcast_to(gamma.reshape(1, 1, H), (B, T, H))
    return dict(u=t(u), h=t(h), q=t(q), k=t(keys[:, :, :, 0]), v=t(values[:, :, :, 0]), g=t(decay),
                erase_raw=t(logit(erase[:, :, :, 0])), write_raw=t(logit(write[:, :, :, 0])),
                gamma=t(gam))


@pytest.mark.parametrize("name,chunk", CASES)
def test_chunk_forward_and_vjp_equal_token_recurrence(name, chunk):
    g = load_golden(name)
    inp = _model_inputs(g)
    st = golden_state(g)
    C0 = None if st is None else torch.from_numpy(st[0])
    S0 = None if st is None else torch.from_numpy(st[1])
    model = Model(chunk=chunk)
    y, C_T, S_T, saved = model.forward(inp, C0, S0)
    assert rel_l2(y.numpy(), g["out"]) < 1e-10
    assert rel_l2(C_T.numpy(), g["C_T"]) < 1e-10 or np.abs(g["C_T"]).max() == 0
    assert rel_l2(S_T.numpy(), g["S_T"]) < 1e-10
    grads, _ = model.backward(inp, saved, torch.from_numpy(g["dy"]),
                              torch.from_numpy(g["dC_T"]), torch.from_numpy(g["dS_T"]))
    ref = orc.backward(*golden_inputs(g), g["dy"], dC_T=g["dC_T"], dS_T=g["dS_T"], initial_state=st)
    erase, write = g["in_erase"][:, :, :, 0], g["in_write"][:, :, :, 0]
    expect = dict(u=ref["u"], h=ref["h"], q=ref["q"], k=ref["keys"], v=ref["values"], g=ref["log_decay"],
                  erase_raw=ref["erase"] * erase * (1 - erase), write_raw=ref["write"] * write * (1 - write),
                  gamma=ref["geometry_write"])
    if st is not None:
        expect["C0"], expect["S0"] = ref["C0"], ref["S0"]
    for key, val in expect.items():
        assert rel_l2(grads[key].numpy(), val) < 1e-9, key
