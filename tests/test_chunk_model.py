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


@pytest.mark.parametrize("scale", [0.4, 3.0, 16.0])
def test_chunk_algebra_is_exact_under_strong_forgetting(scale):
    """Per-token log decays down to -16 (upstream tests/core/test_rebuild_semantics.py:411
    runs its exterior owner at decay_scale 16): the chunk prefix reaches -1000, far past
    what a reciprocal-retention factor could hold.  Per-channel rates span four decades."""
    rng = np.random.default_rng(int(scale * 10))
    B, T, H, r, V = 1, 150, 2, 16, 16
    rate = scale * np.exp(rng.uniform(np.log(1e-3), 0.0, size=(1, 1, H, r)))
    g = -rate * (0.75 + 0.25 * rng.random((B, T, H, r)))
    u, h, q, k = (rng.standard_normal((B, T, H, r)) for _ in range(4))
    v = rng.standard_normal((B, T, H, V))
    er, wr = rng.standard_normal((B, T, H, r)), rng.standard_normal((B, T, H, V))
    gam = 1 / (1 + np.exp(-(rng.standard_normal((B, T, H)) + 1.0)))
    C0, S0 = 0.2 * rng.standard_normal((B, H, r, r)), 0.5 * rng.standard_normal((B, H, r, V))
    dy, dC, dS = rng.standard_normal((B, T, H, V)), rng.standard_normal(C0.shape), rng.standard_normal(S0.shape)
    sig = lambda x: 1 / (1 + np.exp(-x))
    args = (u, h, q, k, v, g, sig(er), sig(wr), gam)
    yo, so = orc.forward(*args, initial_state=(C0, S0))
    ref = orc.backward(*args, dy, dC_T=dC, dS_T=dS, initial_state=(C0, S0))
    t = torch.from_numpy
    inp = dict(u=t(u), h=t(h), q=t(q), k=t(k), v=t(v), g=t(g), erase_raw=t(er), write_raw=t(wr), gamma=t(gam))
    model = Model(chunk=64)
    y, C_T, S_T, saved = model.forward(inp, t(C0), t(S0))
    assert rel_l2(y.numpy(), yo) < 1e-9
    assert rel_l2(C_T.numpy(), so.predictor) < 1e-9
    assert rel_l2(S_T.numpy(), so.S) < 1e-9
    grads, _ = model.backward(inp, saved, t(dy), t(dC), t(dS))
    expect = dict(u=ref["u"], h=ref["h"], q=ref["q"], k=ref["keys"], v=ref["values"], g=ref["log_decay"],
                  erase_raw=ref["erase"] * sig(er) * (1 - sig(er)), write_raw=ref["write"] * sig(wr) * (1 - sig(wr)),
                  gamma=ref["geometry_write"], C0=ref["C0"], S0=ref["S0"])
    for key, val in expect.items():
        assert np.isfinite(grads[key].numpy()).all(), key
        assert rel_l2(grads[key].numpy(), val) < 1e-8, key
