"""Pins the FP64 CPU checker (oracle/) to the upstream oracle.

Golden vectors in tests/golden were produced by the upstream
``solvedelta_reference`` + torch.autograd (see tests/golden/make_golden.py).
The known-answer cases restate upstream tests
tests/core/test_rebuild_semantics.py:135-167 (accumulated primal / local dual),
:170-228 (pre-decay residual, right channel gate), :231-249 (frame radius),
:296-316 (zero geometry write reduces to the GDN2 edit) and :319-360
(masks, resets, split/continue).
"""
import numpy as np
import pytest

from oracle import solvedelta_oracle as orc
from tests.helpers import golden_inputs, golden_names, golden_state, load_golden


def _normalize(x):
    return x / np.maximum(np.linalg.norm(x, axis=-1, keepdims=True), 1e-12)


@pytest.mark.parametrize("name", golden_names())
def test_forward_matches_upstream_golden(name):
    g = load_golden(name)
    y, st = orc.forward(*golden_inputs(g), initial_state=golden_state(g),
                        valid_mask=g.get("valid"), reset_mask=g.get("reset"))
    np.testing.assert_allclose(y, g["out"], rtol=2e-12, atol=2e-12)
    np.testing.assert_allclose(st.predictor, g["C_T"], rtol=2e-12, atol=2e-12)
    np.testing.assert_allclose(st.S, g["S_T"], rtol=2e-12, atol=2e-12)


@pytest.mark.parametrize("name", golden_names())
def test_vjp_matches_upstream_autograd(name):
    g = load_golden(name)
    grads = orc.backward(*golden_inputs(g), g["dy"], dC_T=g["dC_T"], dS_T=g["dS_T"],
                         initial_state=golden_state(g), valid_mask=g.get("valid"),
                         reset_mask=g.get("reset"))
    for key in ("u", "h", "q", "log_decay"):
        np.testing.assert_allclose(grads[key], g["grad_" + key], rtol=1e-9, atol=1e-11, err_msg=key)
    for key in ("keys", "values", "erase", "write"):
        np.testing.assert_allclose(grads[key], g["grad_" + key][:, :, :, 0], rtol=1e-9, atol=1e-11, err_msg=key)
    expected_gamma = g["grad_geometry_write"]
    got_gamma = grads["geometry_write"]
    if expected_gamma.ndim < 3:  # per-head parameter: autograd summed over B,T
        got_gamma = got_gamma.sum(axis=(0, 1)).reshape(expected_gamma.shape)
    np.testing.assert_allclose(got_gamma, expected_gamma, rtol=1e-9, atol=1e-11)
    if "grad_C0" in g:
        np.testing.assert_allclose(grads["C0"], g["grad_C0"], rtol=1e-9, atol=1e-11)
        np.testing.assert_allclose(grads["S0"], g["grad_S0"], rtol=1e-9, atol=1e-11)


def test_primal_uses_accumulated_predictor_while_dual_stays_local():
    u = np.array([[[[1.0, 0.0]], [[0.0, 1.0]]]])
    h = np.array([[[[0.0, 1.0]], [[0.0, 0.0]]]])
    q = np.array([[[[1.0, 0.0]], [[1.0, 0.0]]]])
    keys = np.array([[[[[1.0, 0.0]]], [[[0.0, 1.0]]]]])
    values = np.array([0.0, 1.0]).reshape(1, 2, 1, 1, 1)
    log_decay = np.zeros((1, 2, 1, 2))
    y, st = orc.forward(u, h, q, keys, values, log_decay, np.zeros_like(keys),
                        np.ones_like(values), np.ones(1))
    np.testing.assert_allclose(y[:, 1], np.ones_like(y[:, 1]), atol=1e-15)
    np.testing.assert_allclose(st.predictor, np.array([[[[0.0, 0.0], [1.0, 0.0]]]]), atol=1e-15)


def test_forgetting_uses_pre_decay_residual_and_right_channel_gate():
    u = np.array([[[[1.0, 0.0]]]])
    C0 = np.array([[[[2.0, 3.0], [4.0, 1.0]]]])
    h = np.array([[[[2.0, 4.0]]]])
    q = np.array([[[[1.0, 0.0]]]])
    keys = np.array([[[[[1.0, 0.0]]]]])
    values = np.zeros((1, 1, 1, 1, 1))
    log_decay = np.array([np.log(0.25), 0.0]).reshape(1, 1, 1, 2)
    S0 = np.array([[[[5.0], [7.0]]]])
    _, st = orc.forward(u, h, q, keys, values, log_decay, np.zeros_like(keys),
                        np.zeros_like(values), np.array([0.75]), initial_state=(C0, S0))
    retention = np.exp(log_decay[:, 0])  # [1,1,2]
    np.testing.assert_allclose(st.predictor, C0 * retention[..., None, :], atol=1e-15)
    np.testing.assert_allclose(st.S, retention[..., :, None] * S0, atol=1e-15)
    assert not np.allclose(st.predictor, retention[..., :, None] * C0)


def test_frame_radius_bounds_adversarial_residual():
    radius = orc.RELATIVE_FRAME_RADIUS
    direction = _normalize(np.array([1.0, -2.0, 3.0]))
    for sign in (-1.0, 1.0):
        update = sign * 1.0e6 * direction
        scale = radius / np.sqrt(radius**2 + (direction**2).sum() * (update**2).sum())
        den = 1.0 + (scale * update) @ direction
        assert 1.0 - radius < den < 1.0 + radius


def test_zero_geometry_write_reduces_to_gdn2_edit():
    g = load_golden("seed7_zero_geometry")
    args = golden_inputs(g)
    y, st = orc.forward(*args)
    _, _, q, keys, values, decay, erase, write, _ = args
    q, keys = _normalize(q), _normalize(keys)
    B, T, H, r = q.shape
    memory = np.zeros_like(st.S)
    rows = []
    for t in range(T):
        memory = np.exp(decay[:, t])[..., None] * memory
        key = keys[:, t, :, 0]
        erase_key = erase[:, t, :, 0] * key
        value = write[:, t, :, 0] * values[:, t, :, 0]
        prediction = np.einsum("bhrv,bhr->bhv", memory, erase_key)
        memory = memory + key[..., :, None] * (value - prediction)[..., None, :]
        rows.append(np.einsum("bhrv,bhr->bhv", memory, q[:, t]))
    np.testing.assert_allclose(y, np.stack(rows, axis=1), rtol=2e-12, atol=2e-12)
    np.testing.assert_allclose(st.S, memory, rtol=2e-12, atol=2e-12)
    np.testing.assert_allclose(st.predictor, 0.0, atol=0)


def test_masks_resets_and_split_continuation():
    g = load_golden("seed7_masks_resets_state")
    args = golden_inputs(g)
    valid, reset = g["valid"], g["reset"]
    state = golden_state(g)
    y, st = orc.forward(*args, initial_state=state, valid_mask=valid, reset_mask=reset)
    assert np.all(y[~valid] == 0.0)
    split = 4
    left = [a[:, :split] for a in args[:-1]] + [args[-1]]
    right = [a[:, split:] for a in args[:-1]] + [args[-1]]
    yl, sl = orc.forward(*left, initial_state=state, valid_mask=valid[:, :split], reset_mask=reset[:, :split])
    yr, sr = orc.forward(*right, initial_state=sl, valid_mask=valid[:, split:], reset_mask=reset[:, split:])
    np.testing.assert_allclose(np.concatenate([yl, yr], axis=1), y, rtol=2e-12, atol=2e-12)
    np.testing.assert_allclose(sr.predictor, st.predictor, rtol=2e-12, atol=2e-12)
    np.testing.assert_allclose(sr.S, st.S, rtol=2e-12, atol=2e-12)


def test_rejects_multiple_edits():
    g = load_golden("seed7_dense")
    args = golden_inputs(g)
    for i in (3, 4, 6, 7):
        args[i] = np.repeat(args[i], 2, axis=3)
    with pytest.raises(ValueError, match="num_edits=1"):
        orc.forward(*args)
