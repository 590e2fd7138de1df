"""Mixer glue kernels and the SolveDelta mixer module on the GPU vs the FP64
numpy checker (oracle/mixer_oracle.py, pinned to upstream vectors in
tests/test_mixer_oracle.py).

Cases follow upstream tests/model/test_modeling_solvedelta.py: projection
layout (:321-341), forward/backward through the mixer (:343-420), state
continuation across a split (:423-470).

The checker sees exactly the numbers the GPU sees: inputs and weights rounded
to the dtype the CUDA path reads, and the activations stored between two
kernels rounded to BF16 at the same points.  Tolerance: max relative error (max|a-b| / max|b|) <= 2e-2 on
outputs and gradients, 1e-3 on FP32 operator states.
"""
import numpy as np
import pytest
import torch

from oracle import mixer_oracle as mo
from solvedelta_b200 import (SolveDelta, SolveDeltaConfig, SolveDeltaLayerState, SolveDeltaState, conv4_silu,
                             kda_decay_gate, rms_norm_gated)
from tests.helpers import max_rel, rel_l2
from tests.mixer_helpers import golden_config, golden_params, load_mixer_golden

pytestmark = pytest.mark.gpu

TOL = 2e-2
STATE_TOL = 1e-3


def _np(t):
    return t.detach().double().cpu().numpy()


def _bf16(x):
    return torch.as_tensor(np.asarray(x)).to(torch.bfloat16)


@pytest.mark.parametrize("B,T,D,stateful", [(2, 37, 96, True), (1, 1, 64, True), (3, 130, 328, False),
                                            (2, 257, 1024, True)])
def test_conv4_silu_matches_checker(B, T, D, stateful):
    gen = torch.Generator().manual_seed(B * 1000 + T)
    wide = torch.randn(B, T, D + 24, generator=gen).to(torch.bfloat16)  # x is a strided view of a wider row
    w = (0.5 * torch.randn(D, 4, generator=gen)).float()
    s0 = torch.randn(B, D, 3, generator=gen).to(torch.bfloat16) if stateful else None
    dy = torch.randn(B, T, D, generator=gen).to(torch.bfloat16)
    wide_g = wide.cuda().requires_grad_()
    xg = wide_g[..., 8:8 + D]
    wg = w.cuda().requires_grad_()
    sg = None if s0 is None else s0.cuda().requires_grad_()
    y, fin = conv4_silu(xg, wg, sg, return_final_state=True)
    (y.float() * dy.cuda().float()).sum().backward()
    yo, fo, saved = mo.conv4_silu_forward(_np(wide[..., 8:8 + D]), _np(w), None if s0 is None else _np(s0))
    dxo, dwo, dso = mo.conv4_silu_backward(_np(dy), _np(w), saved)
    assert max_rel(_np(y), yo) <= TOL
    assert np.array_equal(_np(fin), fo)  # the state is a copy of BF16 inputs
    dx = _np(wide_g.grad)
    assert np.all(dx[..., :8] == 0) and np.all(dx[..., 8 + D:] == 0)
    assert max_rel(dx[..., 8:8 + D], dxo) <= TOL
    assert max_rel(_np(wg.grad), dwo) <= TOL
    if stateful:
        assert max_rel(_np(sg.grad), dso) <= TOL


def _conv_masks(B, T, kind, gen):
    valid = torch.ones(B, T, dtype=torch.bool)
    reset = torch.zeros(B, T, dtype=torch.bool)
    if kind == "left_padding":           # rows open with runs of padding longer than a tile
        for b in range(B):
            valid[b, :min(T - 1, 70 + 9 * b)] = False
        reset[:, 1] = True               # a reset on a padded token is ignored
    elif kind == "sparse":               # few valid tokens, far apart: windows reach across tiles
        valid[:] = torch.rand(B, T, generator=gen) < 0.04
        reset[:] = torch.rand(B, T, generator=gen) < 0.01
    elif kind == "mixed":
        valid[:] = torch.rand(B, T, generator=gen) < 0.8
        reset[:] = torch.rand(B, T, generator=gen) < 0.05
        valid[0, :] = False              # a row without valid tokens keeps its state
        reset[1, 0] = True
        valid[1, 0] = True
        if B > 2:
            valid[2, -5:] = False
    return valid, reset


@pytest.mark.parametrize("B,T,D,stateful,kind", [(3, 200, 96, True, "left_padding"), (2, 300, 70, True, "sparse"),
                                                 (3, 150, 328, True, "mixed"), (3, 131, 64, False, "mixed"),
                                                 (2, 5, 32, True, "mixed")])
def test_masked_conv4_silu_matches_checker(B, T, D, stateful, kind):
    """Masks and resets inside the conv kernels (no repacking, no host synchronisation): output, final
    state and all gradients against the masked token loop of the checker."""
    gen = torch.Generator().manual_seed(B * 1000 + T)
    valid, reset = _conv_masks(B, T, kind, gen)
    wide = torch.randn(B, T, D + 24, generator=gen).to(torch.bfloat16)
    w = (0.5 * torch.randn(D, 4, generator=gen)).float()
    s0 = torch.randn(B, D, 3, generator=gen).to(torch.bfloat16) if stateful else None
    dy = torch.randn(B, T, D, generator=gen).to(torch.bfloat16)
    wide_g = wide.cuda().requires_grad_()
    wg = w.cuda().requires_grad_()
    sg = None if s0 is None else s0.cuda().requires_grad_()
    valid_g, reset_g, dy_g = valid.cuda(), reset.cuda(), dy.cuda()
    torch.cuda.synchronize()
    torch.cuda.set_sync_debug_mode("error")
    try:
        y, fin = conv4_silu(wide_g[..., 8:8 + D], wg, sg, return_final_state=True, valid_mask=valid_g,
                            reset_mask=reset_g)
        (y.float() * dy_g.float()).sum().backward()
    finally:
        torch.cuda.set_sync_debug_mode("default")
    yo, fo, saved = mo.conv4_silu_masked_forward(_np(wide[..., 8:8 + D]), _np(w), None if s0 is None else _np(s0),
                                                 valid.numpy(), reset.numpy())
    dxo, dwo, dso = mo.conv4_silu_masked_backward(np.where(valid.numpy()[..., None], _np(dy), 0.0), _np(w), saved)
    assert max_rel(_np(y), yo) <= TOL
    assert np.all(_np(y)[~valid.numpy()] == 0)
    assert np.array_equal(_np(fin), fo)
    dx = _np(wide_g.grad)[..., 8:8 + D]
    assert max_rel(dx, dxo) <= TOL
    assert np.all(dx[~valid.numpy()] == 0)
    assert max_rel(_np(wg.grad), dwo) <= TOL
    if stateful:
        assert max_rel(_np(sg.grad), dso) <= TOL


@pytest.mark.parametrize("shape", [(2, 19, 2, 16), (1, 130, 4, 64), (3, 64, 8, 128), (1, 70, 16, 128)])
def test_kda_decay_gate_matches_checker(shape):
    gen = torch.Generator().manual_seed(sum(shape))
    H, r = shape[-2:]
    raw = (2.0 * torch.randn(*shape, generator=gen)).to(torch.bfloat16)
    log_rate = torch.empty(H).uniform_(0.0, 2.5, generator=gen)
    bias = torch.randn(H, r, generator=gen)
    dout = torch.randn(*shape, generator=gen)
    rg, ag, bg = raw.cuda().requires_grad_(), log_rate.cuda().requires_grad_(), bias.cuda().requires_grad_()
    out = kda_decay_gate(rg, ag, bg)
    assert out.dtype == torch.float32
    (out * dout.cuda()).sum().backward()
    oo, saved = mo.kda_gate_forward(_np(raw), _np(log_rate), _np(bias))
    draw, dA, db = mo.kda_gate_backward(_np(dout), saved)
    assert max_rel(_np(out), oo) <= 1e-5
    assert (out <= 0).all()
    assert max_rel(_np(rg.grad), draw) <= TOL  # BF16 gradient
    assert max_rel(_np(ag.grad), dA) <= 1e-4
    assert max_rel(_np(bg.grad), db) <= 1e-4


@pytest.mark.parametrize("shape", [(2, 19, 2, 16), (1, 130, 4, 64), (3, 64, 8, 128), (2, 5, 3, 40)])
def test_rms_norm_gated_matches_checker(shape):
    gen = torch.Generator().manual_seed(sum(shape) + 1)
    V = shape[-1]
    x = torch.randn(*shape, generator=gen).to(torch.bfloat16)
    gate = (2.0 * torch.randn(*shape, generator=gen)).to(torch.bfloat16)
    w = 1.0 + 0.3 * torch.randn(V, generator=gen)
    dy = torch.randn(*shape, generator=gen).to(torch.bfloat16)
    xg, gg, wg = x.cuda().requires_grad_(), gate.cuda().requires_grad_(), w.cuda().requires_grad_()
    y = rms_norm_gated(xg, gg, wg, 1e-6)
    (y.float() * dy.cuda().float()).sum().backward()
    yo, saved = mo.norm_gate_forward(_np(x), _np(gate), _np(w), 1e-6)
    dxo, dgo, dwo = mo.norm_gate_backward(_np(dy), _np(w), saved)
    assert max_rel(_np(y), yo) <= TOL
    assert max_rel(_np(xg.grad), dxo) <= TOL
    assert max_rel(_np(gg.grad), dgo) <= TOL
    assert max_rel(_np(wg.grad), dwo) <= 1e-3


@pytest.mark.parametrize("shape,out_features,bias", [((2, 19, 2, 16), 24, True), ((1, 130, 8, 128), 256, False)])
def test_norm_followed_by_linear_recomputes_the_normalised_panel(shape, out_features, bias):
    """The fused owner (causallsso/ops/norm_gate.py:46-159) against the checker's norm chained with an FP64
    linear, and nothing of the size of the normalised panel is kept for the reverse pass."""
    from solvedelta_b200 import rms_norm_gated_linear

    gen = torch.Generator().manual_seed(sum(shape) + out_features)
    H, V = shape[-2:]
    x = torch.randn(*shape, generator=gen).to(torch.bfloat16)
    gate = (2.0 * torch.randn(*shape, generator=gen)).to(torch.bfloat16)
    w = 1.0 + 0.3 * torch.randn(V, generator=gen)
    W = (torch.randn(out_features, H * V, generator=gen) / (H * V) ** 0.5).to(torch.bfloat16)
    b = torch.randn(out_features, generator=gen).to(torch.bfloat16) if bias else None
    dout = torch.randn(*shape[:-2], out_features, generator=gen).to(torch.bfloat16)
    xg, gg, wg = x.cuda().requires_grad_(), gate.cuda().requires_grad_(), w.cuda().requires_grad_()
    Wg = W.cuda().requires_grad_()
    bg = None if b is None else b.cuda().requires_grad_()
    out = rms_norm_gated_linear(xg, gg, wg, Wg, bg, 1e-6)
    saved = [t for t in out.grad_fn.saved_tensors]
    assert all(t.shape != torch.Size(shape) or t.data_ptr() in (xg.data_ptr(), gg.data_ptr()) for t in saved)
    (out.float() * dout.cuda().float()).sum().backward()
    yo, norm_saved = mo.norm_gate_forward(_np(x), _np(gate), _np(w), 1e-6)
    y2 = yo.reshape(-1, H * V)
    oo = y2 @ _np(W).T + (0.0 if b is None else _np(b))
    d2 = _np(dout).reshape(-1, out_features)
    dxo, dgo, dwo = mo.norm_gate_backward((d2 @ _np(W)).reshape(shape), _np(w), norm_saved)
    assert max_rel(_np(out).reshape(-1, out_features), oo) <= TOL
    assert max_rel(_np(xg.grad), dxo) <= TOL
    assert max_rel(_np(gg.grad), dgo) <= TOL
    assert max_rel(_np(wg.grad), dwo) <= 5e-3
    assert max_rel(_np(Wg.grad), d2.T @ y2) <= TOL
    if b is not None:
        assert max_rel(_np(bg.grad), d2.sum(0)) <= TOL


# ------------------------------------------------------------------ module

LINEAR_WEIGHTS = ("in_proj.weight", "in_proj.bias", "output_proj.weight", "output_proj.bias", "decay_proj.weight",
                  "output_gate_proj.weight", "output_gate_proj.bias")


def _module_and_checker(cfg, params):
    """GPU module holding `params`; checker holding the same numbers as the GPU reads them
    (linear weights in BF16, conv / gate / norm parameters in FP32)."""
    config = SolveDeltaConfig(hidden_size=cfg["hidden_size"], num_heads=cfg["num_heads"],
                              head_k_dim=cfg["head_k_dim"], head_v_dim=cfg["head_v_dim"],
                              use_short_conv=cfg.get("use_short_conv", True), bias=cfg.get("bias", False),
                              norm_eps=cfg.get("norm_eps", 1e-6))
    module = SolveDelta(config)
    seen = {}
    with torch.no_grad():
        for name, param in module.named_parameters():
            value = torch.as_tensor(np.asarray(params[name])).float()
            if name in LINEAR_WEIGHTS:
                value = value.to(torch.bfloat16).float()
            param.copy_(value.reshape(param.shape))
            seen[name] = _np(param)
    assert set(seen) == set(params)
    module = module.cuda()
    bf16_round = lambda z: torch.as_tensor(z).to(torch.bfloat16).double().numpy()
    checker = mo.MixerOracle(seen, hidden_size=config.hidden_size, num_heads=config.num_heads,
                             head_k_dim=config.resolved_head_k_dim, head_v_dim=config.resolved_head_v_dim,
                             use_short_conv=config.use_short_conv, norm_eps=config.norm_eps,
                             activation_rounding=bf16_round)
    return module, checker


def _compare_grads(module, pgrads, tol=TOL):
    for name, param in module.named_parameters():
        assert param.grad is not None, name
        ref = pgrads[name]
        got = _np(param.grad).reshape(ref.shape)
        assert np.isfinite(got).all(), name
        assert max_rel(got, ref) <= tol, (name, max_rel(got, ref))


OPERANDS = ("u", "h", "q", "keys", "values", "log_decay", "erase_raw", "write_raw", "geometry_write")


class _OperatorSpy:
    """Stands in for ``solvedelta_native`` at the module-level name the mixer calls
    (the call site upstream's tests patch too) and records the gradient autograd
    delivers to every operand and initial state."""

    def __init__(self, monkeypatch):
        import solvedelta_b200.model as model_module

        self.grads = {}
        self.real = model_module.solvedelta_native
        monkeypatch.setattr(model_module, "solvedelta_native", self)

    def __call__(self, *operands, initial_state=None, **kw):
        def keep(name):
            return lambda grad: self.grads.__setitem__(name, grad.detach().clone())

        for name, tensor in zip(OPERANDS, operands):
            if tensor.requires_grad:
                tensor.register_hook(keep(name))
        if initial_state is not None:
            for name, tensor in zip(("C0", "S0"), initial_state):
                if tensor.requires_grad:
                    tensor.register_hook(keep(name))
        return self.real(*operands, initial_state=initial_state, **kw)

    def numpy_grads(self, shapes):
        out = {}
        for name, grad in self.grads.items():
            g = _np(grad)
            out[name] = g.reshape(shapes[name]) if name in shapes else g
        return out


def _check_backward_in_two_steps(module, checker, spy, xg, dout, state_cotangents=None, state_grads=None):
    """(1) The operator's VJP inside the module against the checker's, at the operator
    tolerance.  (2) The glue's adjoint alone: the checker chains the gradients the GPU
    operator produced through its own FP64 glue and must reproduce x.grad and every
    parameter gradient.  (Compared end to end, sums over all tokens such as the decay
    rate gradient amplify the operator's admissible 2e-2 error by their cancellation.)"""
    kw = state_cotangents or {}
    dx_ref, _, _, _ = checker.backward(_np(dout), **kw)
    ref = checker.operator_grads
    c = checker.cache
    shapes = {"u": c["u"].shape, "h": c["u"].shape, "q": c["u"].shape, "keys": c["u"].shape,
              "values": c["v"].shape, "log_decay": c["u"].shape, "erase_raw": c["u"].shape,
              "write_raw": c["v"].shape, "geometry_write": c["gamma"].shape}
    got = spy.numpy_grads(shapes)
    for name in OPERANDS:
        assert max_rel(got[name], ref[name]) <= TOL, (name, max_rel(got[name], ref[name]))
    dx, pg, dconv0, _ = checker.backward(_np(dout), operator_grads=got, **{k: v for k, v in kw.items()
                                                                            if k == "dconv_T"})
    assert max_rel(_np(xg.grad), dx) <= TOL
    _compare_grads(module, pg)
    return dconv0


@pytest.mark.parametrize("name", ["mixer_small", "mixer_noconv_bias"])
def test_mixer_module_matches_checker_on_upstream_parameters(name, monkeypatch):
    g = load_mixer_golden(name)
    module, checker = _module_and_checker(golden_config(g), golden_params(g))
    spy = _OperatorSpy(monkeypatch)
    x = _bf16(g["in_x"])
    dout = _bf16(g["dout"])
    xg = x.cuda().requires_grad_()
    out = module(xg)
    assert out.dtype == torch.bfloat16 and out.shape == x.shape
    (out.float() * dout.cuda().float()).sum().backward()
    oo, _, _ = checker.forward(_np(x))
    assert max_rel(_np(out), oo) <= TOL
    # The FP64 upstream output itself is within BF16 weight rounding of ours.
    assert rel_l2(_np(out), g["out"]) <= 5e-2
    _check_backward_in_two_steps(module, checker, spy, xg, dout)


def test_mixer_module_state_continuation(monkeypatch):
    g = load_mixer_golden("mixer_small_state")
    module, checker = _module_and_checker(golden_config(g), golden_params(g))
    spy = _OperatorSpy(monkeypatch)
    x, dout = _bf16(g["in_x"]), _bf16(g["dout"])
    conv0 = _bf16(g["in_conv0"])
    C0, S0 = torch.as_tensor(g["in_C0"]).float(), torch.as_tensor(g["in_S0"]).float()
    dC, dS = torch.as_tensor(g["dC_T"]).float(), torch.as_tensor(g["dS_T"]).float()
    xg = x.cuda().requires_grad_()
    c0g, s0g, cvg = C0.cuda().requires_grad_(), S0.cuda().requires_grad_(), conv0.cuda().requires_grad_()
    out, fin = module(xg, initial_state=SolveDeltaLayerState(SolveDeltaState(c0g, s0g), cvg),
                      return_final_state=True)
    loss = ((out.float() * dout.cuda().float()).sum() + (fin.operator.predictor * dC.cuda()).sum()
            + (fin.operator.S * dS.cuda()).sum())
    loss.backward()
    oo, fo, conv_T = checker.forward(_np(x), conv_state=_np(conv0), operator_state=(_np(C0), _np(S0)))
    assert max_rel(_np(out), oo) <= TOL
    assert max_rel(_np(fin.operator.predictor), fo[0]) <= 5e-3  # BF16 activations feed the FP32 state
    assert max_rel(_np(fin.operator.S), fo[1]) <= 5e-3
    assert max_rel(_np(fin.conv), conv_T) <= 1e-2               # BF16 copy of the projection row
    dconv0 = _check_backward_in_two_steps(module, checker, spy, xg, dout,
                                          state_cotangents=dict(dC_T=_np(dC), dS_T=_np(dS)))
    ref = checker.backward(_np(dout), dC_T=_np(dC), dS_T=_np(dS))[3]
    assert max_rel(_np(c0g.grad), ref[0]) <= TOL
    assert max_rel(_np(s0g.grad), ref[1]) <= TOL
    assert max_rel(_np(cvg.grad), dconv0) <= TOL

    # Split continuation: running [0,t) then [t,T) with the carried state equals one pass.
    with torch.no_grad():
        state0 = SolveDeltaLayerState(SolveDeltaState(C0.cuda(), S0.cuda()), conv0.cuda())
        whole, fin_whole = module(x.cuda(), initial_state=state0, return_final_state=True)
        a, mid = module(x.cuda()[:, :3], initial_state=state0, return_final_state=True)
        b, fin_split = module(x.cuda()[:, 3:], initial_state=mid, return_final_state=True)
    assert max_rel(_np(torch.cat([a, b], 1)), _np(whole)) <= TOL
    assert torch.equal(fin_split.conv, fin_whole.conv)
    assert max_rel(_np(fin_split.operator.S), _np(fin_whole.operator.S)) <= 5e-3


def test_mixer_module_masks_and_resets(monkeypatch):
    """valid / reset masks with carried conv and operator states (upstream mask semantics,
    causallsso/model.py:146-164 and reference.py:156-227), against the masked checker."""
    g = load_mixer_golden("mixer_masks_state")
    module, checker = _module_and_checker(golden_config(g), golden_params(g))
    x, dout = _bf16(g["in_x"]), _bf16(g["dout"])
    conv0 = _bf16(g["in_conv0"])
    C0, S0 = torch.as_tensor(g["in_C0"]).float(), torch.as_tensor(g["in_S0"]).float()
    dC, dS = torch.as_tensor(g["dC_T"]).float(), torch.as_tensor(g["dS_T"]).float()
    valid, reset = torch.as_tensor(g["valid_mask"]), torch.as_tensor(g["reset_mask"])
    xg = x.cuda().requires_grad_()
    c0g, s0g, cvg = C0.cuda().requires_grad_(), S0.cuda().requires_grad_(), conv0.cuda().requires_grad_()
    valid_g, reset_g, dout_g, dC_g, dS_g = valid.cuda(), reset.cuda(), dout.cuda(), dC.cuda(), dS.cuda()
    torch.cuda.synchronize()
    torch.cuda.set_sync_debug_mode("error")   # masks never leave the device: the masked mixer does not synchronise
    try:
        out, fin = module(xg, initial_state=SolveDeltaLayerState(SolveDeltaState(c0g, s0g), cvg),
                          valid_mask=valid_g, reset_mask=reset_g, return_final_state=True)
        loss = ((out.float() * dout_g.float()).sum() + (fin.operator.predictor * dC_g).sum()
                + (fin.operator.S * dS_g).sum())
        loss.backward()
    finally:
        torch.cuda.set_sync_debug_mode("default")
    oo, fo, conv_T = checker.forward(_np(x), conv_state=_np(conv0), operator_state=(_np(C0), _np(S0)),
                                     valid_mask=g["valid_mask"], reset_mask=g["reset_mask"])
    assert max_rel(_np(out), oo) <= TOL
    # invalid tokens: the operator and the conv contribute nothing, the output is the bias-free projection of zero
    assert float(out.detach()[~valid.cuda()].abs().max()) == 0.0
    assert max_rel(_np(fin.operator.predictor), fo[0]) <= 5e-3
    assert max_rel(_np(fin.operator.S), fo[1]) <= 5e-3
    assert max_rel(_np(fin.conv), conv_T) <= 1e-2
    # a row without valid tokens hands its states through untouched
    assert torch.equal(fin.conv[2], conv0.cuda()[2])
    assert torch.equal(fin.operator.S[2], S0.cuda()[2])
    dx, pg, dconv0, (dC0, dS0) = checker.backward(_np(dout), dC_T=_np(dC), dS_T=_np(dS))
    # end-to-end gradients of the tensors whose sums do not cancel: input, states
    assert rel_l2(_np(xg.grad), dx) <= 5e-2
    assert max_rel(_np(c0g.grad), dC0) <= TOL
    assert max_rel(_np(s0g.grad), dS0) <= TOL
    assert rel_l2(_np(cvg.grad), dconv0) <= 5e-2
    assert float(xg.grad[2].abs().max()) == 0.0
    for name in ("in_proj.weight", "output_proj.weight", "conv_weight", "output_norm.weight"):
        got = _np(dict(module.named_parameters())[name].grad).reshape(pg[name].shape)
        assert rel_l2(got, pg[name]) <= 5e-2, (name, rel_l2(got, pg[name]))


def test_mixer_module_tiny_configuration(monkeypatch):
    """The upstream CPU-runnable configuration: hidden 256, 4 heads, 64/64, B=2, T=128."""
    torch.manual_seed(5)
    config = SolveDeltaConfig(hidden_size=256, num_heads=4, head_k_dim=64, head_v_dim=64)
    module = SolveDelta(config)
    assert module.projection_sizes == (256, 256, 256, 256, 256, 256, 256, 4, 64, 64)
    params = {n: _np(p) for n, p in module.named_parameters()}
    module, checker = _module_and_checker(dict(hidden_size=256, num_heads=4, head_k_dim=64, head_v_dim=64), params)
    spy = _OperatorSpy(monkeypatch)
    gen = torch.Generator().manual_seed(11)
    x = torch.randn(2, 128, 256, generator=gen).to(torch.bfloat16)
    dout = torch.randn(2, 128, 256, generator=gen).to(torch.bfloat16)
    xg = x.cuda().requires_grad_()
    out = module(xg)
    (out.float() * dout.cuda().float()).sum().backward()
    oo, _, _ = checker.forward(_np(x))
    assert max_rel(_np(out), oo) <= TOL
    _check_backward_in_two_steps(module, checker, spy, xg, dout)


def test_mixer_module_rejects_cpu_inputs():
    module = SolveDelta(SolveDeltaConfig(hidden_size=64, num_heads=2, head_k_dim=16, head_v_dim=16)).cuda()
    with pytest.raises(TypeError):
        module(torch.zeros(1, 4, 64))
    with pytest.raises(ValueError):
        module(torch.zeros(1, 4, 32, dtype=torch.bfloat16, device="cuda"))


def test_inference_glue_kernels_match_pytorch():
    """The two inference-only kernels of the block: residual add + RMSNorm, and SiLU(gate) * value."""
    from solvedelta_b200.mixer_ops import add_rmsnorm, swiglu

    gen = torch.Generator().manual_seed(3)
    for rows, D in ((5, 1024), (3, 200), (2, 4100)):
        x = torch.randn(rows, D, generator=gen).to(torch.bfloat16).cuda()
        d = torch.randn(rows, D, generator=gen).to(torch.bfloat16).cuda()
        w = (1.0 + 0.2 * torch.randn(D, generator=gen)).cuda()
        total, normed = add_rmsnorm(x, d, w, 1e-6)
        want_sum = x + d
        assert torch.equal(total, want_sum)
        s = want_sum.float()
        want = s * torch.rsqrt(s.pow(2).mean(-1, keepdim=True) + 1e-6) * w
        assert float((normed.float() - want).abs().max()) <= 1e-2 * float(want.abs().max())
        gv = torch.randn(rows, 2 * D, generator=gen).to(torch.bfloat16).cuda()
        out = swiglu(gv)
        g, v = gv.float().chunk(2, dim=-1)
        want = torch.nn.functional.silu(g) * v
        assert out.shape == (rows, D)
        assert float((out.float() - want).abs().max()) <= 1e-2 * float(want.abs().max())


@pytest.mark.parametrize("rows,D,with_delta", [(37, 256, True), (64, 1024, True), (19, 768, False), (5, 2048, True)])
def test_add_rmsnorm_reverse_matches_float64_autograd(rows, D, with_delta):
    """Residual add + RMSNorm with its one reverse kernel: both outputs, the gradient x and delta share, and the
    weight gradient against FP64 autograd of the same formula (the sum rounded to BF16 as the kernel stores it)."""
    from solvedelta_b200.mixer_ops import add_rmsnorm

    gen = torch.Generator().manual_seed(rows + D)
    x = torch.randn(rows, D, generator=gen).to(torch.bfloat16)
    d = torch.randn(rows, D, generator=gen).to(torch.bfloat16) if with_delta else None
    w = (1.0 + 0.3 * torch.randn(D, generator=gen))
    ds = torch.randn(rows, D, generator=gen).to(torch.bfloat16)
    dn = torch.randn(rows, D, generator=gen).to(torch.bfloat16)
    xg, wg = x.cuda().requires_grad_(), w.cuda().requires_grad_()
    dg = d.cuda().requires_grad_() if with_delta else None
    total, normed = add_rmsnorm(xg, dg, wg, 1e-6)
    (total.float() * ds.cuda().float()).sum().backward(retain_graph=True)
    (normed.float() * dn.cuda().float()).sum().backward()
    # FP64 reference
    xr, wr = x.double().requires_grad_(), w.double().requires_grad_()
    dr = d.double().requires_grad_() if with_delta else None
    s = xr + dr if with_delta else xr
    s = s + (s.detach().to(torch.bfloat16).double() - s.detach())   # the stored sum, identity derivative
    n = s * torch.rsqrt(s.pow(2).mean(-1, keepdim=True) + 1e-6) * wr
    ((s * ds.double()).sum() + (n * dn.double()).sum()).backward()
    assert torch.equal(total.detach().cpu().double(), s.detach())
    assert max_rel(_np(normed), n.detach().numpy()) <= TOL
    assert max_rel(_np(xg.grad), xr.grad.numpy()) <= TOL
    if with_delta:
        assert torch.equal(dg.grad, xg.grad)
    assert max_rel(_np(wg.grad), wr.grad.numpy()) <= 1e-3


def test_add_rmsnorm_reverse_refuses_other_widths():
    from solvedelta_b200.mixer_ops import add_rmsnorm

    x = torch.randn(4, 200).to(torch.bfloat16).cuda().requires_grad_()
    with pytest.raises(ValueError):
        add_rmsnorm(x, x.detach(), torch.ones(200, device="cuda"), 1e-6)


@pytest.mark.parametrize("rows,I", [(33, 64), (7, 2816), (5, 100)])
def test_swiglu_reverse_matches_float64_autograd(rows, I):
    from solvedelta_b200.mixer_ops import swiglu

    gen = torch.Generator().manual_seed(rows + I)
    gv = (1.5 * torch.randn(rows, 2 * I, generator=gen)).to(torch.bfloat16)
    do = torch.randn(rows, I, generator=gen).to(torch.bfloat16)
    gg = gv.cuda().requires_grad_()
    out = swiglu(gg)
    (out.float() * do.cuda().float()).sum().backward()
    gr = gv.double().requires_grad_()
    g, v = gr.chunk(2, dim=-1)
    want = torch.nn.functional.silu(g) * v
    (want * do.double()).sum().backward()
    assert max_rel(_np(out), want.detach().numpy()) <= TOL
    assert max_rel(_np(gg.grad), gr.grad.numpy()) <= TOL


def test_pack_rows_writes_the_slices_side_by_side():
    from solvedelta_b200.mixer_ops import pack_rows

    gen = torch.Generator().manual_seed(11)
    widths = (48, 16, 8, 24)
    pieces = [torch.randn(3, 37, w, generator=gen).to(torch.bfloat16).cuda() for w in widths]
    pieces[2] = None
    row = pack_rows(pieces, widths, (3, 37, 128), torch.device("cuda", 0))
    want = torch.zeros(3, 37, 128, dtype=torch.bfloat16, device="cuda")
    start = 0
    for g, w in zip(pieces, widths):
        if g is not None:
            want[..., start:start + w] = g
        start += w
    assert torch.equal(row, want)
    # layouts the kernel does not take are left to the caller
    assert pack_rows([pieces[0][..., :5]], (5,), (3, 37, 8), torch.device("cuda", 0)) is None


@pytest.mark.parametrize("rows,K,N,swiglu_on,with_bias", [(1, 1024, 7488, False, False), (4, 2816, 1024, False, True),
                                                          (2, 1024, 5632, True, False), (3, 64, 24, True, True)])
def test_small_linear_matches_the_library_projection(rows, K, N, swiglu_on, with_bias):
    from solvedelta_b200.mixer_ops import small_linear

    gen = torch.Generator().manual_seed(rows + K + N)
    wide = torch.randn(rows, 1, K + 64, generator=gen).to(torch.bfloat16).cuda()
    x = wide[..., 8:8 + K]                      # a strided view, as a slice of the projection row is
    w = (torch.randn(N, K, generator=gen) / K ** 0.5).to(torch.bfloat16).cuda()
    b = torch.randn(N, generator=gen).to(torch.bfloat16).cuda() if with_bias else None
    with torch.no_grad():
        got = small_linear(x, w, b, swiglu=swiglu_on)
        want = torch.nn.functional.linear(x.float(), w.float(), b.float() if with_bias else None)
        if swiglu_on:
            g, v = want.to(torch.bfloat16).float().chunk(2, dim=-1)
            want = torch.nn.functional.silu(g) * v
    assert got is not None and got.shape == want.shape and got.dtype == torch.bfloat16
    assert float((got.float() - want).abs().max()) <= 1e-2 * float(want.abs().max()) + 1e-3
    with torch.no_grad():   # layouts the kernel does not take are left to the caller
        assert small_linear(torch.zeros(5, K, dtype=torch.bfloat16, device="cuda"), w) is None
        assert small_linear(x.float(), w) is None
    assert small_linear(x.clone().requires_grad_(), w) is None
