"""CUDA path vs the FP64 CPU checker, through the public entry points.

Cases follow upstream tests/core/test_rebuild_semantics.py: forward + full VJP
with continuation states (:540-597), r=128 multi-tile (:600-696), extreme
forgetting stays finite (:699-747), aligned recurrent split (:850-867),
ragged tails T=1/19 (:870-897), single-token recurrent inference (:900-929),
strided views bit-equal to packed operands (:487-537), zero geometry write
reduces to the GDN2 edit (:296-316).

Tolerances: outputs and gradients max relative error (max|a-b| / max|b|)
<= 2e-2 and relative L2 <= 3e-2 (upstream :560-597); FP32 states max relative
error <= 1e-3.
"""
import numpy as np
import pytest
import torch

from oracle import solvedelta_oracle as orc
from solvedelta_b200 import SolveDeltaState, solvedelta_native
from tests.gpu_harness import make_inputs, oracle_args, oracle_state, raw_gate_grads
from tests.helpers import golden_inputs, golden_state, load_golden, max_rel, rel_l2

pytestmark = pytest.mark.gpu

OUT_TOL = 2e-2
STATE_TOL = 1e-3
GRAD_L2_TOL = 3e-2


def _native(dev, *, grad=False, return_final_state=True):
    names = ("u", "h", "q", "keys", "values", "log_decay", "erase_raw", "write_raw", "geometry_write")
    leaves = [dev[n].detach().clone().requires_grad_(grad) for n in names]
    state = None
    if dev["C0"] is not None:
        state = SolveDeltaState(dev["C0"].detach().clone().requires_grad_(grad),
                                dev["S0"].detach().clone().requires_grad_(grad))
    y, fin = solvedelta_native(*leaves, initial_state=state, return_final_state=return_final_state)
    return leaves, state, y, fin


def _np(t):
    return t.detach().float().cpu().numpy()


def _check_forward(cpu, y, fin):
    yo, so = orc.forward(*oracle_args(cpu), initial_state=oracle_state(cpu))
    assert torch.isfinite(y).all()
    assert max_rel(_np(y), yo) <= OUT_TOL
    assert rel_l2(_np(y), yo) <= OUT_TOL
    assert max_rel(_np(fin.predictor), so.predictor) <= STATE_TOL or np.abs(so.predictor).max() < 1e-12
    assert max_rel(_np(fin.S), so.S) <= STATE_TOL
    return yo, so


def _check_vjp(cpu, leaves, state, y, fin, seed=29):
    gen = torch.Generator().manual_seed(seed)
    dy = torch.randn(y.shape, generator=gen).to(torch.bfloat16)
    dC = torch.randn(fin.predictor.shape, generator=gen)
    dS = torch.randn(fin.S.shape, generator=gen)
    loss = (y.float() * dy.cuda().float()).sum() + (fin.predictor * dC.cuda()).sum() + (fin.S * dS.cuda()).sum()
    wrt = list(leaves) + (list(state) if state is not None else [])
    got = torch.autograd.grad(loss, wrt)
    ref = orc.backward(*oracle_args(cpu), dy.double().numpy(), dC_T=dC.double().numpy(),
                       dS_T=dS.double().numpy(), initial_state=oracle_state(cpu))
    d_er, d_wr = raw_gate_grads(cpu, ref)
    gam = ref["geometry_write"]
    if cpu["geometry_write"].ndim == 1:
        gam = gam.sum(axis=(0, 1))
    want = [ref["u"], ref["h"], ref["q"], ref["keys"][:, :, :, None], ref["values"][:, :, :, None],
            ref["log_decay"], d_er[:, :, :, None], d_wr[:, :, :, None], gam]
    names = ["u", "h", "q", "keys", "values", "log_decay", "erase_raw", "write_raw", "geometry_write"]
    if state is not None:
        want += [ref["C0"], ref["S0"]]
        names += ["C0", "S0"]
    for name, g, w in zip(names, got, want):
        g = g.float().cpu().numpy()
        assert np.isfinite(g).all(), name
        assert g.shape == w.shape, (name, g.shape, w.shape)
        assert rel_l2(g, w) <= GRAD_L2_TOL, (name, rel_l2(g, w))
        assert max_rel(g, w) <= OUT_TOL, (name, max_rel(g, w))


@pytest.mark.parametrize("B,T,H,r,V,gamma_mode", [
    (1, 16, 2, 16, 16, "token"),      # upstream _native_inputs geometry
    (2, 150, 2, 32, 48, "head"),      # crosses chunk boundaries, ragged tail, r != V
    (1, 32, 1, 128, 128, "token"),    # multi-tile widths
    (1, 256, 2, 128, 128, "token"),   # benchmark head geometry, four chunks
    (1, 19, 2, 16, 16, "token"),      # ragged tail
    (1, 1, 2, 16, 16, "token"),       # single token through the autograd path
])
def test_forward_and_full_vjp_match_checker(B, T, H, r, V, gamma_mode):
    cpu, dev = make_inputs(B, T, H, r, V, seed=23, gamma_mode=gamma_mode)
    leaves, state, y, fin = _native(dev, grad=True)
    assert y.dtype == torch.bfloat16 and fin.predictor.dtype == torch.float32
    _check_forward(cpu, y, fin)
    _check_vjp(cpu, leaves, state, y, fin)


def test_upstream_test_distribution_small_decay():
    # decay -0.02*rand, gate logits 0.5*randn, gamma 0.2 (upstream :375-398)
    cpu, dev = make_inputs(1, 16, 2, 16, 16, seed=7, decay_scale=0.02)
    cpu["geometry_write"] = torch.full((1, 16, 2), 0.2)
    dev["geometry_write"] = cpu["geometry_write"].cuda()
    leaves, state, y, fin = _native(dev, grad=True)
    _check_forward(cpu, y, fin)
    _check_vjp(cpu, leaves, state, y, fin)


@pytest.mark.parametrize("name", ["benchlike_r16_state", "benchlike_r32_t150_state"])
def test_committed_golden_vectors(name):
    """Upstream-generated vectors whose inputs are exactly BF16/FP32 representable."""
    g = load_golden(name)
    bf = lambda x: torch.from_numpy(x).to(torch.bfloat16).cuda()
    f32 = lambda x: torch.from_numpy(x).float().cuda()
    u, h, q, keys, values, decay, _, _, gamma = golden_inputs(g)
    C0, S0 = golden_state(g)
    leaves = [bf(u), bf(h), bf(q), bf(keys), bf(values), f32(decay), bf(g["in_erase_raw"]),
              bf(g["in_write_raw"]), f32(gamma)]
    for leaf, src in zip(leaves, (u, h, q, keys, values, decay, g["in_erase_raw"], g["in_write_raw"], gamma)):
        assert np.array_equal(leaf.double().cpu().numpy(), src)  # nothing was rounded
        leaf.requires_grad_()
    state = SolveDeltaState(f32(C0).requires_grad_(), f32(S0).requires_grad_())
    y, fin = solvedelta_native(*leaves, initial_state=state, return_final_state=True)
    assert max_rel(_np(y), g["out"]) <= OUT_TOL
    assert max_rel(_np(fin.predictor), g["C_T"]) <= STATE_TOL
    assert max_rel(_np(fin.S), g["S_T"]) <= STATE_TOL
    loss = ((y.float() * f32(g["dy"])).sum() + (fin.predictor * f32(g["dC_T"])).sum()
            + (fin.S * f32(g["dS_T"])).sum())
    got = torch.autograd.grad(loss, leaves + list(state))
    er, wr = g["in_erase"], g["in_write"]
    want = [g["grad_u"], g["grad_h"], g["grad_q"], g["grad_keys"], g["grad_values"], g["grad_log_decay"],
            g["grad_erase"] * er * (1 - er), g["grad_write"] * wr * (1 - wr), g["grad_geometry_write"],
            g["grad_C0"], g["grad_S0"]]
    for i, (a, b) in enumerate(zip(got, want)):
        assert rel_l2(_np(a), b) <= GRAD_L2_TOL, i


def test_zero_geometry_write_reduces_to_gdn2_edit():
    cpu, dev = make_inputs(1, 100, 2, 32, 32, seed=5, gamma_mode="zero", with_state=False)
    _, _, y, fin = _native(dev)
    # explicit GDN2 loop in FP64 on the same quantised inputs
    q = torch.nn.functional.normalize(cpu["q"].double(), dim=-1)
    k = torch.nn.functional.normalize(cpu["keys"].double()[:, :, :, 0], dim=-1)
    er = torch.sigmoid(cpu["erase_raw"].double()[:, :, :, 0])
    wr = torch.sigmoid(cpu["write_raw"].double()[:, :, :, 0])
    v = cpu["values"].double()[:, :, :, 0]
    mem = torch.zeros(1, 2, 32, 32, dtype=torch.float64)
    rows = []
    for t in range(100):
        mem = cpu["log_decay"][:, t].double().exp()[..., None] * mem
        pred = torch.einsum("bhrv,bhr->bhv", mem, er[:, t] * k[:, t])
        mem = mem + k[:, t][..., :, None] * (wr[:, t] * v[:, t] - pred)[..., None, :]
        rows.append(torch.einsum("bhrv,bhr->bhv", mem, q[:, t]))
    want = torch.stack(rows, dim=1)
    assert max_rel(_np(y), want.numpy()) <= OUT_TOL
    assert max_rel(_np(fin.S), mem.numpy()) <= STATE_TOL
    assert float(fin.predictor.abs().max()) == 0.0


def test_aligned_and_ragged_split_continuation():
    cpu, dev = make_inputs(1, 160, 2, 32, 32, seed=9)
    _, _, y, fin = _native(dev)
    for split in (64, 100):
        def part(lo, hi, state):
            sub = {n: (t[:, lo:hi] if n not in ("C0", "S0") and t.ndim >= 3 else t) for n, t in dev.items()}
            sub["C0"], sub["S0"] = state
            return _native(sub)
        _, _, y1, s1 = part(0, split, (dev["C0"], dev["S0"]))
        _, _, y2, s2 = part(split, 160, (s1.predictor, s1.S))
        both = torch.cat([y1, y2], dim=1)
        if split % 64 == 0:  # chunk-aligned: identical arithmetic, identical bits
            assert torch.equal(both, y) and torch.equal(s2.predictor, fin.predictor) and torch.equal(s2.S, fin.S)
        else:
            assert max_rel(_np(both), _np(y)) <= OUT_TOL
            assert max_rel(_np(s2.S), _np(fin.S)) <= STATE_TOL
            assert max_rel(_np(s2.predictor), _np(fin.predictor)) <= STATE_TOL


def test_single_token_recurrent_inference_matches_checker():
    cpu, dev = make_inputs(2, 1, 2, 64, 64, seed=13)
    with torch.no_grad():
        _, _, y, fin = _native(dev)
    assert y.shape == (2, 1, 2, 64)
    _check_forward(cpu, y, fin)
    # sixteen decode steps equal one dense pass (upstream tests/model:264-301)
    cpu, dev = make_inputs(1, 16, 2, 32, 32, seed=17)
    _, _, y_dense, fin_dense = _native(dev)
    state = (dev["C0"], dev["S0"])
    outs = []
    with torch.no_grad():
        for t in range(16):
            sub = {n: (x[:, t:t + 1] if n not in ("C0", "S0") and x.ndim >= 3 else x) for n, x in dev.items()}
            sub["C0"], sub["S0"] = state
            _, _, yt, st = _native(sub)
            outs.append(yt)
            state = (st.predictor, st.S)
    assert max_rel(_np(torch.cat(outs, 1)), _np(y_dense)) <= OUT_TOL
    assert max_rel(_np(state[1]), _np(fin_dense.S)) <= STATE_TOL


def test_strided_projection_views_are_bit_equal_to_packed():
    cpu, dev = make_inputs(1, 40, 2, 16, 16, seed=19)
    _, _, y_ref, fin_ref = _native(dev)
    # place every BF16 operand inside a wider row with an odd (non 16-byte) pitch
    def strided(t):
        wide = torch.zeros(*t.shape[:-1], 23, dtype=t.dtype, device=t.device)
        wide[..., 3:3 + t.shape[-1]] = t
        return wide[..., 3:3 + t.shape[-1]]
    sub = dict(dev)
    for n in ("u", "h", "q", "keys", "values", "erase_raw", "write_raw"):
        sub[n] = strided(dev[n])
        assert not sub[n].is_contiguous()
    leaves, state, y, fin = _native(sub, grad=False)
    # _native clones leaves (making them packed); call the entry point on the views directly
    y, fin = solvedelta_native(sub["u"], sub["h"], sub["q"], sub["keys"], sub["values"], sub["log_decay"],
                               sub["erase_raw"], sub["write_raw"], sub["geometry_write"],
                               initial_state=SolveDeltaState(sub["C0"], sub["S0"]), return_final_state=True)
    assert torch.equal(y, y_ref) and torch.equal(fin.S, fin_ref.S) and torch.equal(fin.predictor, fin_ref.predictor)


def test_extreme_forgetting_remains_finite():
    cpu, dev = make_inputs(1, 70, 2, 32, 32, seed=21)
    dev["log_decay"] = torch.full_like(dev["log_decay"], -100.0)
    leaves, state, y, fin = _native(dev, grad=True)
    loss = y.float().sum() + fin.predictor.sum() + fin.S.sum()
    grads = torch.autograd.grad(loss, list(leaves) + list(state))
    assert torch.isfinite(y).all() and torch.isfinite(fin.S).all() and torch.isfinite(fin.predictor).all()
    for g in grads:
        assert torch.isfinite(g).all()


def _strong_decay_inputs(B, T, H, r, V, scale, seed):
    """Per-channel decay rates spread over four decades up to `scale` nats per token
    (upstream runs its exterior owner at decay_scale 16, tests/core/test_rebuild_semantics.py:411)."""
    cpu, dev = make_inputs(B, T, H, r, V, seed=seed)
    gen = torch.Generator().manual_seed(seed + 1)
    rate = scale * torch.exp(torch.rand(1, 1, H, r, generator=gen) * np.log(1e-4))
    cpu["log_decay"] = -rate * (0.75 + 0.25 * torch.rand(B, T, H, r, generator=gen))
    dev["log_decay"] = cpu["log_decay"].cuda()
    return cpu, dev


@pytest.mark.parametrize("scale", [1.5, 16.0])
@pytest.mark.parametrize("T,H,r,V", [(150, 2, 16, 16), (200, 1, 128, 128)])
def test_strong_forgetting_forward_matches_checker(scale, T, H, r, V):
    # chunk prefixes reach -1000: exact only without reciprocal-retention factors
    cpu, dev = _strong_decay_inputs(1, T, H, r, V, scale, seed=41)
    leaves, state, y, fin = _native(dev, grad=False)
    _check_forward(cpu, y, fin)


# 3.6 nats per token: 16-token blocks forget up to 58 nats, just inside the tensor-core path for
# diagonal blocks (60); 16: far outside it
@pytest.mark.parametrize("scale", [1.5, 3.6, 16.0])
@pytest.mark.parametrize("T,H,r,V", [(150, 2, 16, 16), (200, 1, 128, 128)])
def test_strong_forgetting_full_vjp_matches_checker(scale, T, H, r, V):
    cpu, dev = _strong_decay_inputs(1, T, H, r, V, scale, seed=43)
    leaves, state, y, fin = _native(dev, grad=True)
    _check_forward(cpu, y, fin)
    _check_vjp(cpu, leaves, state, y, fin)


def test_forgetting_bursts_mix_fast_and_direct_blocks():
    """Mild decay with bursts of 16 nats per token: inside one chunk some 16-token blocks take the
    tensor-core path for their diagonal block and others the direct evaluation."""
    cpu, dev = make_inputs(1, 200, 2, 32, 32, seed=47)
    ld = cpu["log_decay"].clone()
    ld[:, 40:60] = -16.0 * (0.75 + 0.25 * torch.rand(1, 20, 2, 32, generator=torch.Generator().manual_seed(3)))
    ld[:, 100:131, 1] = -9.0
    ld[:, 190:, :, :8] = -30.0
    cpu["log_decay"] = ld
    dev["log_decay"] = ld.cuda()
    leaves, state, y, fin = _native(dev, grad=True)
    _check_forward(cpu, y, fin)
    _check_vjp(cpu, leaves, state, y, fin)


def test_return_final_state_false_and_none_cotangents():
    cpu, dev = make_inputs(1, 70, 1, 16, 16, seed=25)
    leaves, state, y, fin = _native(dev, grad=True, return_final_state=False)
    assert fin is None
    (y.float().sum()).backward()
    assert all(leaf.grad is not None and torch.isfinite(leaf.grad).all() for leaf in leaves)
    # only a state cotangent, no output cotangent
    leaves, state, y, fin = _native(dev, grad=True)
    grads = torch.autograd.grad(fin.S.sum(), leaves[:5])
    assert all(torch.isfinite(g).all() for g in grads)


def test_contract_errors_match_upstream_types():
    cpu, dev = make_inputs(1, 8, 1, 16, 16, seed=1)
    a = [dev[n] for n in ("u", "h", "q", "keys", "values", "log_decay", "erase_raw", "write_raw", "geometry_write")]
    with pytest.raises(ValueError, match="num_edits=1"):
        bad = list(a)
        bad[3] = a[3].expand(-1, -1, -1, 2, -1)
        solvedelta_native(*bad)
    with pytest.raises(TypeError):
        bad = list(a)
        bad[5] = a[5].double()
        solvedelta_native(*bad)
    with pytest.raises(ValueError, match="unit innermost stride"):
        bad = list(a)
        bad[0] = a[0].repeat_interleave(2, dim=-1)[..., ::2]
        solvedelta_native(*bad)
    with pytest.raises(ValueError, match="initial_state"):
        solvedelta_native(*a, initial_state=SolveDeltaState(dev["C0"][:, :, :8], dev["S0"]))
    with pytest.raises(TypeError, match="FP32"):
        solvedelta_native(*a, initial_state=SolveDeltaState(dev["C0"].double(), dev["S0"].double()))


def _masked_case(cpu, dev, valid, reset, *, state_tol=STATE_TOL):
    """Forward + full VJP of the masked entry point against the checker; the call itself must not
    synchronise with the host (the masks are read inside the kernels)."""
    from solvedelta_b200 import build_packed_segments, solvedelta_segmented_native

    plan = build_packed_segments(valid.cuda(), reset.cuda())
    names = ("u", "h", "q", "keys", "values", "log_decay", "erase_raw", "write_raw", "geometry_write")
    leaves = [dev[n].detach().clone().requires_grad_() for n in names]
    state = SolveDeltaState(dev["C0"].clone().requires_grad_(), dev["S0"].clone().requires_grad_())
    torch.cuda.synchronize()
    torch.cuda.set_sync_debug_mode("error")
    try:
        y, fin = solvedelta_segmented_native(*leaves, plan, initial_state=state, return_final_state=True)
    finally:
        torch.cuda.set_sync_debug_mode("default")
    yo, so = orc.forward(*oracle_args(cpu), initial_state=oracle_state(cpu), valid_mask=valid.numpy(),
                         reset_mask=reset.numpy())
    assert torch.equal(y[~valid.cuda()], torch.zeros_like(y[~valid.cuda()]))
    assert max_rel(_np(y), yo) <= OUT_TOL
    assert max_rel(_np(fin.predictor), so.predictor) <= state_tol and max_rel(_np(fin.S), so.S) <= state_tol
    gen = torch.Generator().manual_seed(3)
    dy = torch.randn(y.shape, generator=gen).to(torch.bfloat16).cuda()
    dC, dS = torch.randn(fin.predictor.shape, generator=gen), torch.randn(fin.S.shape, generator=gen)
    dCd, dSd = dC.cuda(), dS.cuda()
    torch.cuda.synchronize()
    torch.cuda.set_sync_debug_mode("error")
    try:
        got = torch.autograd.grad((y, fin.predictor, fin.S), leaves + list(state), (dy, dCd, dSd))
    finally:
        torch.cuda.set_sync_debug_mode("default")
    ref = orc.backward(*oracle_args(cpu), dy.cpu().double().numpy(), dC_T=dC.double().numpy(),
                       dS_T=dS.double().numpy(), initial_state=oracle_state(cpu), valid_mask=valid.numpy(),
                       reset_mask=reset.numpy())
    d_er, d_wr = raw_gate_grads(cpu, ref)
    want = [ref["u"], ref["h"], ref["q"], ref["keys"][:, :, :, None], ref["values"][:, :, :, None],
            ref["log_decay"], d_er[:, :, :, None], d_wr[:, :, :, None], ref["geometry_write"], ref["C0"], ref["S0"]]
    off = (~valid).cuda()
    for name, g, w in zip(names + ("C0", "S0"), got, want):
        assert torch.isfinite(g).all(), name
        assert rel_l2(_np(g), w) <= GRAD_L2_TOL, (name, rel_l2(_np(g), w))
        assert max_rel(_np(g), w) <= OUT_TOL, (name, max_rel(_np(g), w))
        if name not in ("C0", "S0"):
            assert torch.equal(g[off], torch.zeros_like(g[off])), name   # masked tokens: exact zeros
    return fin


def test_segmented_masks_resets_and_vjp_match_checker():
    """Masked tokens, a mid-row reset and an all-invalid batch row (upstream :932-1039)."""
    cpu, dev = make_inputs(2, 19, 1, 16, 16, seed=149, decay_scale=0.03, gamma_max=0.9)
    valid = torch.tensor([[1, 1, 0, 1, 1, 1, 1, 0, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1], [0] * 19], dtype=torch.bool)
    reset = torch.zeros_like(valid)
    reset[0, 8] = True
    fin = _masked_case(cpu, dev, valid, reset)
    # the all-invalid row returns its initial state untouched
    assert torch.equal(fin.S[1], dev["S0"][1]) and torch.equal(fin.predictor[1], dev["C0"][1])


@pytest.mark.parametrize("r,V,decay_scale", [(32, 32, None), (128, 128, None), (16, 24, 1.5)])
def test_masks_and_resets_across_chunks(r, V, decay_scale):
    """Several chunks with holes, resets in the first row of a chunk, on its last row, twice inside one
    16-token block, on a masked token (ignored), at the very first token, and a row that is reset late."""
    B, T, H = 3, 200, 2
    cpu, dev = make_inputs(B, T, H, r, V, seed=151, decay_scale=decay_scale, gamma_max=0.5)
    gen = torch.Generator().manual_seed(9)
    valid = torch.rand(B, T, generator=gen) > 0.15
    valid[1, :70] = False           # left padding over more than one chunk
    valid[2, 150:] = False          # right padding
    reset = torch.zeros(B, T, dtype=torch.bool)
    for b, t in ((0, 0), (0, 37), (0, 39), (0, 63), (0, 64), (0, 130), (1, 100), (2, 5), (2, 128), (2, 149)):
        reset[b, t] = True
    reset[0, 90] = True
    valid[0, 90] = False            # a reset on a masked token does nothing
    _masked_case(cpu, dev, valid, reset)
