"""Benchmark-size checks (B=8, H=8, T=4096, r=V=128) that do not need the CPU
checker on the whole tensor: size-independent properties of the recurrence,
plus the checker on two single streams of the full-length run."""
import numpy as np
import pytest
import torch

from oracle import solvedelta_oracle as orc
from solvedelta_b200 import SolveDeltaState, solvedelta_native
from tests.helpers import max_rel, rel_l2

pytestmark = pytest.mark.gpu

B, T, H, R, V = 8, 4096, 8, 128, 128
NAMES = ("u", "h", "q", "keys", "values", "log_decay", "erase_raw", "write_raw", "geometry_write")


@pytest.fixture(scope="module")
def workload():
    from bench import make_cpu_inputs

    cpu = make_cpu_inputs(B, T, H, R, V, seed=0)
    dev = {k: v.cuda() for k, v in cpu.items()}
    return cpu, dev


def _run(dev, *, lo=0, hi=T, state=None, scale_values=1.0):
    args = [dev[n][:, lo:hi] for n in NAMES]
    if scale_values != 1.0:
        args[4] = args[4] * scale_values
    if state is None:
        state = SolveDeltaState(dev["C0"], dev["S0"])
    with torch.no_grad():
        return solvedelta_native(*args, initial_state=state, return_final_state=True)


def test_split_continuation_is_bit_equal_at_full_length(workload):
    _, dev = workload
    y, fin = _run(dev)
    y1, s1 = _run(dev, hi=T // 2)
    y2, s2 = _run(dev, lo=T // 2, state=s1)
    assert torch.equal(torch.cat([y1, y2], dim=1), y)
    assert torch.equal(s2.predictor, fin.predictor) and torch.equal(s2.S, fin.S)
    assert torch.isfinite(y).all()


def test_memory_side_is_linear_in_values_and_initial_memory(workload):
    # y and S are linear in (values, S0); a factor of two commutes with every rounding
    _, dev = workload
    y, fin = _run(dev)
    y2, fin2 = _run(dev, state=SolveDeltaState(dev["C0"], 2.0 * dev["S0"]), scale_values=2.0)
    assert torch.equal(y2.float(), 2.0 * y.float())
    assert torch.equal(fin2.S, 2.0 * fin.S)
    assert torch.equal(fin2.predictor, fin.predictor)  # the predictor never sees the values


def test_streams_are_independent(workload):
    _, dev = workload
    y, fin = _run(dev)
    perm = torch.tensor([3, 0, 7, 1, 6, 2, 5, 4], device="cuda")
    shuffled = {k: v[perm] for k, v in dev.items()}
    yp, finp = _run(shuffled)
    assert torch.equal(yp, y[perm])
    assert torch.equal(finp.S, fin.S[perm]) and torch.equal(finp.predictor, fin.predictor[perm])


@pytest.mark.parametrize("world", [2, 8, 16])
def test_stream_shards_of_the_product_reassemble_the_full_run(workload, world):
    """The strong-scaling layout of bench.py --strong on one GPU: every rank's shard (batch rows first, then
    heads) run through the operator, forward and VJP, and put back together, is bit-equal to the full run."""
    from solvedelta_b200.sharding import stream_shard

    _, dev = workload
    names = NAMES

    def fwd_bwd(d):
        leaves = [d[n].detach().requires_grad_() for n in names]
        state = SolveDeltaState(d["C0"].detach().requires_grad_(), d["S0"].detach().requires_grad_())
        y, fin = solvedelta_native(*leaves, initial_state=state, return_final_state=True)
        grads = torch.autograd.grad((y, fin.predictor, fin.S), leaves + list(state), (d["dy"], d["dC_T"], d["dS_T"]))
        return y.detach(), fin.predictor.detach(), fin.S.detach(), grads

    y, C, S, grads = fwd_bwd(dev)
    B, H = y.shape[0], y.shape[2]
    for rank in range(world):
        bs, hs = stream_shard(B, H, rank, world)
        part = {k: (v[bs][:, hs] if k in ("C0", "S0", "dC_T", "dS_T") else v[bs][:, :, hs]).contiguous()
                for k, v in dev.items()}
        yp, Cp, Sp, gp = fwd_bwd(part)
        assert torch.equal(yp, y[bs][:, :, hs])
        assert torch.equal(Cp, C[bs][:, hs]) and torch.equal(Sp, S[bs][:, hs])
        for full, got, name in zip(grads, gp, list(names) + ["C0", "S0"]):
            want = full[bs][:, hs] if name in ("C0", "S0") else full[bs][:, :, hs]
            assert torch.equal(got, want), name


def _zero_geometry(workload):
    """The benchmark workload with the geometry rate at zero and no initial predictor state: the operator
    is then exactly the GDN2 edit / read (upstream tests/core/test_rebuild_semantics.py:296-316)."""
    cpu, dev = workload
    cpu0, dev0 = dict(cpu), dict(dev)
    for d in (cpu0, dev0):
        d["geometry_write"] = torch.zeros_like(d["geometry_write"])
        d["C0"] = torch.zeros_like(d["C0"])
    return cpu0, dev0


@pytest.mark.parametrize("gamma_zero", [False, True])
@pytest.mark.parametrize("b,h", [(0, 0), (7, 7)])
def test_single_streams_of_the_full_run_match_the_checker(workload, b, h, gamma_zero):
    cpu, dev = _zero_geometry(workload) if gamma_zero else workload
    leaves = [dev[n].detach().clone().requires_grad_() for n in NAMES]
    state = SolveDeltaState(dev["C0"].clone().requires_grad_(), dev["S0"].clone().requires_grad_())
    y, fin = solvedelta_native(*leaves, initial_state=state, return_final_state=True)
    grads = torch.autograd.grad((y, fin.predictor, fin.S), leaves + list(state),
                                (dev["dy"], dev["dC_T"], dev["dS_T"]))
    d = lambda x: x[b:b + 1, :, h:h + 1].double().numpy()
    args = [d(cpu["u"]), d(cpu["h"]), d(cpu["q"]), d(cpu["keys"]), d(cpu["values"]), d(cpu["log_decay"]),
            d(torch.sigmoid(cpu["erase_raw"].double())), d(torch.sigmoid(cpu["write_raw"].double())),
            d(cpu["geometry_write"])]
    st = (cpu["C0"][b:b + 1, h:h + 1].double().numpy(), cpu["S0"][b:b + 1, h:h + 1].double().numpy())
    yo, so = orc.forward(*args, initial_state=st)
    ref = orc.backward(*args, d(cpu["dy"]), dC_T=cpu["dC_T"][b:b + 1, h:h + 1].double().numpy(),
                       dS_T=cpu["dS_T"][b:b + 1, h:h + 1].double().numpy(), initial_state=st)
    sl = lambda x: x[b:b + 1, :, h:h + 1].detach().float().cpu().numpy()
    assert max_rel(sl(y), yo) <= 2e-2
    if gamma_zero:
        # nothing writes the predictor: it stays at its (zero) initial value, and the exterior is the GDN2 loop
        assert float(np.abs(so.predictor).max()) == 0.0 and float(fin.predictor[b, h].abs().max()) == 0.0
        assert max_rel(sl(y), _gdn2_outputs(cpu, b, h)) <= 2e-2
    else:
        assert max_rel(fin.predictor[b:b + 1, h:h + 1].detach().cpu().numpy(), so.predictor) <= 1e-3
    assert max_rel(fin.S[b:b + 1, h:h + 1].detach().cpu().numpy(), so.S) <= 1e-3
    se = torch.sigmoid(cpu["erase_raw"].double()).numpy()[b:b + 1, :, h:h + 1, 0]
    sw = torch.sigmoid(cpu["write_raw"].double()).numpy()[b:b + 1, :, h:h + 1, 0]
    want = [ref["u"], ref["h"], ref["q"], ref["keys"][:, :, :, None], ref["values"][:, :, :, None],
            ref["log_decay"], (ref["erase"] * se * (1 - se))[:, :, :, None],
            (ref["write"] * sw * (1 - sw))[:, :, :, None], ref["geometry_write"]]
    for name, g, w in zip(NAMES, grads[:9], want):
        g = sl(g)
        assert rel_l2(g, w) <= 3e-2, (name, rel_l2(g, w))
        assert max_rel(g, w) <= 2e-2, (name, max_rel(g, w))
    gC = grads[9][b:b + 1, h:h + 1].cpu().numpy()
    gS = grads[10][b:b + 1, h:h + 1].cpu().numpy()
    assert rel_l2(gC, ref["C0"]) <= 3e-2 and rel_l2(gS, ref["S0"]) <= 3e-2


def _gdn2_outputs(cpu, b, h):
    """The explicit GDN2 recurrence in FP64 for one stream: S <- diag(alpha) S; S += k (w*v - S^T (e*k))^T;
    y = S^T q, with normalised q, k (upstream tests/core/test_rebuild_semantics.py:296-316)."""
    f = lambda x: x[b, :, h].double().numpy()
    q, k = f(cpu["q"]), f(cpu["keys"][:, :, :, 0])
    q = q / np.linalg.norm(q, axis=-1, keepdims=True)
    k = k / np.linalg.norm(k, axis=-1, keepdims=True)
    v = f(cpu["values"][:, :, :, 0])
    alpha = np.exp(f(cpu["log_decay"]))
    e = 1.0 / (1.0 + np.exp(-f(cpu["erase_raw"][:, :, :, 0])))
    w = 1.0 / (1.0 + np.exp(-f(cpu["write_raw"][:, :, :, 0])))
    S = cpu["S0"][b, h].double().numpy().copy()
    out = np.empty((1, q.shape[0], 1, v.shape[-1]))
    for t in range(q.shape[0]):
        S = alpha[t][:, None] * S
        S = S + np.outer(k[t], w[t] * v[t] - S.T @ (e[t] * k[t]))
        out[0, t, 0] = S.T @ q[t]
    return out


def test_long_prefill_then_decode_steps_equal_one_pass():
    """Long-context continuation at the operator (upstream tests/model/test_modeling_solvedelta.py:264-301):
    a 32 768-token prefill at B=1, H=8 followed by 256 single-token recurrent steps ends in the same (C, S)
    as one pass over all 33 024 tokens, and produces the same outputs for the 256 tokens."""
    from bench import make_cpu_inputs

    prefill, steps = 32768, 256
    cpu = make_cpu_inputs(1, prefill + steps, H, R, V, seed=4)
    dev = {k: v.cuda() for k, v in cpu.items()}
    args = lambda lo, hi: [dev[n][:, lo:hi] for n in NAMES]
    start = SolveDeltaState(dev["C0"], dev["S0"])
    with torch.no_grad():
        y_all, fin_all = solvedelta_native(*args(0, prefill + steps), initial_state=start, return_final_state=True)
        _, state = solvedelta_native(*args(0, prefill), initial_state=start, return_final_state=True)
        pieces = []
        for t in range(prefill, prefill + steps):
            y_t, state = solvedelta_native(*args(t, t + 1), initial_state=state, return_final_state=True)
            pieces.append(y_t)
    y_dec = torch.cat(pieces, dim=1).float().cpu().numpy()
    assert max_rel(y_dec, y_all[:, prefill:].float().cpu().numpy()) <= 2e-2
    assert max_rel(state.predictor.cpu().numpy(), fin_all.predictor.cpu().numpy()) <= 1e-3
    assert max_rel(state.S.cpu().numpy(), fin_all.S.cpu().numpy()) <= 1e-3
    assert torch.isfinite(y_all).all()


@pytest.mark.gpu
def test_no_bounded_wait_ran_out(workload):
    """Every device-side wait of the kernels is bounded; none of them may have given up during a full-size run."""
    from solvedelta_b200 import _lib

    _run(workload[1])
    assert _lib.load().sd_device_fault() == 0
