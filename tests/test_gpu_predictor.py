"""The predictor sub-owner entry (upstream oja_residual, causallsso/ops/residual_frame/predictor.py:285-305)
against the token recurrence it abbreviates (causallsso/reference.py:170-199: residual, update, state and the
frame action C'^T k), differentiated by torch.autograd in FP64 on the CPU."""
import numpy as np
import pytest
import torch

from tests.helpers import max_rel

pytestmark = pytest.mark.gpu

OUT_TOL, STATE_TOL, GRAD_TOL, GRAD_L2 = 2e-2, 1e-3, 2e-2, 3e-2


def _token_loop(target, source, beta, log_decay, query, C0):
    """FP64: residual = h - C u, update = beta residual, C' = C diag(exp(g)) + update u^T, action = C'^T k."""
    B, T, H, r = target.shape
    C = torch.zeros(B, H, r, r, dtype=torch.float64) if C0 is None else C0
    actions, updates = [], []
    for t in range(T):
        u = source[:, t]
        residual = target[:, t] - (C @ u.unsqueeze(-1)).squeeze(-1)
        update = beta[:, t, :, None] * residual
        C = C * log_decay[:, t].exp()[..., None, :] + update[..., :, None] * u[..., None, :]
        actions.append((C.transpose(-1, -2) @ query[:, t].unsqueeze(-1)).squeeze(-1))
        updates.append(update)
    return torch.stack(actions, 1), torch.stack(updates, 1), C


def _inputs(B, T, H, r, seed, stateful):
    gen = torch.Generator().manual_seed(seed)
    unit = lambda x: torch.nn.functional.normalize(x.float(), dim=-1).to(torch.bfloat16)
    target = torch.randn(B, T, H, r, generator=gen).to(torch.bfloat16)
    source = unit(torch.randn(B, T, H, r, generator=gen))
    query = unit(torch.randn(B, T, H, r, generator=gen))
    beta = 0.1 * torch.rand(B, T, H, generator=gen)
    log_decay = torch.nn.functional.logsigmoid(torch.randn(B, T, H, r, generator=gen) + 3.0)
    C0 = 0.02 * torch.randn(B, H, r, r, generator=gen) if stateful else None
    cot = dict(action=torch.randn(B, T, H, r, generator=gen).to(torch.bfloat16),
               update=torch.randn(B, T, H, r, generator=gen).to(torch.bfloat16),
               C=torch.randn(B, H, r, r, generator=gen))
    return target, source, beta, log_decay, query, C0, cot


def _rel_l2(a, b):
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30))


@pytest.mark.parametrize("B,T,H,r,stateful", [(1, 70, 2, 32, True), (2, 130, 2, 64, False), (1, 200, 1, 128, True),
                                              (2, 19, 3, 16, True)])
def test_oja_residual_matches_the_token_recurrence(B, T, H, r, stateful):
    from solvedelta_b200 import oja_residual

    target, source, beta, log_decay, query, C0, cot = _inputs(B, T, H, r, 7 * T + r, stateful)
    names = ("target", "source", "beta", "log_decay", "query")
    cpu = [t.double().requires_grad_() for t in (target, source, beta, log_decay, query)]
    c0_cpu = None if C0 is None else C0.double().requires_grad_()
    a_ref, u_ref, C_ref = _token_loop(*cpu, c0_cpu)
    ((a_ref * cot["action"].double()).sum() + (u_ref * cot["update"].double()).sum()
     + (C_ref * cot["C"].double()).sum()).backward()

    dev = [t.cuda().requires_grad_() for t in (target, source, beta, log_decay, query)]
    c0_dev = None if C0 is None else C0.cuda().requires_grad_()
    action, update, final = oja_residual(dev[0], dev[1], dev[2], dev[3], dev[4], c0_dev, chunk_size=32,
                                         output_final_state=True)
    assert action.dtype == update.dtype == torch.bfloat16 and final.dtype == torch.float32
    ((action.float() * cot["action"].cuda().float()).sum() + (update.float() * cot["update"].cuda().float()).sum()
     + (final * cot["C"].cuda()).sum()).backward()
    np_ = lambda t: t.detach().double().cpu().numpy()
    assert max_rel(np_(action), np_(a_ref)) <= OUT_TOL
    assert max_rel(np_(update), np_(u_ref)) <= OUT_TOL
    assert max_rel(np_(final), np_(C_ref)) <= STATE_TOL
    for name, d, c in zip(names, dev, cpu):
        assert max_rel(np_(d.grad), np_(c.grad)) <= GRAD_TOL, name
        assert _rel_l2(np_(d.grad), np_(c.grad)) <= GRAD_L2, name
    if stateful:
        assert max_rel(np_(c0_dev.grad), np_(c0_cpu.grad)) <= GRAD_TOL


def test_oja_residual_accepts_missing_cotangents_and_checks_its_arguments():
    from solvedelta_b200 import oja_residual

    target, source, beta, log_decay, query, C0, cot = _inputs(1, 40, 2, 32, 3, True)
    dev = [t.cuda().requires_grad_() for t in (target, source, beta, log_decay, query)]
    action, update, final = oja_residual(*dev, None, output_final_state=False)
    assert final is None
    update.float().sum().backward()      # the action's cotangent is absent
    assert all(t.grad is not None and torch.isfinite(t.grad.float()).all() for t in dev)
    with pytest.raises(TypeError):
        oja_residual(dev[0].float(), dev[1], dev[2], dev[3], dev[4], None)
    with pytest.raises(TypeError):
        oja_residual(dev[0], dev[1], dev[2].to(torch.bfloat16), dev[3], dev[4], None)
    with pytest.raises(ValueError):
        oja_residual(dev[0], dev[1][:, :5], dev[2], dev[3], dev[4], None)
