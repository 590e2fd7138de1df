"""Kernel-by-kernel localisation: every intermediate panel the CUDA library
writes is compared with the chunk-form model evaluated in FP64 on the same
quantised inputs.  All panels are checked before the test fails, so one run
names every kernel that is off."""
import pytest
import torch

from tests.chunk_model import Model
from tests.gpu_harness import RawRun, make_inputs, model_inputs
from tests.helpers import rel_l2

SAVED = ("Lam", "G", "Delta", "Dprim", "Zt", "CtCk", "SCk", "N", "Aed", "Aqd", "Xg", "Ag", "DtB")
FWD = ("Upd", "Qc", "Ubar", "Wd", "Ud", "Dt")
BWD = ("Pp", "Qp", "Dyf", "dR", "dSeCk", "SdS",
       "duPart", "dkPart", "dGPart", "DG", "Dd", "Xext", "Tu", "Khat", "dDelta", "Ppp", "Qpp", "Rneg",
       "dRr", "dCeCk")


def _pad(x):
    """[S,NC,rows,cols] model panel -> [chunks, rows', 128-or-L] zero padded like the library's."""
    S, NC = x.shape[0], x.shape[1]
    x = x.reshape(S * NC, *x.shape[2:]) if x.ndim == 4 else x.reshape(S * NC, 1, x.shape[-1])
    return x


def _compare(got, want):
    want = _pad(want).float()
    rows, cols = want.shape[1], want.shape[2]
    crop = got[:, :rows, :cols]
    err = rel_l2(crop.numpy(), want.numpy())
    # whatever lies outside the true extent must be zero padding
    total = float(got.double().pow(2).sum())
    inside = float(crop.double().pow(2).sum())
    spill = max(total - inside, 0.0) ** 0.5 / max(total ** 0.5, 1e-30)
    return err, spill


@pytest.mark.gpu
@pytest.mark.parametrize("B,T,H,r,V", [(1, 150, 2, 32, 32), (1, 200, 1, 128, 128), (2, 70, 1, 16, 24)])
def test_every_panel_matches_chunk_model(B, T, H, r, V):
    cpu, dev = make_inputs(B, T, H, r, V, seed=3)
    gen = torch.Generator().manual_seed(11)
    dy = torch.randn(B, T, H, V, generator=gen).to(torch.bfloat16)
    dC = torch.randn(B, H, r, r, generator=gen)
    dS = torch.randn(B, H, r, V, generator=gen)
    run = RawRun(dev, dy.cuda(), dC.cuda(), dS.cuda())
    model = Model(chunk=64)
    inp = model_inputs(cpu)
    y, C_T, S_T, saved = model.forward(inp, cpu["C0"].double(), cpu["S0"].double())
    grads, bwd_panels = model.backward(inp, saved, dy.double(), dC.double(), dS.double())
    report, bad = [], []
    fwd_ref = dict(saved["panels"])
    fwd_ref["Ag"] = bwd_panels["Ag"]          # -e exp(G) and the BF16 copy of Dt are written by the forward pass
    fwd_ref["DtB"] = saved["panels"]["Dt"]
    for which, names, ref in ((0, SAVED, fwd_ref), (1, FWD, fwd_ref), (2, BWD, bwd_panels)):
        for name in names:
            got, dtype = run.panel(which, name)
            err, spill = _compare(got, ref[name])
            report.append(f"{('saved', 'fwd', 'bwd')[which]:5s} {name:8s} {dtype:4s} rel={err:.2e} pad={spill:.1e}")
            if name == "Lam":
                spill = 0.0  # channels beyond r carry exp(0) = 1, not zero
            # FP32 panels come from TF32 contractions, BF16 panels from BF16 ones
            tol = 1.5e-2 if (dtype == "bf16" or which == 2) else 5e-3
            if not (err < tol) or not (spill < 1e-6):
                bad.append(name)
    outs = dict(y=(run.y.float().cpu(), y), C_T=(run.C_T.cpu(), C_T), S_T=(run.S_T.cpu(), S_T))
    for name, (got, want) in outs.items():
        err = rel_l2(got.numpy(), want.numpy())
        report.append(f"out   {name:8s} rel={err:.2e}")
        if not (err < 1e-2):
            bad.append(name)
    key = dict(u="u", h="h", q="q", keys="k", values="v", log_decay="g", erase_raw="erase_raw",
               write_raw="write_raw", geometry_write="gamma", C0="C0", S0="S0")
    for name, mk in key.items():
        err = rel_l2(run.grads[name].float().cpu().numpy(), grads[mk].numpy())
        report.append(f"grad  {name:14s} rel={err:.2e}")
        if not (err < 1e-2):
            bad.append("grad_" + name)
    print("\n".join(report))
    assert not bad, "panels off: " + ", ".join(bad) + "\n" + "\n".join(report)
