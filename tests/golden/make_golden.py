"""Regenerate tests/golden/*.npz from the upstream FP64 oracle.

Run where the upstream tree is mounted:

    python tests/golden/make_golden.py /path/to/SolveDelta

It loads ``causallsso/reference.py`` straight from that tree (the file needs
only torch), evaluates ``solvedelta_reference`` in FP64 on small seeded cases
and differentiates it with torch.autograd.  Inputs, cotangents, outputs,
final states and every gradient are stored, so the committed vectors pin both
the CPU checker under ``oracle/`` and the CUDA path without the upstream tree.

Input distributions follow the upstream tests
(tests/core/test_rebuild_semantics.py:31-57 for the seed-7 draw,
:319-329 for the mask/reset pattern, :296-299 for the zero-geometry case).
"""
from __future__ import annotations

import importlib.util
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def load_reference(root: str):
    path = os.path.join(root, "causallsso", "reference.py")
    spec = importlib.util.spec_from_file_location("upstream_reference", path)
    mod = importlib.util.module_from_spec(spec)
    sys.modules["upstream_reference"] = mod
    spec.loader.exec_module(mod)
    return mod


def seed7_inputs(length=6, rank=8, value_dim=5):
    torch.manual_seed(7)
    batch, heads = 2, 2
    u = torch.randn(batch, length, heads, rank, dtype=torch.float64)
    h = torch.randn_like(u)
    q = torch.randn_like(u)
    keys = torch.randn(batch, length, heads, 1, rank, dtype=torch.float64)
    values = torch.randn(batch, length, heads, 1, value_dim, dtype=torch.float64)
    decay = -0.02 * torch.rand(batch, length, heads, rank, dtype=torch.float64)
    erase = torch.rand_like(keys)
    write = torch.rand_like(values)
    gamma = torch.full((heads,), 0.25, dtype=torch.float64)
    return [u, h, q, keys, values, decay, erase, write, gamma]


RAW_GATES = {}


def bench_like_inputs(batch, length, heads, rank, value_dim, seed):
    """Same distributions as the benchmark workload.  Every value is exactly
    representable in the dtype the CUDA path takes (BF16 vectors and raw gate
    logits, FP32 decay / geometry rate), so the GPU consumes these vectors
    without a rounding step of its own; the FP64 oracle sees the same numbers."""
    gen = torch.Generator().manual_seed(seed)
    rn = lambda *s: torch.randn(*s, generator=gen, dtype=torch.float64)
    bf = lambda x: x.to(torch.bfloat16).to(torch.float64)
    f32 = lambda x: x.to(torch.float32).to(torch.float64)
    u, h, q = bf(rn(batch, length, heads, rank)), bf(rn(batch, length, heads, rank)), bf(rn(batch, length, heads, rank))
    keys = bf(rn(batch, length, heads, 1, rank))
    values = bf(rn(batch, length, heads, 1, value_dim))
    decay = f32(torch.nn.functional.logsigmoid(rn(batch, length, heads, rank) + 4.0))
    erase_raw = bf(rn(batch, length, heads, 1, rank))
    write_raw = bf(rn(batch, length, heads, 1, value_dim))
    gamma = f32(0.1 * torch.rand(batch, length, heads, generator=gen, dtype=torch.float64))
    RAW_GATES["erase_raw"], RAW_GATES["write_raw"] = erase_raw, write_raw
    return [u, h, q, keys, values, decay, torch.sigmoid(erase_raw), torch.sigmoid(write_raw), gamma]


def run_case(ref, name, args, *, state=None, valid=None, reset=None, seed=29, raw_gates=None):
    leaves = [a.clone().requires_grad_() for a in args]
    st = None
    if state is not None:
        st = ref.SolveDeltaState(*(s.clone().requires_grad_() for s in state))
    out, fin = ref.solvedelta_reference(
        *leaves, initial_state=st, valid_mask=valid, reset_mask=reset)
    gen = torch.Generator().manual_seed(seed)
    dy = torch.randn(out.shape, generator=gen, dtype=torch.float64)
    if raw_gates is not None:
        dy = dy.to(torch.bfloat16).to(torch.float64)
    dC = torch.randn(fin.predictor.shape, generator=gen, dtype=torch.float64)
    dS = torch.randn(fin.S.shape, generator=gen, dtype=torch.float64)
    loss = (out * dy).sum() + (fin.predictor * dC).sum() + (fin.S * dS).sum()
    wrt = leaves + (list(st) if st is not None else [])
    grads = torch.autograd.grad(loss, wrt)
    names = ["u", "h", "q", "keys", "values", "log_decay", "erase", "write", "geometry_write"]
    blob = {}
    for n, a in zip(names, args):
        blob["in_" + n] = a.numpy()
    for n, g_ in zip(names, grads[:9]):
        blob["grad_" + n] = g_.numpy()
    if st is not None:
        blob["in_C0"], blob["in_S0"] = state[0].numpy(), state[1].numpy()
        blob["grad_C0"], blob["grad_S0"] = grads[9].numpy(), grads[10].numpy()
    if raw_gates is not None:
        blob["in_erase_raw"] = raw_gates["erase_raw"].numpy()
        blob["in_write_raw"] = raw_gates["write_raw"].numpy()
    if valid is not None:
        blob["valid"] = valid.numpy()
    if reset is not None:
        blob["reset"] = reset.numpy()
    blob["dy"], blob["dC_T"], blob["dS_T"] = dy.numpy(), dC.numpy(), dS.numpy()
    blob["out"] = out.detach().numpy()
    blob["C_T"] = fin.predictor.detach().numpy()
    blob["S_T"] = fin.S.detach().numpy()
    np.savez_compressed(os.path.join(HERE, name + ".npz"), **blob)
    print(name, {k: v.shape for k, v in blob.items() if k.startswith("in_")})


def main():
    if len(sys.argv) < 2:
        raise SystemExit("usage: make_golden.py /path/to/SolveDelta")
    root = sys.argv[1]
    ref = load_reference(root)

    run_case(ref, "seed7_dense", seed7_inputs())

    args = seed7_inputs()
    args[-1] = torch.zeros_like(args[-1])
    run_case(ref, "seed7_zero_geometry", args)

    args = seed7_inputs(length=8)
    valid = torch.tensor([[1, 1, 0, 1, 1, 1, 1, 1], [1, 0, 1, 1, 1, 0, 1, 1]], dtype=torch.bool)
    reset = torch.zeros_like(valid)
    reset[0, 4] = True
    reset[1, 2] = True
    torch.manual_seed(31)
    state = (0.3 * torch.randn(2, 2, 8, 8, dtype=torch.float64),
             0.3 * torch.randn(2, 2, 8, 5, dtype=torch.float64))
    run_case(ref, "seed7_masks_resets_state", args, state=state, valid=valid, reset=reset)

    args = bench_like_inputs(1, 40, 2, 16, 12, seed=0)
    torch.manual_seed(131)
    state = ((0.02 * torch.randn(1, 2, 16, 16)).double(), (0.02 * torch.randn(1, 2, 16, 12)).double())
    run_case(ref, "benchlike_r16_state", args, state=state, raw_gates=dict(RAW_GATES))

    # chunk-spanning case for the chunked CUDA path: T=150 crosses two 64-token
    # chunk boundaries and ends on a ragged tail
    args = bench_like_inputs(1, 150, 1, 32, 32, seed=1)
    torch.manual_seed(137)
    state = ((0.02 * torch.randn(1, 1, 32, 32)).double(), (0.02 * torch.randn(1, 1, 32, 32)).double())
    run_case(ref, "benchlike_r32_t150_state", args, state=state, raw_gates=dict(RAW_GATES))


if __name__ == "__main__":
    main()
