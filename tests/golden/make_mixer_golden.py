"""Regenerate tests/golden/mixer_*.npz from the upstream SolveDelta mixer.

Run where the upstream tree is mounted (its imports need torch, transformers
and fla; everything executes on the CPU branches):

    python tests/golden/make_mixer_golden.py /path/to/SolveDelta

The upstream ``causallsso.model.SolveDelta`` module is built in FP64 on small
seeded configurations, run once, and differentiated with torch.autograd.
Parameters, input, cotangents, output, final states and every gradient are
stored so the committed vectors pin the numpy mixer checker under ``oracle/``
(and through it the CUDA glue kernels) without the upstream tree.

The upstream CPU branch rounds the gate pre-activations to FP32
(causallsso/model.py:383-394,433-438), so an FP64 restatement agrees with
these vectors to about 1e-6, not to FP64 round-off.
"""
from __future__ import annotations

import os
import sys
import warnings

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))

CASES = {
    # name: (config kwargs, batch, length, with initial/final state)
    "mixer_small": (dict(hidden_size=64, num_heads=2, head_k_dim=16, head_v_dim=16), 2, 10, False),
    "mixer_small_state": (dict(hidden_size=64, num_heads=2, head_k_dim=16, head_v_dim=16), 2, 7, True),
    "mixer_noconv_bias": (dict(hidden_size=48, num_heads=3, head_k_dim=8, head_v_dim=16,
                               use_short_conv=False, bias=True), 1, 9, False),
    # valid / reset masks (pattern of upstream tests/core/test_rebuild_semantics.py:319-329 stretched to
    # 12 tokens, plus a row that opens invalid and a one-token segment), carried states
    "mixer_masks_state": (dict(hidden_size=64, num_heads=2, head_k_dim=16, head_v_dim=16), 3, 12, True),
}

MASKS = {
    "mixer_masks_state": (
        [[1, 1, 0, 1, 1, 1, 0, 0, 1, 1, 1, 1], [0, 0, 1, 1, 1, 1, 1, 0, 1, 1, 0, 0], [0] * 12],
        [[0, 0, 0, 1, 0, 0, 0, 1, 0, 0, 1, 1], [0, 0, 1, 0, 0, 0, 0, 0, 0, 1, 0, 0], [0] * 12]),
}


def make_case(name, SolveDelta, SolveDeltaConfig, SolveDeltaLayerState, SolveDeltaState):
    kwargs, batch, length, stateful = CASES[name]
    seed = sum(name.encode()) % 1000
    torch.manual_seed(seed)
    config = SolveDeltaConfig(num_hidden_layers=1, vocab_size=32, **kwargs)
    module = SolveDelta(config).double()
    with torch.no_grad():
        # Move the scalar parameters off their symmetric initial values so
        # every gradient is exercised.
        module.geometry_write_bias.add_(0.3 * torch.randn_like(module.geometry_write_bias))
        module.associative_log_rate.add_(0.3 * torch.randn_like(module.associative_log_rate))
        module.associative_decay_bias.add_(0.3 * torch.randn_like(module.associative_decay_bias))
        module.output_norm.weight.add_(0.2 * torch.randn_like(module.output_norm.weight))
        module.output_gate_proj.bias.add_(0.2 * torch.randn_like(module.output_gate_proj.bias))
        for lin in (module.in_proj, module.output_proj, module.decay_proj, module.output_gate_proj):
            lin.weight.mul_(4.0)
            if lin.bias is not None and lin is not module.output_gate_proj:
                lin.bias.add_(0.1 * torch.randn_like(lin.bias))
    heads, rank, vdim = config.num_heads, config.head_k_dim, config.head_v_dim
    x = torch.randn(batch, length, config.hidden_size, dtype=torch.float64, requires_grad=True)
    record = {"seed": np.int64(seed)}
    for key, value in kwargs.items():
        record["cfg_" + key] = np.asarray(value)
    record["cfg_norm_eps"] = np.asarray(config.norm_eps)
    leaves = {"x": x}
    masks = {}
    if name in MASKS:
        valid, reset = (torch.tensor(m, dtype=torch.bool) for m in MASKS[name])
        masks = dict(valid_mask=valid, reset_mask=reset)
        record["valid_mask"], record["reset_mask"] = valid.numpy(), reset.numpy()
    if stateful:
        c0 = (0.2 * torch.randn(batch, heads, rank, rank, dtype=torch.float64)).requires_grad_()
        s0 = (0.5 * torch.randn(batch, heads, rank, vdim, dtype=torch.float64)).requires_grad_()
        conv0 = torch.randn(batch, 2 * heads * rank + heads * vdim, 3, dtype=torch.float64).requires_grad_()
        leaves.update(C0=c0, S0=s0, conv0=conv0)
        initial = SolveDeltaLayerState(SolveDeltaState(c0, s0), conv0)
        out, final = module(x, initial_state=initial, return_final_state=True, **masks)
        cot = {"dout": torch.randn_like(out), "dC_T": torch.randn_like(final.operator.predictor),
               "dS_T": torch.randn_like(final.operator.S), "dconv_T": torch.randn_like(final.conv)}
        loss = ((out * cot["dout"]).sum() + (final.operator.predictor * cot["dC_T"]).sum()
                + (final.operator.S * cot["dS_T"]).sum() + (final.conv * cot["dconv_T"]).sum())
        record.update(C_T=final.operator.predictor.detach().numpy(), S_T=final.operator.S.detach().numpy(),
                      conv_T=final.conv.detach().numpy())
    else:
        out = module(x, **masks)
        cot = {"dout": torch.randn_like(out)}
        loss = (out * cot["dout"]).sum()
    loss.backward()
    record["out"] = out.detach().numpy()
    for key, value in cot.items():
        record[key] = value.numpy()
    for key, value in leaves.items():
        record["in_" + key] = value.detach().numpy()
        record["grad_" + key] = value.grad.numpy()
    for pname, param in module.named_parameters():
        record["param_" + pname] = param.detach().numpy()
        record["pgrad_" + pname] = (torch.zeros_like(param) if param.grad is None else param.grad).numpy()
    np.savez_compressed(os.path.join(HERE, name + ".npz"), **record)
    print(name, "out", tuple(out.shape), "params", sum(p.numel() for p in module.parameters()))


def main():
    root = sys.argv[1]
    sys.path.insert(0, root)
    warnings.filterwarnings("ignore")
    from causallsso.config import SolveDeltaConfig
    from causallsso.model import SolveDelta, SolveDeltaLayerState
    from causallsso.reference import SolveDeltaState

    for name in CASES:
        make_case(name, SolveDelta, SolveDeltaConfig, SolveDeltaLayerState, SolveDeltaState)


if __name__ == "__main__":
    main()
