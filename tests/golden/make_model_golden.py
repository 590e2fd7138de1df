"""Regenerate tests/golden/model_tiny.npz from the upstream SolveDelta causal LM.

Run where the upstream tree is mounted (imports need torch, transformers and
fla; everything executes on the CPU branches, in FP64):

    python tests/golden/make_model_golden.py /path/to/SolveDelta

The installed fla release predates three names that upstream's
``causallsso/modeling_solvedelta.py:12-18`` imports; none of them takes part in
the arithmetic of an attention-free, swish-MLP model, so the script registers
stand-ins before the import: ``fla.models.hybrid.get_hybrid_attention_spec``
(answers "no attention layer", what upstream's returns for ``attn=None``),
``FLAUnsupportedCacheGenerationMixin`` (an empty mixin) and the ``powglu``
activations (unused with ``hidden_act="swish"``).  Everything else, the
blocks, the cache adapter, the label shift and the loss, is upstream's own
code (``modeling_solvedelta.py:31-501``).

Stored: configuration, every parameter, token ids, full-pass logits and loss
(labels = ids), the gradient of the loss with respect to every parameter, the
logits of a 7-token prefill followed by five one-token cached steps, and the
cache after them (``recurrent_state`` (C, S) and ``conv_state`` per layer).
"""
from __future__ import annotations

import os
import sys
import types
import warnings

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))

CONFIG = dict(hidden_size=64, num_heads=2, head_k_dim=16, head_v_dim=16, num_hidden_layers=2, vocab_size=32,
              hidden_ratio=4, initializer_range=0.2, norm_eps=1e-6,
              fuse_norm=False, fuse_swiglu=False, fuse_cross_entropy=False, fuse_linear_cross_entropy=False)
BATCH, LENGTH, PREFILL = 2, 12, 7


def _stand_ins():
    import fla.models.utils as fla_utils
    import fla.modules.activations as activations

    hybrid = types.ModuleType("fla.models.hybrid")
    hybrid.get_hybrid_attention_spec = lambda attn, layer_idx=None: None
    sys.modules.setdefault("fla.models.hybrid", hybrid)
    if not hasattr(fla_utils, "FLAUnsupportedCacheGenerationMixin"):
        fla_utils.FLAUnsupportedCacheGenerationMixin = type("FLAUnsupportedCacheGenerationMixin", (), {})
    for name in ("powglu", "powglu_linear"):
        if not hasattr(activations, name):
            setattr(activations, name, None)


def main():
    root = sys.argv[1]
    sys.path.insert(0, root)
    warnings.filterwarnings("ignore")
    _stand_ins()
    from causallsso.config import SolveDeltaConfig
    from causallsso.modeling_solvedelta import SolveDeltaForCausalLM

    torch.manual_seed(20)
    config = SolveDeltaConfig(**CONFIG)
    model = SolveDeltaForCausalLM(config).double()
    with torch.no_grad():
        for name, param in model.named_parameters():
            if name.endswith("norm.weight"):
                param.add_(0.2 * torch.randn_like(param))
    ids = torch.randint(0, config.vocab_size, (BATCH, LENGTH))
    record = {"input_ids": ids.numpy(), "prefill": np.int64(PREFILL)}
    for key, value in CONFIG.items():
        record["cfg_" + key] = np.asarray(value)
    record["cfg_intermediate_size"] = np.asarray(model.model.layers[0].mlp.intermediate_size)

    model.train()
    out = model(input_ids=ids, labels=ids)
    out.loss.backward()
    record["logits"] = out.logits.detach().numpy()
    record["loss"] = np.float64(out.loss.item())
    for name, param in model.named_parameters():
        record["param_" + name] = param.detach().numpy()
        record["pgrad_" + name] = (torch.zeros_like(param) if param.grad is None else param.grad).float().numpy()

    model.eval()
    with torch.no_grad():
        step = model(input_ids=ids[:, :PREFILL], use_cache=True)
        cache, pieces = step.past_key_values, [step.logits]
        for t in range(PREFILL, LENGTH):
            step = model(input_ids=ids[:, t:t + 1], past_key_values=cache, use_cache=True)
            cache = step.past_key_values
            pieces.append(step.logits)
    record["logits_cached"] = torch.cat(pieces, dim=1).numpy()
    for layer in range(config.num_hidden_layers):
        state = cache[layer]
        record[f"cache_{layer}_C"] = state["recurrent_state"][0].numpy()
        record[f"cache_{layer}_S"] = state["recurrent_state"][1].numpy()
        record[f"cache_{layer}_conv"] = state["conv_state"].numpy()
    np.savez_compressed(os.path.join(HERE, "model_tiny.npz"), **record)
    gap = np.abs(record["logits_cached"] - record["logits"]).max()
    print("model_tiny: loss %.6f, logits %s, cached-vs-single-pass gap %.2e, %d parameters"
          % (record["loss"], record["logits"].shape, gap, sum(p.numel() for p in model.parameters())))


if __name__ == "__main__":
    main()
