"""CPU restatement (numpy, FP64) of the SolveDelta causal LM's forward pass.

TEST INFRASTRUCTURE: only tests/, the smoke check and the CPU leg of bench.py
may import this file; the product package never does.

Follows upstream ``causallsso/modeling_solvedelta.py``: embedding lookup
(:372-374), per block ``x + mixer(rmsnorm(x))`` then ``x + mlp(rmsnorm(x))``
(:231-255) with the packed gate/up swish MLP (:69-101), the final norm (:391),
the language-model head and the shifted-label mean cross entropy (:461-489);
the cache carries ``(C, S)`` and the three-token convolution tail per layer
(:104-115,184-192).  The mixer is ``oracle.mixer_oracle.MixerOracle``.
Pinned by tests/golden/model_tiny.npz, which upstream's own code produced.
"""
from __future__ import annotations

import numpy as np

from .mixer_oracle import MixerOracle

IGNORE_INDEX = -100


def rms_norm(x, weight, eps):
    """torch.nn.RMSNorm: x / sqrt(mean(x^2) + eps) * weight."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps) * weight


def swish_mlp(x, gate_up, down, rnd=lambda z: z):
    packed = rnd(x @ gate_up.T)
    gate, value = np.split(packed, 2, axis=-1)
    return rnd(rnd(rnd(gate / (1.0 + np.exp(-gate))) * value) @ down.T)


def shifted_cross_entropy(logits, labels):
    """Mean over the positions whose NEXT token is a label (modeling_solvedelta.py:473-489)."""
    shifted = np.concatenate([labels[:, 1:], np.full_like(labels[:, :1], IGNORE_INDEX)], axis=1).reshape(-1)
    flat = logits.reshape(-1, logits.shape[-1])
    keep = shifted != IGNORE_INDEX
    flat, shifted = flat[keep], shifted[keep]
    top = flat.max(axis=-1, keepdims=True)
    logz = top[:, 0] + np.log(np.exp(flat - top).sum(axis=-1))
    return float(np.mean(logz - flat[np.arange(flat.shape[0]), shifted]))


class ModelOracle:
    """``params``: upstream ``state_dict`` names -> arrays.  ``config``: dict with hidden_size,
    num_heads, head_k_dim, head_v_dim, num_hidden_layers, norm_eps (and use_short_conv)."""

    def __init__(self, params, config, activation_rounding=None):
        """``activation_rounding``: optional callable applied wherever a reduced-precision model
        stores an activation (residual stream, norm and projection outputs, MLP intermediates,
        logits; inside the mixer as ``MixerOracle`` documents).  None = exact FP64."""
        self.rnd = activation_rounding if activation_rounding is not None else (lambda z: z)
        self.p = {k: np.asarray(v, dtype=np.float64) for k, v in params.items()}
        self.cfg = dict(config)
        self.layers = int(config["num_hidden_layers"])
        self.eps = float(config.get("norm_eps", 1e-6))
        self.mixers = []
        for i in range(self.layers):
            prefix = f"model.layers.{i}.mixer.mixer."
            sub = {k[len(prefix):]: v for k, v in self.p.items() if k.startswith(prefix)}
            self.mixers.append(MixerOracle(
                sub, hidden_size=int(config["hidden_size"]), num_heads=int(config["num_heads"]),
                head_k_dim=int(config["head_k_dim"]), head_v_dim=int(config["head_v_dim"]),
                use_short_conv=bool(config.get("use_short_conv", True)), norm_eps=self.eps,
                activation_rounding=activation_rounding))

    def forward(self, input_ids, cache=None, labels=None):
        """Returns (logits, loss or None, new cache).  ``cache``: list per layer of
        {"recurrent_state": (C, S), "conv_state": conv} or None for a fresh sequence."""
        p, rnd = self.p, self.rnd
        x = p["model.embeddings.weight"][np.asarray(input_ids)]
        new_cache = []
        for i, mixer in enumerate(self.mixers):
            pre = f"model.layers.{i}."
            state = cache[i] if cache is not None else None
            operator_state = state["recurrent_state"] if state is not None else None
            conv_state = state["conv_state"] if state is not None else None
            mixed, fin, conv = mixer.forward(rnd(rms_norm(x, p[pre + "mixer_norm.weight"], self.eps)),
                                             conv_state=conv_state, operator_state=operator_state)
            x = rnd(x + rnd(mixed))
            x = rnd(x + swish_mlp(rnd(rms_norm(x, p[pre + "mlp_norm.weight"], self.eps)),
                                  p[pre + "mlp.gate_up_proj.weight"], p[pre + "mlp.down_proj.weight"], rnd))
            new_cache.append({"recurrent_state": tuple(fin), "conv_state": conv})
        x = rnd(rms_norm(x, p["model.norm.weight"], self.eps))
        logits = rnd(x @ p["lm_head.weight"].T)
        loss = None if labels is None else shifted_cross_entropy(logits, np.asarray(labels))
        return logits, loss, new_cache
