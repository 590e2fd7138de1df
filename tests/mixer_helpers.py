"""Shared pieces of the mixer tests: golden loading and checker construction."""
import os

import numpy as np

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def load_mixer_golden(name):
    with np.load(os.path.join(GOLDEN, name + ".npz")) as z:
        return {k: z[k] for k in z.files}


def golden_config(g):
    cfg = {k[4:]: g[k].item() for k in g if k.startswith("cfg_")}
    cfg.setdefault("use_short_conv", True)
    cfg.setdefault("bias", False)
    return cfg


def golden_params(g):
    return {k[len("param_"):]: g[k] for k in g if k.startswith("param_")}


def oracle_from_golden(g):
    from oracle.mixer_oracle import MixerOracle

    cfg = golden_config(g)
    return MixerOracle(golden_params(g), hidden_size=cfg["hidden_size"], num_heads=cfg["num_heads"],
                       head_k_dim=cfg["head_k_dim"], head_v_dim=cfg["head_v_dim"],
                       use_short_conv=cfg["use_short_conv"], norm_eps=cfg["norm_eps"])
