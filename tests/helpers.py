"""Shared helpers for the parity tests."""
from __future__ import annotations

import glob
import os

import numpy as np

GOLDEN_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
OPERANDS = ("u", "h", "q", "keys", "values", "log_decay", "erase", "write", "geometry_write")


def golden_names():
    """Operator-level vectors (the mixer_* and model_* files hold whole-module vectors)."""
    names = sorted(os.path.basename(p)[:-4] for p in glob.glob(os.path.join(GOLDEN_DIR, "*.npz")))
    return [n for n in names if not n.startswith(("mixer_", "model_"))]


def load_golden(name):
    with np.load(os.path.join(GOLDEN_DIR, name + ".npz")) as z:
        return {k: z[k] for k in z.files}


def golden_inputs(g):
    return [g["in_" + n] for n in OPERANDS]


def golden_state(g):
    if "in_C0" in g:
        return (g["in_C0"], g["in_S0"])
    return None


def rel_l2(a, b):
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30))


def max_rel(a, b):
    """max|a-b| / max|b|: the 'max relative error' used for state tolerances."""
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    return float(np.abs(a - b).max() / max(np.abs(b).max(), 1e-30))
