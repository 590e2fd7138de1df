"""Mixer configuration: the subset of upstream's ``SolveDeltaConfig``
(causallsso/config.py:8-199) that the mixer reads, with the same field names,
defaults, validation messages and head-width resolution.  It is a plain
object (no Hugging Face base class): the CausalLM shell is not part of this
package."""
from __future__ import annotations

import math
from typing import Optional


class SolveDeltaConfig:
    model_type = "solvedelta"

    def __init__(self, hidden_size: int = 2048, num_heads: int = 16, head_k_dim: Optional[int] = None,
                 head_v_dim: Optional[int] = None, expand_k: float = 1.0, expand_v: float = 1.0,
                 num_edits: int = 1, use_short_conv: bool = True, bias: bool = False, *,
                 norm_eps: float = 1e-6, **unused) -> None:
        self.hidden_size = hidden_size
        self.num_heads = num_heads
        self.head_k_dim = head_k_dim
        self.head_v_dim = head_v_dim
        self.expand_k = expand_k
        self.expand_v = expand_v
        self.num_edits = num_edits
        self.use_short_conv = use_short_conv
        self.bias = bias
        self.norm_eps = norm_eps
        self.extra = dict(unused)  # fields of the CausalLM shell are accepted and kept, not used
        self._validate()

    def _validate(self) -> None:
        for name in ("hidden_size", "num_heads", "num_edits"):
            value = getattr(self, name)
            if isinstance(value, bool) or not isinstance(value, int):
                raise TypeError(f"{name} must be an int, got {type(value).__name__}")
            if value <= 0:
                raise ValueError(f"{name} must be positive, got {value}")
        if self.num_edits != 1:
            raise ValueError("the current SolveDelta production contract requires num_edits=1")
        for name in ("head_k_dim", "head_v_dim"):
            value = getattr(self, name)
            if value is not None:
                if isinstance(value, bool) or not isinstance(value, int):
                    raise TypeError(f"{name} must be an int or None")
                if value <= 0:
                    raise ValueError(f"{name} must be positive, got {value}")
        for name in ("expand_k", "expand_v", "norm_eps"):
            value = getattr(self, name)
            if isinstance(value, bool) or not isinstance(value, (int, float)):
                raise TypeError(f"{name} must be a real number")
            if not math.isfinite(float(value)) or value <= 0:
                raise ValueError(f"{name} must be finite and positive")
        for name in ("use_short_conv", "bias"):
            if not isinstance(getattr(self, name), bool):
                raise TypeError(f"{name} must be a bool, got {type(getattr(self, name)).__name__}")
        _ = self.resolved_head_k_dim
        _ = self.resolved_head_v_dim

    def _resolve_head_dim(self, explicit, expand, name) -> int:
        if explicit is not None:
            return explicit
        total_float = self.hidden_size * float(expand)
        total = round(total_float)
        if not math.isclose(total_float, total, rel_tol=0.0, abs_tol=1e-9):
            raise ValueError(f"hidden_size * {name} must be an integer, got {total_float}")
        if total % self.num_heads:
            raise ValueError(f"resolved total width {total} must be divisible by num_heads={self.num_heads}")
        return total // self.num_heads

    @property
    def resolved_head_k_dim(self) -> int:
        return self._resolve_head_dim(self.head_k_dim, self.expand_k, "expand_k")

    @property
    def resolved_head_v_dim(self) -> int:
        return self._resolve_head_dim(self.head_v_dim, self.expand_v, "expand_v")

    @property
    def key_dim(self) -> int:
        return self.num_heads * self.resolved_head_k_dim

    @property
    def value_dim(self) -> int:
        return self.num_heads * self.resolved_head_v_dim


__all__ = ["SolveDeltaConfig"]
