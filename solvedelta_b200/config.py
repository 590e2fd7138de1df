"""Configuration of the mixer and of the causal LM around it: the fields of
upstream's ``SolveDeltaConfig`` (causallsso/config.py:8-199) that this package
reads, with the same names, defaults, validation messages and head-width
resolution.  It is a plain object (no Hugging Face base class).  Switches that
only select between implementations of the same arithmetic upstream
(``fuse_norm``, ``fuse_swiglu``, ``fuse_cross_entropy``) are accepted and kept;
hybrid attention layers (``attn``) are not built and are refused."""
from __future__ import annotations

import math
from typing import Optional


class SolveDeltaConfig:
    model_type = "solvedelta"

    def __init__(self, hidden_size: int = 2048, num_heads: int = 16, head_k_dim: Optional[int] = None,
                 head_v_dim: Optional[int] = None, expand_k: float = 1.0, expand_v: float = 1.0,
                 num_edits: int = 1, use_short_conv: bool = True, bias: bool = False, *,
                 num_hidden_layers: int = 24, hidden_ratio: Optional[int] = 4,
                 intermediate_size: Optional[int] = None, hidden_act: str = "swish",
                 norm_eps: float = 1e-6, max_position_embeddings: int = 2048, attn=None, use_cache: bool = True,
                 vocab_size: int = 32000, initializer_range: float = 0.02, pad_token_id: Optional[int] = None,
                 bos_token_id: int = 1, eos_token_id: int = 2, tie_word_embeddings: bool = False,
                 **unused) -> None:
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
        self.num_hidden_layers = num_hidden_layers
        self.hidden_ratio = hidden_ratio
        self.intermediate_size = intermediate_size
        self.hidden_act = hidden_act
        self.max_position_embeddings = max_position_embeddings
        self.attn = attn
        self.use_cache = use_cache
        self.vocab_size = vocab_size
        self.initializer_range = initializer_range
        self.pad_token_id = pad_token_id
        self.bos_token_id = bos_token_id
        self.eos_token_id = eos_token_id
        self.tie_word_embeddings = tie_word_embeddings
        self.extra = dict(unused)  # implementation switches of upstream's shell: accepted and kept, not used
        self._validate()

    def _validate(self) -> None:
        for name in ("hidden_size", "num_heads", "num_edits", "num_hidden_layers", "vocab_size",
                     "max_position_embeddings"):
            value = getattr(self, name)
            if isinstance(value, bool) or not isinstance(value, int):
                raise TypeError(f"{name} must be an int, got {type(value).__name__}")
            if value <= 0:
                raise ValueError(f"{name} must be positive, got {value}")
        if self.num_edits != 1:
            raise ValueError("the current SolveDelta production contract requires num_edits=1")
        for name in ("head_k_dim", "head_v_dim", "intermediate_size"):
            value = getattr(self, name)
            if value is not None:
                if isinstance(value, bool) or not isinstance(value, int):
                    raise TypeError(f"{name} must be an int or None")
                if value <= 0:
                    raise ValueError(f"{name} must be positive, got {value}")
        if self.hidden_ratio is not None:
            if isinstance(self.hidden_ratio, bool) or not isinstance(self.hidden_ratio, int):
                raise TypeError("hidden_ratio must be an int or None")
            if self.hidden_ratio <= 0:
                raise ValueError("hidden_ratio must be positive")
        if self.hidden_act not in ("swish", "powlu"):
            raise ValueError(f"Unsupported hidden_act: {self.hidden_act}")
        if self.attn is not None:
            raise NotImplementedError("hybrid attention layers are not part of this package")
        for name in ("expand_k", "expand_v", "norm_eps", "initializer_range"):
            value = getattr(self, name)
            if isinstance(value, bool) or not isinstance(value, (int, float)):
                raise TypeError(f"{name} must be a real number")
            if not math.isfinite(float(value)) or value <= 0:
                raise ValueError(f"{name} must be finite and positive")
        for name in ("use_short_conv", "bias", "use_cache", "tie_word_embeddings"):
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
