"""Configuration of the mixer and of the causal LM around it, as a Hugging Face config.

Field names and defaults are those of upstream's ``SolveDeltaConfig``
(causallsso/config.py:8-80), so an upstream ``config.json`` loads unchanged and
``AutoConfig.for_model("solvedelta", ...)`` resolves to this class.  Fields that only
choose between implementations of the same arithmetic upstream (``fuse_norm``,
``fuse_swiglu``, ``fuse_cross_entropy``, ...) are accepted and kept as plain attributes;
hybrid attention layers (``attn``) are not built and are refused.
"""
from __future__ import annotations

import math
from typing import Any, Callable, Dict, Optional

from transformers import PreTrainedConfig


def _whole(optional: bool = False) -> Callable[[str, Any], None]:
    """A strictly positive int (bools are not ints here); None allowed when optional."""
    def check(name: str, value: Any) -> None:
        if value is None and optional:
            return
        if type(value) is not int:
            raise TypeError(f"{name}: expected an int{' or None' if optional else ''}, got {type(value).__name__}")
        if value < 1:
            raise ValueError(f"{name}: expected a value >= 1, got {value}")
    return check


def _positive_real(name: str, value: Any) -> None:
    if type(value) not in (int, float):
        raise TypeError(f"{name}: expected a real number, got {type(value).__name__}")
    if not (math.isfinite(value) and value > 0):
        raise ValueError(f"{name}: expected a finite value > 0, got {value}")


def _flag(name: str, value: Any) -> None:
    if type(value) is not bool:
        raise TypeError(f"{name}: expected True or False, got {type(value).__name__}")


def _activation(name: str, value: Any) -> None:
    if value not in ("swish", "powlu"):
        raise ValueError(f"{name}: {value!r} is not one of 'swish', 'powlu'")


def _no_hybrid_layers(name: str, value: Any) -> None:
    if value is not None:
        raise NotImplementedError("hybrid attention layers (attn) are not part of this package")


_RULES: Dict[str, Callable[[str, Any], None]] = {
    "hidden_size": _whole(), "num_heads": _whole(), "num_edits": _whole(), "num_hidden_layers": _whole(),
    "vocab_size": _whole(), "max_position_embeddings": _whole(),
    "head_k_dim": _whole(optional=True), "head_v_dim": _whole(optional=True),
    "intermediate_size": _whole(optional=True), "hidden_ratio": _whole(optional=True),
    "expand_k": _positive_real, "expand_v": _positive_real, "norm_eps": _positive_real,
    "initializer_range": _positive_real,
    "use_short_conv": _flag, "bias": _flag, "use_cache": _flag, "tie_word_embeddings": _flag,
    "hidden_act": _activation, "attn": _no_hybrid_layers,
    "fuse_norm": _flag, "fuse_swiglu": _flag, "fuse_cross_entropy": _flag, "fuse_linear_cross_entropy": _flag,
}


class SolveDeltaConfig(PreTrainedConfig):
    model_type = "solvedelta"
    keys_to_ignore_at_inference = ["past_key_values"]

    hidden_size: int = 2048
    num_heads: int = 16
    head_k_dim: Optional[int] = None
    head_v_dim: Optional[int] = None
    expand_k: float = 1.0
    expand_v: float = 1.0
    num_edits: int = 1
    use_short_conv: bool = True
    bias: bool = False
    num_hidden_layers: int = 24
    hidden_ratio: Optional[int] = 4
    intermediate_size: Optional[int] = None
    hidden_act: str = "swish"
    norm_eps: float = 1e-6
    max_position_embeddings: int = 2048
    attn: Optional[Any] = None
    use_cache: bool = True
    vocab_size: int = 32000
    initializer_range: float = 0.02
    pad_token_id: Optional[int] = None
    bos_token_id: Optional[int] = 1
    eos_token_id: Optional[int] = 2
    tie_word_embeddings: bool = False
    # implementation switches of upstream (config.py:34-37): the first two choose between owners of the same
    # arithmetic there and change nothing here (the fused kernels are used whenever the layout allows);
    # fuse_cross_entropy takes the loss from the two cross-entropy kernels on the BF16 logits instead of
    # F.cross_entropy on an FP32 copy; fuse_linear_cross_entropy makes the causal LM compute its loss through the
    # chunked linear + cross-entropy head and return no logits, as upstream does
    fuse_norm: bool = True
    fuse_swiglu: bool = True
    fuse_cross_entropy: bool = True
    fuse_linear_cross_entropy: bool = False

    def __post_init__(self, **kwargs):
        for name, rule in _RULES.items():
            rule(name, getattr(self, name))
        if self.fuse_cross_entropy and self.fuse_linear_cross_entropy:
            raise ValueError("fuse_cross_entropy and fuse_linear_cross_entropy are mutually exclusive")
        if self.num_edits != 1:
            raise ValueError("num_edits: the production path carries exactly one edit per token (num_edits=1)")
        self.head_width(self.head_k_dim, self.expand_k, "expand_k")
        self.head_width(self.head_v_dim, self.expand_v, "expand_v")
        super().__post_init__(**kwargs)

    def head_width(self, explicit: Optional[int], expand: float, name: str) -> int:
        """Width of one head: the explicit value, else hidden_size * expand split evenly over the heads."""
        if explicit is not None:
            return explicit
        total = self.hidden_size * expand
        whole = int(total + 0.5)
        if abs(total - whole) > 1e-9:
            raise ValueError(f"{name}: hidden_size * {name} = {total} is not a whole number of channels")
        per_head, rest = divmod(whole, self.num_heads)
        if rest:
            raise ValueError(f"{name}: {whole} channels do not split evenly over {self.num_heads} heads")
        return per_head

    @property
    def resolved_head_k_dim(self) -> int:
        return self.head_width(self.head_k_dim, self.expand_k, "expand_k")

    @property
    def resolved_head_v_dim(self) -> int:
        return self.head_width(self.head_v_dim, self.expand_v, "expand_v")

    @property
    def key_dim(self) -> int:
        return self.num_heads * self.resolved_head_k_dim

    @property
    def value_dim(self) -> int:
        return self.num_heads * self.resolved_head_v_dim


__all__ = ["SolveDeltaConfig"]
