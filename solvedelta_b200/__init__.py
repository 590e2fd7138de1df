"""B200-native SolveDelta chunked recurrence (forward + full VJP).

Drop-in for the upstream operator entry points
(causallsso/ops/__init__.py:3, causallsso/ops/operator.py:13-26):
``solvedelta_native`` keeps its name, signature, dtype/stride contract,
error types and autograd behaviour; the arithmetic runs in hand-written
sm_100a CUDA kernels behind a C ABI (include/solvedelta_b200.h).
"""
from ._lib import build, load
from .config import SolveDeltaConfig
from .mixer_ops import conv4_silu, conv4_silu_segmented, kda_decay_gate, rms_norm_gated, rms_norm_gated_linear
from .model import RMSNormGated, SolveDelta, SolveDeltaLayerState
from .modeling import (GraphedDecoder, SolveDeltaBlock, SolveDeltaCache, SolveDeltaCacheAdapter, SolveDeltaForCausalLM,
                       SolveDeltaMLP, SolveDeltaModel, SolveDeltaPreTrainedModel)
from .training import (BF16ShadowWeights, BucketedGradientAverager, SolveDeltaGraphedTrainingStep,
                       allreduce_gradients, causal_lm_loss,
                       fixed_dense_linear_cross_entropy, fused_cross_entropy)
from .packing import PackedSegments, build_packed_segments, pack_tokens, unpack_tokens
from .ops import (
    SolveDeltaState,
    solvedelta_native,
    oja_residual,
    solvedelta_masked_native,
    solvedelta_segmented_native,
    solvedelta_residual_frame_native,
    solvedelta_zero_state,
)

# Hugging Face registration, as upstream's package import does (causallsso/__init__.py:23-50)
from transformers import AutoConfig, AutoModel, AutoModelForCausalLM

AutoConfig.register(SolveDeltaConfig.model_type, SolveDeltaConfig, exist_ok=True)
AutoModel.register(SolveDeltaConfig, SolveDeltaModel, exist_ok=True)
AutoModelForCausalLM.register(SolveDeltaConfig, SolveDeltaForCausalLM, exist_ok=True)

__all__ = [
    "SolveDeltaPreTrainedModel",
    "BF16ShadowWeights",
    "BucketedGradientAverager",
    "SolveDeltaGraphedTrainingStep",
    "allreduce_gradients",
    "causal_lm_loss",
    "fixed_dense_linear_cross_entropy",
    "fused_cross_entropy",
    "GraphedDecoder",
    "SolveDeltaBlock",
    "SolveDeltaCache",
    "SolveDeltaCacheAdapter",
    "SolveDeltaForCausalLM",
    "SolveDeltaMLP",
    "SolveDeltaModel",
    "SolveDelta",
    "SolveDeltaConfig",
    "SolveDeltaLayerState",
    "RMSNormGated",
    "conv4_silu",
    "conv4_silu_segmented",
    "kda_decay_gate",
    "rms_norm_gated",
    "rms_norm_gated_linear",
    "SolveDeltaState",
    "build",
    "load",
    "solvedelta_native",
    "oja_residual",
    "solvedelta_masked_native",
    "solvedelta_segmented_native",
    "solvedelta_residual_frame_native",
    "PackedSegments",
    "build_packed_segments",
    "pack_tokens",
    "unpack_tokens",
    "solvedelta_zero_state",
]
