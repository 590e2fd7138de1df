"""The causal LM around the SolveDelta mixer and its decode cache.

Mirror of upstream ``causallsso/modeling_solvedelta.py:31-501`` for
attention-free models: the same module tree and parameter names
(``model.embeddings``, ``model.layers.N.{mixer_norm,mixer.mixer,mlp_norm,mlp}``,
``model.norm``, ``lm_head``), so an upstream ``state_dict`` loads as it is; the
same packed gate/up MLP, pre-norm residual blocks, label shift and loss; the
same cache entries per layer, ``{"recurrent_state": (C, S), "conv_state":
[B, D, 3]}``.  The mixer is this package's CUDA one, everything around it is
PyTorch (cuBLAS GEMMs, elementwise glue): activations are BF16 on a CUDA
device, and there is no CPU path.
"""
from __future__ import annotations

from typing import Any, Dict, List, Optional, Sequence, Tuple, Union

import torch
import torch.nn.functional as F
from torch import nn
from transformers import PreTrainedModel
from transformers.generation import GenerationMixin
from transformers.modeling_outputs import BaseModelOutputWithPast, CausalLMOutputWithPast

from . import _lib
from .config import SolveDeltaConfig
from .ops import SolveDeltaState
from .mixer_ops import add_rmsnorm, add_rmsnorm_reverse_supported, small_linear, swiglu
from .model import SolveDelta, SolveDeltaLayerState

FP32_PARAMETERS = ("geometry_write_bias", "associative_log_rate", "associative_decay_bias")


class SolveDeltaCache:
    """Per-layer decode state (the part of upstream's FLA ``Cache`` this model uses,
    modeling_solvedelta.py:104-115,184-192): ``cache[layer]`` is a dict with
    ``recurrent_state`` = (C [B,H,r,r], S [B,H,r,V]) and ``conv_state`` [B,D,3]."""

    def __init__(self) -> None:
        self.states: List[Dict[str, Any]] = []
        self._seen_tokens = 0

    @classmethod
    def from_legacy_cache(cls, past: Optional[Sequence[Dict[str, Any]]] = None) -> "SolveDeltaCache":
        cache = cls()
        if past is not None:
            cache.states = [dict(state) for state in past]
        return cache

    def to_legacy_cache(self) -> Tuple[Dict[str, Any], ...]:
        return tuple(self.states)

    def __getitem__(self, layer_idx: int) -> Dict[str, Any]:
        if layer_idx >= len(self.states):
            raise KeyError(f"Cache only has {len(self.states)} layers, attempted to access layer {layer_idx}")
        return self.states[layer_idx]

    def __len__(self) -> int:
        return len(self.states)

    def __iter__(self):
        return iter(self.states)

    def get_seq_length(self, layer_idx: int = 0) -> int:
        return self._seen_tokens if len(self.states) > layer_idx else 0

    def layer_state(self, layer_idx: int) -> Optional[SolveDeltaLayerState]:
        """What layer ``layer_idx`` continues from: None while the cache has nothing for it."""
        if layer_idx >= len(self.states):
            return None
        entry = self.states[layer_idx]
        pair = entry.get("recurrent_state")
        if pair is None:
            return None
        try:
            predictor, memory = pair
        except (TypeError, ValueError):
            raise ValueError("SolveDelta cache recurrent_state must contain (predictor,S)") from None
        return SolveDeltaLayerState(operator=SolveDeltaState(predictor, memory), conv=entry.get("conv_state"))

    def update(self, layer_idx: int, recurrent_state, conv_state, offset: int = 1) -> Dict[str, Any]:
        if layer_idx == 0:
            self._seen_tokens += offset
        state = {"recurrent_state": recurrent_state, "attn_state": None, "conv_state": conv_state,
                 "ffn_state": None}
        if layer_idx < len(self.states):
            self.states[layer_idx] = state
        elif layer_idx == len(self.states):
            self.states.append(state)
        else:
            raise ValueError("cache layers must be filled in order")
        return state


def segment_reset_mask(hidden_states: torch.Tensor, cu_seqlens: torch.Tensor) -> torch.Tensor:
    """Packed batch [1,T,D] with sequence boundaries ``cu_seqlens`` -> bool [1,T], True on the first token
    of every sequence (what upstream's ``_segment_reset_mask`` returns, modeling_solvedelta.py:118-134)."""
    if cu_seqlens.dtype not in (torch.int32, torch.int64):
        raise TypeError("cu_seqlens must have int32 or int64 dtype")
    if cu_seqlens.ndim != 1 or cu_seqlens.numel() < 2:
        raise ValueError("cu_seqlens must be one-dimensional with at least two entries")
    rows, tokens = hidden_states.shape[:2]
    if rows != 1:
        raise ValueError("explicit cu_seqlens require packed hidden states [1,T,D]")
    mask = hidden_states.new_zeros(tokens, dtype=torch.bool)
    mask[cu_seqlens[:-1].to(hidden_states.device, torch.long)] = True
    return mask.unsqueeze(0)


class SolveDeltaMLP(nn.Module):
    """Gated MLP with one common-input gate/up projection (modeling_solvedelta.py:31-101)."""

    def __init__(self, hidden_size: int, hidden_ratio: Optional[int] = None,
                 intermediate_size: Optional[int] = None, hidden_act: str = "swish",
                 powglu_power: float = 3.0) -> None:
        super().__init__()
        if hidden_ratio is None:
            hidden_ratio = 4
        if intermediate_size is None:
            intermediate_size = int(hidden_size * hidden_ratio * 2 / 3)
            intermediate_size = 256 * ((intermediate_size + 255) // 256)
        if hidden_act not in ("swish", "powlu"):
            raise ValueError(f"Unsupported hidden_act: {hidden_act}")
        self.hidden_size = hidden_size
        self.hidden_ratio = hidden_ratio
        self.intermediate_size = intermediate_size
        self.hidden_act = hidden_act
        self.powglu_power = powglu_power
        self.gate_up_proj = nn.Linear(hidden_size, 2 * intermediate_size, bias=False)
        self.down_proj = nn.Linear(intermediate_size, hidden_size, bias=False)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if self.hidden_act == "swish" and x.is_cuda and x.dtype == torch.bfloat16:
            # a cached single-token step: projection + activation in one launch, then the second projection
            act = small_linear(x, self.gate_up_proj.weight, self.gate_up_proj.bias, swiglu=True)
            if act is None:
                act = swiglu(self.gate_up_proj(x))   # activation and product in one kernel
            out = small_linear(act, self.down_proj.weight, self.down_proj.bias)
            return out if out is not None else self.down_proj(act)
        gate, value = self.gate_up_proj(x).chunk(2, dim=-1)
        if self.hidden_act == "swish":
            activated = F.silu(gate)
        else:
            sigmoid = torch.sigmoid(gate)
            positive = gate > 0
            safe = torch.where(positive, gate, torch.ones_like(gate))
            exponent = self.powglu_power / (torch.sqrt(safe) + 1.0)
            activated = torch.where(positive, torch.exp(exponent * torch.log(safe)) * sigmoid, gate * sigmoid)
        return self.down_proj(activated * value)


class SolveDeltaCacheAdapter(nn.Module):
    """Layer/cache boundary around the mixer (modeling_solvedelta.py:137-194): attention mask ->
    valid mask, ``cu_seqlens`` -> reset mask, cache entry <-> ``SolveDeltaLayerState``."""

    def __init__(self, config: SolveDeltaConfig, layer_idx: int) -> None:
        super().__init__()
        self.layer_idx = layer_idx
        self.mixer = SolveDelta(config)

    @staticmethod
    def _valid_tokens(attention_mask: Optional[torch.Tensor], batch: int, length: int) -> Optional[torch.Tensor]:
        """The attention mask covers the whole history; the mixer wants the columns of the current tokens."""
        if attention_mask is None:
            return None
        if attention_mask.ndim != 2 or attention_mask.shape[0] != batch:
            raise ValueError("attention_mask must have shape [B,T]")
        if attention_mask.shape[1] < length:
            raise ValueError("attention_mask is shorter than the current input")
        return attention_mask[:, attention_mask.shape[1] - length:].bool()

    @staticmethod
    def _reset_tokens(hidden_states: torch.Tensor, continuing: bool, options: Dict[str, Any]) -> Optional[torch.Tensor]:
        """An explicit ``solvedelta_reset_mask`` wins; otherwise ``cu_seqlens`` marks the sequence starts.  When
        the call continues a cached state, the boundary at token 0 that ``cu_seqlens`` always lists is not a reset."""
        resets = options.get("solvedelta_reset_mask")
        boundaries = options.get("cu_seqlens")
        if resets is None:
            if boundaries is None:
                return None
            resets = segment_reset_mask(hidden_states, boundaries)
        if resets.dtype != torch.bool or tuple(resets.shape) != tuple(hidden_states.shape[:2]):
            raise ValueError("solvedelta_reset_mask must be bool [B,T]")
        if continuing and boundaries is not None:
            resets = resets.clone()
            resets[0, 0] = False
        return resets

    def forward(self, hidden_states: torch.Tensor, attention_mask: Optional[torch.Tensor] = None,
                past_key_values: Optional[SolveDeltaCache] = None, use_cache: Optional[bool] = False,
                **kwargs) -> Tuple[torch.Tensor, Optional[SolveDeltaCache]]:
        batch, length = hidden_states.shape[:2]
        carried = None if past_key_values is None else past_key_values.layer_state(self.layer_idx)
        keep_state = past_key_values is not None and bool(use_cache)
        # a cached single-token step without gradients updates the cache's own tensors in place
        inplace = keep_state and carried is not None and length == 1 and not torch.is_grad_enabled()
        mixed = self.mixer(hidden_states, initial_state=carried,
                           valid_mask=self._valid_tokens(attention_mask, batch, length),
                           reset_mask=self._reset_tokens(hidden_states, carried is not None, kwargs),
                           return_final_state=keep_state, inplace_state=inplace)
        if not keep_state:
            return mixed, past_key_values
        output, after = mixed
        past_key_values.update(self.layer_idx, recurrent_state=tuple(after.operator), conv_state=after.conv,
                               offset=length)
        return output, past_key_values


def _fp32_weight(norm: nn.Module) -> torch.Tensor:
    """The weight the fused add + norm kernel takes: the parameter itself while gradients are recorded (so that it
    receives one), else a contiguous FP32 copy, refreshed when the weight changes."""
    weight = norm.weight
    if torch.is_grad_enabled() and weight.requires_grad:
        return weight
    if weight.dtype == torch.float32 and weight.is_contiguous():
        return weight.detach()
    key = (weight.data_ptr(), weight._version)
    hit = norm.__dict__.get("_fp32_weight_copy")
    if hit is None or hit[0] != key:
        hit = (key, weight.detach().float().contiguous())
        norm.__dict__["_fp32_weight_copy"] = hit
    return hit[1]


class SolveDeltaBlock(nn.Module):
    """Pre-norm residual block: mixer, then MLP (modeling_solvedelta.py:197-255)."""

    def __init__(self, config: SolveDeltaConfig, layer_idx: int) -> None:
        super().__init__()
        self.config = config
        self.layer_idx = layer_idx
        self.mixer_norm = nn.RMSNorm(config.hidden_size, eps=config.norm_eps)
        self.mixer = SolveDeltaCacheAdapter(config, layer_idx)
        self.mlp_norm = nn.RMSNorm(config.hidden_size, eps=config.norm_eps)
        self.mlp = SolveDeltaMLP(hidden_size=config.hidden_size, hidden_ratio=config.hidden_ratio,
                                 intermediate_size=config.intermediate_size, hidden_act=config.hidden_act)

    @staticmethod
    def fuses(hidden_states: torch.Tensor) -> bool:
        """BF16 CUDA activations: residual adds are folded into the norms that follow them (with gradients recorded,
        for the row widths the reverse kernel takes)."""
        if not (hidden_states.is_cuda and hidden_states.dtype == torch.bfloat16):
            return False
        return not torch.is_grad_enabled() or add_rmsnorm_reverse_supported(hidden_states.shape[-1])

    def forward(self, hidden_states: torch.Tensor, attention_mask: Optional[torch.Tensor] = None,
                past_key_values: Optional[SolveDeltaCache] = None, use_cache: Optional[bool] = False,
                pending: Optional[torch.Tensor] = None, defer_add: bool = False,
                **kwargs):
        """``pending``: the previous block's MLP output, not yet added to ``hidden_states`` (it is added inside this
        block's first norm kernel).  ``defer_add``: return ``(residual, mlp_output, cache)`` and leave the last add
        to the next norm.  Both are only used on the fused path (``fuses``)."""
        fused = self.fuses(hidden_states) and self.mixer_norm.weight is not None and self.mlp_norm.weight is not None
        if pending is not None or (fused and add_rmsnorm_reverse_supported(hidden_states.shape[-1])):
            hidden_states, normed = add_rmsnorm(hidden_states, pending, _fp32_weight(self.mixer_norm),
                                                self.mixer_norm.eps if self.mixer_norm.eps is not None else 1e-6)
            residual, hidden_states = hidden_states, normed
        else:
            residual = hidden_states
            hidden_states = self.mixer_norm(hidden_states)
        hidden_states, past_key_values = self.mixer(hidden_states, attention_mask=attention_mask,
                                                    past_key_values=past_key_values, use_cache=use_cache,
                                                    **kwargs)
        if fused and hidden_states.dtype == torch.bfloat16:
            # the residual add and the norm that follows it in one kernel
            residual, hidden_states = add_rmsnorm(residual, hidden_states, _fp32_weight(self.mlp_norm),
                                                  self.mlp_norm.eps if self.mlp_norm.eps is not None else 1e-6)
        else:
            hidden_states = residual + hidden_states
            residual = hidden_states
            hidden_states = self.mlp_norm(hidden_states)
        hidden_states = self.mlp(hidden_states)
        if defer_add:
            return residual, hidden_states, past_key_values
        return residual + hidden_states, past_key_values


class SolveDeltaPreTrainedModel(PreTrainedModel):
    """Hugging Face base of the two model classes (upstream: modeling_solvedelta.py:259-281): checkpoint
    save / load, ``Auto*`` construction, dtype handling.  The three scalar parameter families of the mixer
    stay FP32 whatever dtype a checkpoint is loaded in."""

    config_class = SolveDeltaConfig
    base_model_prefix = "model"
    supports_gradient_checkpointing = False
    _no_split_modules = ["SolveDeltaBlock"]
    _keep_in_fp32_modules_strict = list(FP32_PARAMETERS)

    def _init_weights(self, module: nn.Module) -> None:
        # projections and embeddings: N(0, initializer_range); the mixer sets its own gate parameters when built
        std = self.config.initializer_range
        if isinstance(module, (nn.Linear, nn.Embedding)):
            nn.init.normal_(module.weight, mean=0.0, std=std)
        if isinstance(module, nn.Linear) and module.bias is not None:
            nn.init.zeros_(module.bias)
        if isinstance(module, nn.Embedding) and module.padding_idx is not None:
            with torch.no_grad():
                module.weight[module.padding_idx].zero_()


class SolveDeltaModel(SolveDeltaPreTrainedModel):
    """Embedding, the stack of blocks, final norm (modeling_solvedelta.py:283-397)."""

    def __init__(self, config: SolveDeltaConfig) -> None:
        super().__init__(config)
        self.padding_idx = config.pad_token_id
        self.vocab_size = config.vocab_size
        self.embeddings = nn.Embedding(config.vocab_size, config.hidden_size, self.padding_idx)
        self.layers = nn.ModuleList(SolveDeltaBlock(config, i) for i in range(config.num_hidden_layers))
        self.norm = nn.RMSNorm(config.hidden_size, eps=config.norm_eps)
        self.post_init()

    def get_input_embeddings(self):
        return self.embeddings

    def set_input_embeddings(self, value):
        self.embeddings = value

    def forward(self, input_ids: Optional[torch.Tensor] = None, attention_mask: Optional[torch.Tensor] = None,
                inputs_embeds: Optional[torch.Tensor] = None,
                past_key_values: Union[SolveDeltaCache, Sequence[Dict[str, Any]], None] = None,
                use_cache: Optional[bool] = None, output_hidden_states: bool = False,
                **kwargs) -> BaseModelOutputWithPast:
        if input_ids is not None and inputs_embeds is not None:
            raise ValueError("specify either input_ids or inputs_embeds, not both")
        if input_ids is None and inputs_embeds is None:
            raise ValueError("input_ids or inputs_embeds is required")
        if use_cache is None:
            use_cache = self.config.use_cache if not self.training else False
        hidden_states = self.embeddings(input_ids) if inputs_embeds is None else inputs_embeds
        if use_cache and not isinstance(past_key_values, SolveDeltaCache):
            past_key_values = SolveDeltaCache.from_legacy_cache(past_key_values)
        elif not use_cache:
            past_key_values = None
        cu_seqlens = kwargs.get("cu_seqlens")
        if cu_seqlens is not None and "solvedelta_reset_mask" not in kwargs:
            kwargs["solvedelta_reset_mask"] = segment_reset_mask(hidden_states, cu_seqlens)
        collected = () if output_hidden_states else None
        # every block leaves its last residual add to the norm kernel that follows it
        defer = SolveDeltaBlock.fuses(hidden_states) and not output_hidden_states and self.norm.weight is not None
        pending = None
        for layer in self.layers:
            if output_hidden_states:
                collected += (hidden_states,)
            if defer:
                hidden_states, pending, past_key_values = layer(
                    hidden_states, attention_mask=attention_mask, past_key_values=past_key_values,
                    use_cache=use_cache, pending=pending, defer_add=True, **kwargs)
            else:
                hidden_states, past_key_values = layer(hidden_states, attention_mask=attention_mask,
                                                       past_key_values=past_key_values, use_cache=use_cache,
                                                       **kwargs)
        if pending is not None:
            _, hidden_states = add_rmsnorm(hidden_states, pending, _fp32_weight(self.norm),
                                           self.norm.eps if self.norm.eps is not None else 1e-6)
        else:
            hidden_states = self.norm(hidden_states)
        if output_hidden_states:
            collected += (hidden_states,)
        return BaseModelOutputWithPast(last_hidden_state=hidden_states, past_key_values=past_key_values,
                                       hidden_states=collected)


class SolveDeltaForCausalLM(SolveDeltaPreTrainedModel, GenerationMixin):
    """Language-model head, label shift and loss over ``SolveDeltaModel``
    (modeling_solvedelta.py:393-501).  ``prepare()`` puts a freshly built or loaded
    model into the layout the CUDA mixer wants: BF16 weights on the device, the three
    scalar parameter families of every mixer kept in FP32.

    ``generate`` is Hugging Face's (``GenerationMixin``): the prefill returns a ``SolveDeltaCache``, which the
    generation loop hands back with one new token at a time; no key/value cache is ever built
    (upstream mixes in FLA's generation adapter for the same purpose, modeling_solvedelta.py:393-395).
    ``greedy_generate`` is this package's own loop, with the option of replaying the cached step from a CUDA graph."""

    ignore_index = -100
    _tied_weights_keys = {"lm_head.weight": "model.embeddings.weight"}

    def __init__(self, config: SolveDeltaConfig) -> None:
        super().__init__(config)
        self.model = SolveDeltaModel(config)
        self.vocab_size = config.vocab_size
        self.lm_head = nn.Linear(config.hidden_size, config.vocab_size, bias=False)
        self.post_init()

    def prepare(self, device: Union[str, torch.device] = "cuda") -> "SolveDeltaForCausalLM":
        self.to(device)
        for name, parameter in self.named_parameters():
            keep = name.rsplit(".", 1)[-1] in FP32_PARAMETERS
            parameter.data = parameter.data.to(torch.float32 if keep else torch.bfloat16)
        return self

    @classmethod
    def _supports_default_dynamic_cache(cls) -> bool:
        return False   # the recurrent cache comes out of the prefill; generate() must not build a key/value cache

    def get_input_embeddings(self):
        return self.model.embeddings

    def get_output_embeddings(self):
        return self.lm_head

    def set_output_embeddings(self, value):
        self.lm_head = value

    def forward(self, input_ids: Optional[torch.Tensor] = None, attention_mask: Optional[torch.Tensor] = None,
                inputs_embeds: Optional[torch.Tensor] = None,
                past_key_values: Union[SolveDeltaCache, Sequence[Dict[str, Any]], None] = None,
                labels: Optional[torch.Tensor] = None, use_cache: Optional[bool] = None,
                output_hidden_states: bool = False, logits_to_keep: Optional[int] = 0,
                **kwargs) -> CausalLMOutputWithPast:
        outputs = self.model(input_ids=input_ids, attention_mask=attention_mask, inputs_embeds=inputs_embeds,
                             past_key_values=past_key_values, use_cache=use_cache,
                             output_hidden_states=output_hidden_states, **kwargs)
        hidden_states = outputs.last_hidden_state
        keep_all = labels is not None or logits_to_keep in (None, 0)
        fused_head = labels is not None and self.config.fuse_linear_cross_entropy
        logits = None
        if not fused_head:
            logits = self.lm_head(hidden_states if keep_all else hidden_states[:, -logits_to_keep:])
        loss = None
        if labels is not None:
            labels = labels.to(hidden_states.device)
            shifted = torch.cat((labels[..., 1:], torch.full_like(labels[:, :1], self.ignore_index)), dim=1)
            if fused_head:
                # head and loss in token chunks, the [tokens, vocab] logits never exist at once and none are
                # returned (modeling_solvedelta.py:460-483); the mean's denominator is counted on the device
                from .training import fixed_dense_linear_cross_entropy

                count = (shifted != self.ignore_index).sum().clamp_min(1)
                loss = fixed_dense_linear_cross_entropy(hidden_states, shifted, self.lm_head.weight,
                                                        self.lm_head.bias, ignore_index=self.ignore_index,
                                                        total=count)
            elif self.config.fuse_cross_entropy and logits.is_cuda and logits.dtype == torch.bfloat16:
                from .training import fused_cross_entropy   # two kernels on the BF16 logits, no FP32 copy

                loss = fused_cross_entropy(logits, shifted, ignore_index=self.ignore_index)
            else:
                loss = F.cross_entropy(logits.reshape(-1, logits.shape[-1]).float(), shifted.reshape(-1),
                                       ignore_index=self.ignore_index)
        return CausalLMOutputWithPast(loss=loss, logits=logits, past_key_values=outputs.past_key_values,
                                      hidden_states=outputs.hidden_states)

    @torch.no_grad()
    def greedy_generate(self, input_ids: torch.Tensor, max_new_tokens: int, graphed: bool = False) -> torch.Tensor:
        """Greedy decoding through the cache: one prefill, then one-token steps (replayed from a
        CUDA graph when ``graphed``)."""
        step = self(input_ids=input_ids, use_cache=True, logits_to_keep=1)
        cache, tokens = step.past_key_values, [input_ids]
        logits = step.logits
        decoder = GraphedDecoder(self, cache, input_ids.shape[0]) if graphed and max_new_tokens > 0 else None
        for _ in range(max_new_tokens):
            nxt = logits[:, -1].argmax(dim=-1, keepdim=True)
            tokens.append(nxt)
            if decoder is not None:
                logits = decoder.step(nxt)
            else:
                logits = self(input_ids=nxt, past_key_values=cache, use_cache=True, logits_to_keep=1).logits
        _lib.check_device_fault()   # one synchronisation at the end of the loop: every bounded wait completed
        return torch.cat(tokens, dim=1)


class GraphedDecoder:
    """One-token cached steps replayed from a CUDA graph.

    A decode step is a few hundred small launches (24 layers of projections, glue kernels and the
    one-token operator kernel), so its cost at small batch is launch and host time.  The step is captured
    once on static buffers (token ids in, logits out, the cache updated in place inside the graph) and
    replayed per token.  Build it from the cache a prefill returned; ``cache`` stays valid and current."""

    def __init__(self, model: "SolveDeltaForCausalLM", cache: SolveDeltaCache, batch: int) -> None:
        self.model = model
        device = next(model.parameters()).device
        self.token = torch.zeros(batch, 1, dtype=torch.long, device=device)
        self.cache = cache
        # static storage for every state; the cache entries point at it from now on
        self.static = []
        for state in cache.states:
            C, S = state["recurrent_state"]
            entry = (C.clone(), S.clone(), None if state["conv_state"] is None else state["conv_state"].clone())
            self.static.append(entry)
        self._point_cache_at_static()
        seen = cache._seen_tokens
        side = torch.cuda.Stream(device=device)
        side.wait_stream(torch.cuda.current_stream(device))
        with torch.cuda.stream(side), torch.no_grad():
            backup = [tuple(None if t is None else t.clone() for t in entry) for entry in self.static]
            for _ in range(2):          # warm-up: lazy initialisation must not fall inside the capture
                self._step()
            for entry, saved in zip(self.static, backup):
                for t, b in zip(entry, saved):
                    if t is not None:
                        t.copy_(b)
        torch.cuda.current_stream(device).wait_stream(side)
        self.graph = torch.cuda.CUDAGraph()
        with torch.no_grad(), torch.cuda.graph(self.graph):
            self.logits = self._step()
        # the capture itself executes nothing; undo the bookkeeping of warm-up and capture
        cache._seen_tokens = seen

    def _point_cache_at_static(self) -> None:
        for state, (C, S, conv) in zip(self.cache.states, self.static):
            state["recurrent_state"] = (C, S)
            state["conv_state"] = conv

    def _step(self) -> torch.Tensor:
        out = self.model(input_ids=self.token, past_key_values=self.cache, use_cache=True, logits_to_keep=1)
        for state, (C, S, conv) in zip(self.cache.states, self.static):
            new_C, new_S = state["recurrent_state"]
            if new_C.data_ptr() != C.data_ptr():   # the step updates the static tensors in place when it can
                C.copy_(new_C)
            if new_S.data_ptr() != S.data_ptr():
                S.copy_(new_S)
            if conv is not None and state["conv_state"].data_ptr() != conv.data_ptr():
                conv.copy_(state["conv_state"])
        self._point_cache_at_static()
        return out.logits

    def step(self, token: torch.Tensor) -> torch.Tensor:
        """``token`` [B,1] -> logits [B,1,vocab] (a static buffer: read it before the next step)."""
        self.token.copy_(token)
        self.graph.replay()
        self.cache._seen_tokens += 1
        return self.logits


__all__ = ["GraphedDecoder", "SolveDeltaBlock", "SolveDeltaCache", "SolveDeltaCacheAdapter", "SolveDeltaForCausalLM",
           "SolveDeltaMLP", "SolveDeltaModel", "SolveDeltaPreTrainedModel", "segment_reset_mask"]
