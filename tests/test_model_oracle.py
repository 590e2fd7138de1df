"""The numpy causal-LM checker against the vectors upstream's own model produced, and the
host-side logic of the shell (configuration, cache, masks) that needs no GPU."""
import numpy as np
import pytest
import torch

from oracle.model_oracle import ModelOracle
from solvedelta_b200 import SolveDeltaCache, SolveDeltaConfig, SolveDeltaForCausalLM
from solvedelta_b200.modeling import segment_reset_mask
from tests.helpers import load_golden

TOL = 5e-6  # upstream's CPU branch rounds the gate pre-activations to FP32


@pytest.fixture(scope="module")
def golden():
    z = load_golden("model_tiny")
    cfg = {k[4:]: z[k].item() for k in z if k.startswith("cfg_")}
    params = {k[6:]: z[k] for k in z if k.startswith("param_")}
    return z, cfg, params


def test_checker_reproduces_upstream_logits_and_loss(golden):
    z, cfg, params = golden
    oracle = ModelOracle(params, cfg)
    logits, loss, _ = oracle.forward(z["input_ids"], labels=z["input_ids"])
    assert np.abs(logits - z["logits"]).max() < TOL * max(1.0, np.abs(z["logits"]).max())
    assert abs(loss - float(z["loss"])) < TOL


def test_checker_cached_steps_match_upstream_cache(golden):
    z, cfg, params = golden
    oracle = ModelOracle(params, cfg)
    ids, prefill = z["input_ids"], int(z["prefill"])
    logits, _, cache = oracle.forward(ids[:, :prefill])
    pieces = [logits]
    for t in range(prefill, ids.shape[1]):
        logits, _, cache = oracle.forward(ids[:, t:t + 1], cache=cache)
        pieces.append(logits)
    got = np.concatenate(pieces, axis=1)
    scale = max(1.0, np.abs(z["logits_cached"]).max())
    assert np.abs(got - z["logits_cached"]).max() < TOL * scale
    for layer in range(cfg["num_hidden_layers"]):
        C, S = cache[layer]["recurrent_state"]
        assert np.abs(C - z[f"cache_{layer}_C"]).max() < TOL * max(1.0, np.abs(z[f"cache_{layer}_C"]).max())
        assert np.abs(S - z[f"cache_{layer}_S"]).max() < TOL * max(1.0, np.abs(z[f"cache_{layer}_S"]).max())
        assert np.abs(cache[layer]["conv_state"] - z[f"cache_{layer}_conv"]).max() < TOL * 10


def test_upstream_state_dict_loads_by_name(golden):
    z, cfg, params = golden
    model = SolveDeltaForCausalLM(SolveDeltaConfig(**cfg))
    model.load_state_dict({k: torch.from_numpy(v) for k, v in params.items()}, strict=True)
    assert model.model.layers[0].mlp.intermediate_size == cfg["intermediate_size"]
    assert sum(p.numel() for p in model.parameters()) == sum(v.size for v in params.values())


def test_configuration_validates_shell_fields():
    with pytest.raises(ValueError):
        SolveDeltaConfig(hidden_size=64, num_heads=2, vocab_size=0)
    with pytest.raises(TypeError):
        SolveDeltaConfig(hidden_size=64, num_heads=2, num_hidden_layers=1.5)
    with pytest.raises(ValueError):
        SolveDeltaConfig(hidden_size=64, num_heads=2, hidden_act="gelu")
    with pytest.raises(NotImplementedError):
        SolveDeltaConfig(hidden_size=64, num_heads=2, attn={"layers": [0]})
    config = SolveDeltaConfig(hidden_size=1024, num_heads=8)
    assert (config.num_hidden_layers, config.vocab_size, config.hidden_ratio) == (24, 32000, 4)
    # upstream's default MLP width: 2/3 * 4 * hidden, rounded up to a multiple of 256
    assert SolveDeltaForCausalLM(SolveDeltaConfig(hidden_size=128, num_heads=2, num_hidden_layers=1,
                                                  vocab_size=16)).model.layers[0].mlp.intermediate_size == 512


def test_cache_layout_and_legacy_round_trip():
    cache = SolveDeltaCache()
    assert len(cache) == 0 and cache.get_seq_length() == 0
    with pytest.raises(ValueError):
        cache.update(1, recurrent_state=(None, None), conv_state=None)
    cache.update(0, recurrent_state=("C", "S"), conv_state="conv", offset=5)
    cache.update(1, recurrent_state=("C1", "S1"), conv_state="conv1", offset=5)
    cache.update(0, recurrent_state=("C2", "S2"), conv_state="conv2", offset=1)
    assert cache.get_seq_length() == 6 and len(cache) == 2
    assert set(cache[0]) == {"recurrent_state", "attn_state", "conv_state", "ffn_state"}
    assert cache[0]["recurrent_state"] == ("C2", "S2")
    again = SolveDeltaCache.from_legacy_cache(cache.to_legacy_cache())
    assert again[1]["conv_state"] == "conv1"
    with pytest.raises(KeyError):
        cache[2]


def test_segment_reset_mask_marks_sequence_starts():
    hidden = torch.zeros(1, 10, 4)
    mask = segment_reset_mask(hidden, torch.tensor([0, 3, 7, 10], dtype=torch.int32))
    assert mask.tolist() == [[True, False, False, True, False, False, False, True, False, False]]
    with pytest.raises(ValueError):
        segment_reset_mask(torch.zeros(2, 10, 4), torch.tensor([0, 10]))
    with pytest.raises(TypeError):
        segment_reset_mask(hidden, torch.tensor([0.0, 10.0]))


def test_model_refuses_cpu_activations(golden):
    _, cfg, _ = golden
    model = SolveDeltaForCausalLM(SolveDeltaConfig(**cfg))
    with pytest.raises(TypeError):
        model(input_ids=torch.zeros(1, 4, dtype=torch.long))
