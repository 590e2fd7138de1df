"""Hugging Face surface of the causal LM (upstream tests/model/test_modeling_solvedelta.py:69-79,136-184):
Auto* registration, config round trip, checkpoint round trip, FP32 parameter families under a BF16 load.
Building, saving and loading a model needs no GPU; only its forward pass does."""
import torch
from transformers import AutoConfig, AutoModel, AutoModelForCausalLM

from solvedelta_b200 import SolveDeltaConfig, SolveDeltaForCausalLM, SolveDeltaModel, SolveDeltaPreTrainedModel


def _tiny(**over):
    base = dict(hidden_size=32, num_heads=2, head_k_dim=16, head_v_dim=16, num_hidden_layers=2, vocab_size=48)
    base.update(over)
    return SolveDeltaConfig(**base)


def test_auto_registration_and_config_round_trip():
    config = _tiny(fuse_norm=True)   # an upstream-only switch: accepted and carried along
    again = SolveDeltaConfig.from_dict(config.to_dict())
    assert again.to_dict() == config.to_dict() and again.fuse_norm is True
    assert isinstance(AutoConfig.for_model("solvedelta", hidden_size=32, num_heads=2), SolveDeltaConfig)
    assert isinstance(AutoModel.from_config(config), SolveDeltaModel)
    lm = AutoModelForCausalLM.from_config(config)
    assert isinstance(lm, SolveDeltaForCausalLM) and isinstance(lm, SolveDeltaPreTrainedModel)
    assert lm.get_input_embeddings() is lm.model.embeddings and lm.get_output_embeddings() is lm.lm_head


def test_checkpoint_round_trip_keeps_values_and_fp32_families(tmp_path):
    torch.manual_seed(2)
    model = SolveDeltaForCausalLM(_tiny(num_hidden_layers=1))
    model.save_pretrained(tmp_path)
    restored = AutoModelForCausalLM.from_pretrained(tmp_path)
    assert isinstance(restored, SolveDeltaForCausalLM)
    want = model.state_dict()
    got = restored.state_dict()
    assert set(got) == set(want)
    for name, value in want.items():
        assert torch.equal(got[name], value), name
    half = AutoModelForCausalLM.from_pretrained(tmp_path, dtype=torch.bfloat16)
    mixer = half.model.layers[0].mixer.mixer
    assert mixer.in_proj.weight.dtype == torch.bfloat16 and half.lm_head.weight.dtype == torch.bfloat16
    for parameter in (mixer.geometry_write_bias, mixer.associative_log_rate, mixer.associative_decay_bias):
        assert parameter.dtype == torch.float32


def test_tied_embeddings_share_one_tensor(tmp_path):
    model = SolveDeltaForCausalLM(_tiny(num_hidden_layers=1, tie_word_embeddings=True))
    assert model.lm_head.weight is model.model.embeddings.weight
    model.save_pretrained(tmp_path)
    restored = SolveDeltaForCausalLM.from_pretrained(tmp_path)
    assert restored.lm_head.weight is restored.model.embeddings.weight
    assert torch.equal(restored.lm_head.weight, model.lm_head.weight)
