"""The causal LM on the GPU: against the vectors upstream's own model produced (tiny
configuration), against the numpy checker on BF16-rounded weights, and through the
properties upstream tests on the full model (cached continuation == single pass,
packed sequences == separate sequences)."""
import numpy as np
import pytest
import torch

from oracle.model_oracle import ModelOracle
from solvedelta_b200 import SolveDeltaConfig, SolveDeltaForCausalLM
from solvedelta_b200.modeling import FP32_PARAMETERS
from tests.helpers import load_golden, rel_l2

pytestmark = pytest.mark.gpu

# Relative L2 of whole tensors.  Activations and weights are BF16 end to end: on the tiny golden
# configuration (64 wide) the numpy checker, made to round where the device stores BF16, already
# sits 2.5e-2 from upstream's FP64 logits, so the device is held to 2e-2 against that checker and
# to 4e-2 against the FP64 vectors; gradients cross the model twice (measured 2e-2 to 7e-2, the
# decay-gate families of the first layer, where the operator's admissible error meets cancellation,
# 1.2e-1) and are held to 1.5e-1 with the direction (cosine) to 0.99.
LOGIT_TOL = 2e-2
FP64_LOGIT_TOL = 4e-2
GRAD_TOL = 1.5e-1
GRAD_COS = 0.99


def _bf16_round(a):
    return torch.from_numpy(np.asarray(a, dtype=np.float64)).to(torch.bfloat16).double().numpy()


@pytest.fixture(scope="module")
def tiny():
    z = load_golden("model_tiny")
    cfg = {k[4:]: z[k].item() for k in z if k.startswith("cfg_")}
    params = {k[6:]: z[k] for k in z if k.startswith("param_")}
    model = SolveDeltaForCausalLM(SolveDeltaConfig(**cfg))
    model.load_state_dict({k: torch.from_numpy(v) for k, v in params.items()}, strict=True)
    model.prepare("cuda")
    rounded = {k: (v if k.rsplit(".", 1)[-1] in FP32_PARAMETERS else _bf16_round(v)) for k, v in params.items()}
    return z, cfg, params, rounded, model


def test_prepare_keeps_scalar_families_in_fp32(tiny):
    *_, model = tiny
    for name, p in model.named_parameters():
        want = torch.float32 if name.rsplit(".", 1)[-1] in FP32_PARAMETERS else torch.bfloat16
        assert p.dtype == want and p.is_cuda, name


def test_logits_and_loss_match_upstream_vectors(tiny):
    z, cfg, params, rounded, model = tiny
    ids = torch.from_numpy(z["input_ids"]).cuda()
    model.train()
    out = model(input_ids=ids, labels=ids)
    logits = out.logits.detach().float().cpu().numpy()
    assert rel_l2(logits, z["logits"]) < FP64_LOGIT_TOL
    assert abs(out.loss.item() - float(z["loss"])) < 3e-2
    # the checker on the weights the device really holds, rounding where the device stores BF16
    want, want_loss, _ = ModelOracle(rounded, cfg, activation_rounding=_bf16_round).forward(
        z["input_ids"], labels=z["input_ids"])
    assert rel_l2(logits, want) < LOGIT_TOL
    assert abs(out.loss.item() - want_loss) < 1e-2


def test_parameter_gradients_match_upstream_vectors(tiny):
    z, cfg, params, rounded, model = tiny
    ids = torch.from_numpy(z["input_ids"]).cuda()
    model.train()
    model.zero_grad(set_to_none=True)
    model(input_ids=ids, labels=ids).loss.backward()
    report, bad = [], []
    for name, p in model.named_parameters():
        want = z["pgrad_" + name].astype(np.float64)
        got = p.grad.double().cpu().numpy()
        err = rel_l2(got, want)
        cos = float((got * want).sum() / max(np.linalg.norm(got) * np.linalg.norm(want), 1e-300))
        report.append(f"{name:55s} rel={err:.3e} cos={cos:.5f}")
        # the geometry-rate bias is one scalar per head summed over all tokens with heavy cancellation: on this
        # 12-token model its error moves between 0.13 and 0.18 with nothing but the rounding order of the
        # operator's (in-tolerance) per-token gradients, so it gets a wider bound; the direction is held as tightly
        tol = 2.5e-1 if name.endswith("geometry_write_bias") else GRAD_TOL
        if err > tol or cos < GRAD_COS:
            bad.append(name)
    print("\n".join(report))
    assert not bad, "gradients off: " + ", ".join(bad) + "\n" + "\n".join(report)


def test_cached_steps_match_upstream_vectors(tiny):
    z, cfg, params, rounded, model = tiny
    ids = torch.from_numpy(z["input_ids"]).cuda()
    prefill = int(z["prefill"])
    model.eval()
    with torch.no_grad():
        step = model(input_ids=ids[:, :prefill], use_cache=True)
        cache, pieces = step.past_key_values, [step.logits]
        for t in range(prefill, ids.shape[1]):
            step = model(input_ids=ids[:, t:t + 1], past_key_values=cache, use_cache=True)
            cache = step.past_key_values
            pieces.append(step.logits)
    got = torch.cat(pieces, dim=1).float().cpu().numpy()
    assert rel_l2(got, z["logits_cached"]) < FP64_LOGIT_TOL
    assert cache.get_seq_length() == ids.shape[1] and len(cache) == cfg["num_hidden_layers"]
    for layer in range(cfg["num_hidden_layers"]):
        C, S = cache[layer]["recurrent_state"]
        assert C.dtype == torch.float32 and S.dtype == torch.float32
        # twelve tokens of BF16 inputs into 16-wide states
        assert rel_l2(C.cpu().numpy(), z[f"cache_{layer}_C"]) < 6e-2
        assert rel_l2(S.cpu().numpy(), z[f"cache_{layer}_S"]) < 6e-2
        assert rel_l2(cache[layer]["conv_state"].float().cpu().numpy(), z[f"cache_{layer}_conv"]) < 2e-2


@pytest.fixture(scope="module")
def medium():
    torch.manual_seed(5)
    config = SolveDeltaConfig(hidden_size=256, num_heads=2, head_k_dim=64, head_v_dim=128, num_hidden_layers=3,
                              vocab_size=512, initializer_range=0.05)
    return config, SolveDeltaForCausalLM(config).prepare("cuda").eval()


def test_cached_continuation_equals_single_pass(medium):
    """Prefill, a block, then one-token steps reproduce the single pass (upstream tests/model:235-301)."""
    config, model = medium
    ids = torch.randint(0, config.vocab_size, (2, 300), device="cuda")
    with torch.no_grad():
        full = model(input_ids=ids).logits.float()
        step = model(input_ids=ids[:, :200], use_cache=True)
        cache, pieces = step.past_key_values, [step.logits]
        step = model(input_ids=ids[:, 200:290], past_key_values=cache, use_cache=True)
        pieces.append(step.logits)
        for t in range(290, 300):
            step = model(input_ids=ids[:, t:t + 1], past_key_values=step.past_key_values, use_cache=True)
            pieces.append(step.logits)
    got = torch.cat(pieces, dim=1).float()
    assert rel_l2(got.cpu().numpy(), full.cpu().numpy()) < LOGIT_TOL
    assert (got.argmax(-1) == full.argmax(-1)).float().mean().item() > 0.97


def test_packed_sequences_equal_separate_sequences(medium):
    config, model = medium
    lengths = [70, 130, 45]
    seqs = [torch.randint(0, config.vocab_size, (1, n), device="cuda") for n in lengths]
    packed = torch.cat(seqs, dim=1)
    cu = torch.tensor([0, 70, 200, 245], dtype=torch.int32, device="cuda")
    with torch.no_grad():
        together = model(input_ids=packed, cu_seqlens=cu).logits.float()
        apart = torch.cat([model(input_ids=s).logits.float() for s in seqs], dim=1)
    # The two runs round differently all the way (other GEMM shapes, and the packed run keeps its sequences
    # inside shared 64-token chunks, where a reset is carried as forgetting, instead of one chunk grid per
    # sequence): each is within LOGIT_TOL of the exact result, so their difference gets 1.5 x that.
    assert rel_l2(together.cpu().numpy(), apart.cpu().numpy()) < 1.5 * LOGIT_TOL


def test_padding_mask_leaves_valid_tokens_unchanged(medium):
    config, model = medium
    ids = torch.randint(0, config.vocab_size, (2, 96), device="cuda")
    mask = torch.ones(2, 96, dtype=torch.bool, device="cuda")
    mask[1, :20] = False  # left padding on the second row
    with torch.no_grad():
        masked = model(input_ids=ids, attention_mask=mask).logits.float()
        alone = model(input_ids=ids[1:, 20:]).logits.float()
    err = rel_l2(masked[1:, 20:].cpu().numpy(), alone.cpu().numpy())
    print(f"padded row against the same tokens alone: rel {err:.3e}")
    # the padded row sits 20 tokens into its first 64-token chunk and shares GEMM shapes with another row: the
    # two runs round differently at every step, each within LOGIT_TOL of the exact result
    assert err < 1.5 * LOGIT_TOL


def test_greedy_generation_follows_the_single_pass(medium):
    config, model = medium
    prompt = torch.randint(0, config.vocab_size, (2, 50), device="cuda")
    out = model.greedy_generate(prompt, max_new_tokens=6)
    assert out.shape == (2, 56) and torch.equal(out[:, :50], prompt)
    with torch.no_grad():
        logits = model(input_ids=out[:, :-1]).logits.float()
    # each generated token is (up to BF16 ties) the argmax of the single pass over its prefix
    agree = (logits[:, 49:].argmax(-1) == out[:, 50:]).float().mean().item()
    assert agree >= 5 / 6


def test_hugging_face_generate_runs_on_the_recurrent_cache(medium):
    """``GenerationMixin.generate`` (greedy) drives prefill + cached one-token steps and returns what the
    package's own loop returns; with left padding it is given the attention mask and still continues each row."""
    config, model = medium
    prompt = torch.randint(3, config.vocab_size, (2, 40), device="cuda")
    own = model.greedy_generate(prompt, max_new_tokens=8)
    hf = model.generate(prompt, max_new_tokens=8, min_new_tokens=8, do_sample=False)
    assert hf.shape == (2, 48) and torch.equal(hf[:, :40], prompt)
    # the two loops run the same kernels on the same tokens (BF16 ties can flip an argmax, then the rows diverge)
    assert (hf[:, :42] == own[:, :42]).all()
    mask = torch.ones_like(prompt)
    mask[1, :9] = 0
    padded = model.generate(prompt, attention_mask=mask, max_new_tokens=4, min_new_tokens=4, do_sample=False,
                            pad_token_id=0)
    assert padded.shape == (2, 44) and torch.equal(padded[0, :42], hf[0, :42])


def test_graphed_decode_equals_eager_decode(medium):
    """The captured one-token step, replayed, gives what the eager cached steps give, and leaves
    the cache where they leave it."""
    config, model = medium
    prompt = torch.randint(0, config.vocab_size, (2, 77), device="cuda")
    eager = model.greedy_generate(prompt, max_new_tokens=12)
    graphed = model.greedy_generate(prompt, max_new_tokens=12, graphed=True)
    assert torch.equal(eager, graphed)
    from solvedelta_b200 import GraphedDecoder

    with torch.no_grad():
        a = model(input_ids=prompt, use_cache=True, logits_to_keep=1)
        b = model(input_ids=prompt, use_cache=True, logits_to_keep=1)
        decoder = GraphedDecoder(model, b.past_key_values, 2)
        token = a.logits[:, -1].argmax(-1, keepdim=True)
        cache = a.past_key_values
        for _ in range(5):
            want = model(input_ids=token, past_key_values=cache, use_cache=True, logits_to_keep=1).logits
            got = decoder.step(token)
            assert torch.equal(got, want)
            token = want[:, -1].argmax(-1, keepdim=True)
    assert b.past_key_values.get_seq_length() == cache.get_seq_length() == 82
    for x, y in zip(cache, b.past_key_values):
        assert torch.equal(x["recurrent_state"][0], y["recurrent_state"][0])
        assert torch.equal(x["recurrent_state"][1], y["recurrent_state"][1])
        assert torch.equal(x["conv_state"], y["conv_state"])


def test_training_step_reduces_the_loss(medium):
    config, _ = medium
    torch.manual_seed(9)
    model = SolveDeltaForCausalLM(config).prepare("cuda").train()
    ids = torch.randint(0, config.vocab_size, (2, 128), device="cuda")
    master = [p.detach().float().clone() for p in model.parameters()]
    losses = []
    for _ in range(8):
        model.zero_grad(set_to_none=True)
        loss = model(input_ids=ids, labels=ids).loss
        loss.backward()
        losses.append(loss.item())
        with torch.no_grad():
            for p, m in zip(model.parameters(), master):
                m.add_(p.grad.float(), alpha=-0.05)
                p.copy_(m.to(p.dtype))
    assert all(np.isfinite(losses)) and losses[-1] < losses[0] - 0.05, losses


def _fresh_medium(seed):
    torch.manual_seed(seed)
    config = SolveDeltaConfig(hidden_size=256, num_heads=2, head_k_dim=64, head_v_dim=128, num_hidden_layers=2,
                              vocab_size=512, initializer_range=0.05)
    return config, SolveDeltaForCausalLM(config).prepare("cuda").train()


def test_chunked_fixed_denominator_loss_equals_the_model_loss():
    from solvedelta_b200 import causal_lm_loss

    config, model = _fresh_medium(3)
    ids = torch.randint(0, config.vocab_size, (2, 96), device="cuda")
    plain = model(input_ids=ids, labels=ids).loss
    plain.backward()
    want = [p.grad.float().clone() for p in model.parameters()]
    model.zero_grad(set_to_none=True)
    fused = causal_lm_loss(model, ids, ids, total=2 * 95, num_chunks=5)
    fused.backward()
    assert abs(fused.item() - plain.item()) < 2e-3
    # the chunked head hands the logit cotangent on in BF16 where the plain loss keeps FP32 logits; the
    # few-element parameter families (per-head biases and rates) show it most (4e-2 measured)
    for (name, p), w in zip(model.named_parameters(), want):
        assert rel_l2(p.grad.float().cpu().numpy(), w.cpu().numpy()) < (2e-2 if p.numel() >= 1024 else 8e-2), name


def test_graphed_training_step_equals_the_eager_step():
    from solvedelta_b200 import SolveDeltaGraphedTrainingStep, causal_lm_loss

    config, model = _fresh_medium(4)
    ids = [torch.randint(0, config.vocab_size, (2, 128), device="cuda") for _ in range(3)]
    step = SolveDeltaGraphedTrainingStep(model, ids[0], ids[0], num_chunks=4)
    assert all(p.grad is not None and not p.grad.any() for p in model.parameters())
    # two replays accumulate two micro-batches
    loss_a = step(ids[1], ids[1]).clone()
    loss_b = step(ids[2], ids[2]).clone()
    got = [p.grad.clone() for p in model.parameters()]
    model.zero_grad(set_to_none=True)
    want_a = causal_lm_loss(model, ids[1], ids[1], total=2 * 127, num_chunks=4)
    want_a.backward()
    want_b = causal_lm_loss(model, ids[2], ids[2], total=2 * 127, num_chunks=4)
    want_b.backward()
    assert loss_a.item() == want_a.item() and loss_b.item() == want_b.item()
    for (name, p), g in zip(model.named_parameters(), got):
        assert torch.equal(p.grad, g), name   # same kernels in the same order: bit-equal
    with pytest.raises(ValueError):
        step(ids[1][:, :64], ids[1][:, :64])
    with pytest.raises(TypeError):
        step(ids[1].int(), ids[1])
    model.eval()
    with pytest.raises(RuntimeError):
        step(ids[1], ids[1])


def test_graphed_steps_with_master_weights_train():
    from solvedelta_b200 import BF16ShadowWeights, SolveDeltaGraphedTrainingStep

    config, model = _fresh_medium(6)
    ids = torch.randint(0, config.vocab_size, (2, 128), device="cuda")
    shadows = BF16ShadowWeights(model, lambda masters: torch.optim.AdamW(masters, lr=2e-3, fused=True))
    step = SolveDeltaGraphedTrainingStep(model, ids, ids)
    losses = []
    for _ in range(10):
        losses.append(step(ids, ids).item())
        shadows.optimizer.step()
        shadows.assert_current()
    assert all(np.isfinite(losses)) and losses[-1] < losses[0] - 0.3, losses
    assert shadows.nbytes == 4 * sum(p.numel() for p in model.parameters())


def test_long_prefill_then_decode_steps_equal_one_pass_through_the_model():
    """The long-context configuration on a two-layer model (upstream tests/model/test_modeling_solvedelta.py:264-301):
    a 32 768-token prefill at B=1 with use_cache, then 256 cached one-token steps, against one pass over all
    33 024 tokens: the per-layer (C, S) cache and the logits of the 256 tokens."""
    torch.manual_seed(11)
    # initializer_range 0.02: with the 0.05 of the short tests this random model's memory grows without bound
    # over tens of thousands of tokens (|S| passes 1e19 by token 8192), which is the model, not the kernels
    config = SolveDeltaConfig(hidden_size=256, num_heads=2, head_k_dim=64, head_v_dim=128, num_hidden_layers=2,
                              vocab_size=512, initializer_range=0.02)
    model = SolveDeltaForCausalLM(config).prepare("cuda").eval()
    prefill, steps = 32768, 256
    ids = torch.randint(0, config.vocab_size, (1, prefill + steps), device="cuda")
    with torch.no_grad():
        full = model(input_ids=ids, use_cache=True)
        step = model(input_ids=ids[:, :prefill], use_cache=True, logits_to_keep=1)
        pieces = []
        for t in range(prefill, prefill + steps):
            step = model(input_ids=ids[:, t:t + 1], past_key_values=step.past_key_values, use_cache=True)
            pieces.append(step.logits)
    got = torch.cat(pieces, dim=1).float().cpu().numpy()
    want = full.logits[:, prefill:].float().cpu().numpy()
    assert np.isfinite(want).all()
    assert rel_l2(got, want) < 1.5 * LOGIT_TOL
    assert step.past_key_values.get_seq_length() == prefill + steps
    for layer in range(config.num_hidden_layers):
        C, S = step.past_key_values[layer]["recurrent_state"]
        Cf, Sf = full.past_key_values[layer]["recurrent_state"]
        # FP32 states fed by BF16 activations that the two runs round differently (other GEMM shapes, the
        # recurrent step instead of the chunk kernels for the last 256 tokens): BF16-grade agreement
        assert rel_l2(C.cpu().numpy(), Cf.cpu().numpy()) < 2e-2
        assert rel_l2(S.cpu().numpy(), Sf.cpu().numpy()) < 2e-2


def test_fused_linear_cross_entropy_head_gives_the_same_loss_and_gradients():
    """``fuse_linear_cross_entropy`` (modeling_solvedelta.py:460-483): the loss comes from the chunked
    linear + cross-entropy head, no logits are returned, and loss and gradients equal the plain head's."""
    def build(fused):
        torch.manual_seed(9)
        config = SolveDeltaConfig(hidden_size=128, num_heads=2, head_k_dim=32, head_v_dim=64, num_hidden_layers=2,
                                  vocab_size=300, initializer_range=0.05, fuse_cross_entropy=not fused,
                                  fuse_linear_cross_entropy=fused)
        return SolveDeltaForCausalLM(config).prepare("cuda").train()

    ids = torch.randint(0, 300, (2, 90), generator=torch.Generator().manual_seed(1)).cuda()
    labels = ids.clone()
    labels[1, 60:] = -100
    plain, fused = build(False), build(True)
    out_p = plain(input_ids=ids, labels=labels)
    out_f = fused(input_ids=ids, labels=labels)
    assert out_f.logits is None and out_p.logits is not None
    assert abs(float(out_p.loss.detach()) - float(out_f.loss.detach())) < 2e-3 * float(out_p.loss.detach())
    out_p.loss.backward()
    out_f.loss.backward()
    for (name, a), (_, b) in zip(plain.named_parameters(), fused.named_parameters()):
        scale = float(a.grad.float().abs().max().clamp_min(1e-12))
        assert float((a.grad.float() - b.grad.float()).abs().max()) <= 3e-2 * scale, name


def test_fused_single_token_step_equals_the_separate_kernels(medium, monkeypatch):
    """A cached one-token step runs conv, decay gate, geometry rate and the recurrent step as ONE launch
    that updates the cache in place; with that path switched off the separate kernels give the same logits
    and leave the same cache."""
    from solvedelta_b200.model import SolveDelta

    config, model = medium
    ids = torch.randint(0, config.vocab_size, (2, 70), device="cuda")

    def run(fused):
        if not fused:
            monkeypatch.setattr(SolveDelta, "_fused_decode_applies", lambda self, *a, **k: False)
        with torch.no_grad():
            step = model(input_ids=ids[:, :60], use_cache=True)
            cache, logits = step.past_key_values, []
            for t in range(60, 70):
                step = model(input_ids=ids[:, t:t + 1], past_key_values=cache, use_cache=True)
                logits.append(step.logits.float())
        monkeypatch.undo()
        return torch.cat(logits, 1), cache

    fused_logits, fused_cache = run(True)
    plain_logits, plain_cache = run(False)
    # conv, gate and geometry rate repeat the separate kernels' expressions; the fused norm sums its row in
    # another order, so from the second layer on the two runs round differently (BF16 activations)
    assert rel_l2(fused_logits[:, :1].cpu().numpy(), plain_logits[:, :1].cpu().numpy()) < 3e-3
    assert rel_l2(fused_logits.cpu().numpy(), plain_logits.cpu().numpy()) < LOGIT_TOL
    for a, b in zip(fused_cache.states, plain_cache.states):
        for x, y in zip(a["recurrent_state"], b["recurrent_state"]):
            assert float((x - y).abs().max()) <= 2e-2 * float(y.abs().max())
        assert float((a["conv_state"].float() - b["conv_state"].float()).abs().max()) <= \
            3e-2 * float(b["conv_state"].float().abs().max())


@pytest.mark.parametrize("rows,vocab", [(37, 1003), (64, 32000), (5, 8)])
def test_fused_cross_entropy_matches_pytorch_on_float32_logits(rows, vocab):
    from solvedelta_b200 import fused_cross_entropy

    gen = torch.Generator().manual_seed(rows + vocab)
    logits = (3.0 * torch.randn(rows, vocab, generator=gen)).to(torch.bfloat16).cuda()
    labels = torch.randint(0, vocab, (rows,), generator=gen).cuda()
    labels[::5] = -100
    got_in = logits.clone().requires_grad_()
    got = fused_cross_entropy(got_in, labels, ignore_index=-100)
    (2.0 * got).backward()
    want_in = logits.float().requires_grad_()
    want = torch.nn.functional.cross_entropy(want_in, labels, ignore_index=-100)
    (2.0 * want).backward()
    assert abs(got.item() - want.item()) <= 2e-4 * max(1.0, abs(want.item()))
    assert got_in.grad.dtype == torch.bfloat16
    err = (got_in.grad.float() - want_in.grad).abs().max().item()
    assert err <= 1e-2 * want_in.grad.abs().max().item()
    assert not got_in.grad[::5].any()
    # no counted token: zero loss and zero gradient
    none = fused_cross_entropy(logits.clone().requires_grad_(), torch.full_like(labels, -100))
    assert none.item() == 0.0
    with pytest.raises(TypeError):
        fused_cross_entropy(logits, labels.int())
