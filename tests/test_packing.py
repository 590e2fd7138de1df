"""Segment plans (CPU): the same facts upstream's plan states, checked against a
plain Python walk over the masks (causallsso/ops/packing.py:43-150)."""
import pytest
import torch

from solvedelta_b200 import build_packed_segments, pack_tokens, unpack_tokens


def _walk(valid, reset):
    """Reference walk: list of (batch row, [token positions], uses_initial)."""
    segments, last = [], []
    for b in range(valid.shape[0]):
        current, first_in_row = None, True
        row_last = -1
        for t in range(valid.shape[1]):
            if not valid[b, t]:
                continue
            if current is None or reset[b, t]:
                current = [b, [], first_in_row and not bool(reset[b, t])]
                segments.append(current)
                first_in_row = False
            current[1].append(t)
            row_last = len(segments) - 1
        last.append(row_last)
    return segments, last


@pytest.mark.parametrize("seed", [0, 1, 2, 3])
def test_plan_matches_a_plain_walk(seed):
    gen = torch.Generator().manual_seed(seed)
    valid = torch.rand(4, 23, generator=gen) > 0.3
    reset = torch.rand(4, 23, generator=gen) > 0.8
    if seed == 2:
        valid[1] = False  # a batch row without any valid token
    plan = build_packed_segments(valid, reset)
    segments, last = _walk(valid, reset)
    assert plan.num_segments == len(segments)
    assert plan.num_tokens == int(valid.sum())
    assert plan.segment_batch.tolist() == [s[0] for s in segments]
    assert plan.segment_lengths.tolist() == [len(s[1]) for s in segments]
    assert plan.use_initial.tolist() == [s[2] for s in segments]
    assert plan.last_segment.tolist() == last
    assert plan.max_seqlen == max(len(s[1]) for s in segments)
    assert plan.cu_seqlens_cpu.tolist() == plan.cu_seqlens.tolist()
    flat = [b * 23 + t for b, ts, _ in segments for t in ts]
    assert plan.indices.tolist() == flat
    ids = [i for i, (_, ts, _) in enumerate(segments) for _ in ts]
    assert plan.segment_ids.tolist() == ids
    x = torch.randn(4, 23, 3, generator=gen)
    packed = pack_tokens(x, plan)
    assert packed.shape == (1, plan.num_tokens, 3)
    back = unpack_tokens(packed, plan)
    assert torch.equal(back[valid], x[valid]) and torch.equal(back[~valid], torch.zeros_like(back[~valid]))


def test_empty_plan_and_argument_errors():
    valid = torch.zeros(2, 5, dtype=torch.bool)
    plan = build_packed_segments(valid, torch.zeros_like(valid))
    assert plan.num_tokens == 0 and plan.num_segments == 0 and plan.max_seqlen == 0
    assert plan.last_segment.tolist() == [-1, -1]
    with pytest.raises(ValueError, match="valid_mask"):
        build_packed_segments(valid.float(), valid)
    with pytest.raises(ValueError, match="reset_mask"):
        build_packed_segments(valid, valid[:, :3])
