"""Reset-delimited segment plan for masked / packed batches.

Same public surface as causallsso/ops/packing.py:12-41 (``PackedSegments``,
``build_packed_segments``, ``pack_tokens``, ``unpack_tokens``): valid tokens of
a ``[B,T]`` batch are cut into segments at batch-row boundaries and at reset
tokens; every segment is a reset-free sequence that the dense operator can run
as one batch row.  Building the plan needs the segment count and the longest
segment on the host, so it performs exactly one small device-to-host transfer
(as upstream, packing.py:127-133); everything else stays on the device.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch


@dataclass(frozen=True)
class PackedSegments:
    """Plan shared by every consumer of one (valid_mask, reset_mask) pair."""

    batch: int
    length: int
    indices: torch.Tensor          # [N] flat positions (b*T + t) of the valid tokens, ascending
    segment_ids: torch.Tensor      # [N] segment of every valid token
    segment_batch: torch.Tensor    # [S] batch row of every segment
    use_initial: torch.Tensor      # [S] segment continues the caller's initial state
    segment_lengths: torch.Tensor  # [S] int32
    cu_seqlens: torch.Tensor       # [S+1] on the mask's device
    cu_seqlens_cpu: torch.Tensor   # [S+1] host mirror
    segment_batch_cpu: torch.Tensor
    use_initial_cpu: torch.Tensor
    last_segment: torch.Tensor     # [B] last segment of each batch row, -1 if the row has none
    valid_mask: torch.Tensor = None  # the two bool [B,T] masks the plan was built from: the operator
    reset_mask: torch.Tensor = None  # kernels read them directly (the gathers above serve the conv)

    @property
    def num_tokens(self) -> int:
        return self.indices.shape[0]

    @property
    def num_segments(self) -> int:
        return self.segment_batch.shape[0]

    @property
    def max_seqlen(self) -> int:
        if self.num_segments == 0:
            return 0
        return int((self.cu_seqlens_cpu[1:] - self.cu_seqlens_cpu[:-1]).max().item())


def build_packed_segments(valid_mask: torch.Tensor, reset_mask: torch.Tensor) -> PackedSegments:
    if valid_mask.ndim != 2 or valid_mask.dtype != torch.bool:
        raise ValueError("valid_mask must be bool [B,T]")
    if reset_mask.shape != valid_mask.shape or reset_mask.dtype != torch.bool:
        raise ValueError("reset_mask must be bool [B,T]")
    if reset_mask.device != valid_mask.device:
        raise ValueError("valid_mask and reset_mask must share one device")
    device = valid_mask.device
    batch, length = valid_mask.shape
    indices = valid_mask.reshape(-1).nonzero().flatten()
    count = indices.shape[0]
    if count == 0:
        empty = torch.empty(0, dtype=torch.long, device=device)
        zero = torch.zeros(1, dtype=torch.long)
        return PackedSegments(
            batch=batch, length=length, indices=indices, segment_ids=empty, segment_batch=empty,
            use_initial=torch.empty(0, dtype=torch.bool, device=device),
            segment_lengths=torch.empty(0, dtype=torch.int32, device=device),
            cu_seqlens=zero.to(device), cu_seqlens_cpu=zero,
            segment_batch_cpu=torch.empty(0, dtype=torch.long),
            use_initial_cpu=torch.empty(0, dtype=torch.bool),
            last_segment=torch.full((batch,), -1, dtype=torch.long, device=device),
            valid_mask=valid_mask, reset_mask=reset_mask)

    row = indices // length
    resets_here = reset_mask.reshape(-1)[indices]
    row_changes = torch.ones(count, dtype=torch.bool, device=device)
    row_changes[1:] = row[1:] != row[:-1]
    opens_segment = row_changes | resets_here
    segment_ids = torch.cumsum(opens_segment, dim=0) - 1
    first_token = opens_segment.nonzero().flatten()
    segment_batch = row[first_token]
    boundaries = torch.cat((first_token, first_token.new_tensor([count])))
    segment_lengths = (boundaries[1:] - boundaries[:-1]).to(torch.int32)
    # a segment inherits the caller's state only if it opens its batch row without a reset
    use_initial = row_changes[first_token] & ~resets_here[first_token]
    numbering = torch.arange(segment_batch.shape[0], dtype=torch.long, device=device)
    last_segment = torch.full((batch,), -1, dtype=torch.long, device=device).scatter_reduce(
        0, segment_batch, numbering, reduce="amax", include_self=True)

    host = torch.stack((segment_lengths.long(), segment_batch, use_initial.long()), dim=1).cpu()
    cu_cpu = torch.cat((torch.zeros(1, dtype=torch.long), host[:, 0].cumsum(0)))
    return PackedSegments(
        batch=batch, length=length, indices=indices, segment_ids=segment_ids,
        segment_batch=segment_batch, use_initial=use_initial, segment_lengths=segment_lengths,
        cu_seqlens=cu_cpu.to(device), cu_seqlens_cpu=cu_cpu, segment_batch_cpu=host[:, 1],
        use_initial_cpu=host[:, 2].bool(), last_segment=last_segment,
        valid_mask=valid_mask, reset_mask=reset_mask)


def pack_tokens(tensor: torch.Tensor, plan: PackedSegments) -> torch.Tensor:
    """[B,T,...] -> [1,N,...]: the valid tokens in plan order."""
    if tensor.shape[:2] != (plan.batch, plan.length):
        raise ValueError("packed tensor must share the plan's [B,T] prefix")
    flat = tensor.reshape(plan.batch * plan.length, *tensor.shape[2:])
    return flat.index_select(0, plan.indices).unsqueeze(0)


def unpack_tokens(tensor: torch.Tensor, plan: PackedSegments) -> torch.Tensor:
    """[1,N,...] -> [B,T,...] with zeros at the invalid tokens."""
    if tensor.ndim < 2 or tensor.shape[0] != 1:
        raise ValueError("packed tensor must have a singleton batch axis")
    body = tensor.squeeze(0)
    full = body.new_zeros(plan.batch * plan.length, *body.shape[1:])
    return full.index_copy(0, plan.indices, body).view(plan.batch, plan.length, *body.shape[1:])


__all__ = ["PackedSegments", "build_packed_segments", "pack_tokens", "unpack_tokens"]
