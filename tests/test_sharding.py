"""N>1 path on CPU: two gloo ranks shard the streams, run their shards through
the CPU checker, and reassemble exactly the single-process result; the
benchmark's time reduction takes the slowest rank."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from solvedelta_b200.sharding import job_throughput, max_over_ranks, rank_seed, shard_streams, stream_shard
from tests.helpers import golden_inputs, golden_state, load_golden


def test_shards_are_disjoint_and_cover_every_stream():
    for batch, heads, world in ((8, 8, 1), (8, 8, 2), (8, 8, 8), (8, 8, 16), (8, 8, 64), (3, 4, 2), (2, 8, 8)):
        seen = np.zeros((batch, heads), dtype=int)
        for bs, hs in shard_streams(batch, heads, world):
            seen[bs, hs] += 1
        assert (seen == 1).all(), (batch, heads, world)
    with pytest.raises(ValueError):
        stream_shard(2, 2, 0, 8)
    assert rank_seed(5, 3) == 8 and job_throughput(100, 0.5, 4) == 800.0


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from oracle import solvedelta_oracle as orc

    orc.set_threads(1)
    g = load_golden("seed7_masks_resets_state")
    args = golden_inputs(g)
    B, T, H, r = args[0].shape
    bs, hs = stream_shard(B, H, rank, world)
    sub = [a[bs][:, :, hs] for a in args[:-1]] + [args[-1][hs]]
    C0, S0 = golden_state(g)
    y, st = orc.forward(*sub, initial_state=(C0[bs][:, hs], S0[bs][:, hs]),
                        valid_mask=g["valid"][bs], reset_mask=g["reset"][bs])
    np.savez(os.path.join(out_dir, f"rank{rank}.npz"), y=y, C=st.predictor, S=st.S)
    slowest = max_over_ranks(10.0 + rank)
    assert slowest == 10.0 + world - 1
    dist.barrier()
    dist.destroy_process_group()


def test_two_gloo_ranks_reassemble_the_full_result(tmp_path):
    world, port = 2, _free_port()
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    g = load_golden("seed7_masks_resets_state")
    y = np.zeros_like(g["out"])
    C, S = np.zeros_like(g["C_T"]), np.zeros_like(g["S_T"])
    B, H = g["out"].shape[0], g["out"].shape[2]
    for rank in range(world):
        bs, hs = stream_shard(B, H, rank, world)
        part = np.load(tmp_path / f"rank{rank}.npz")
        y[bs][:, :, hs] = part["y"]
        C[bs][:, hs] = part["C"]
        S[bs][:, hs] = part["S"]
    np.testing.assert_allclose(y, g["out"], rtol=2e-12, atol=2e-12)
    np.testing.assert_allclose(C, g["C_T"], rtol=2e-12, atol=2e-12)
    np.testing.assert_allclose(S, g["S_T"], rtol=2e-12, atol=2e-12)
