"""Two ranks on two GPUs (skipped on a single-GPU box): the distributed graphed training step
averages the gradients over NCCL and leaves both ranks with the same weights."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    device = torch.device("cuda", rank)
    torch.cuda.set_device(device)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=device)
    from solvedelta_b200 import (BF16ShadowWeights, SolveDeltaConfig, SolveDeltaForCausalLM,
                                 SolveDeltaGraphedTrainingStep)

    torch.manual_seed(11)   # same weights everywhere
    config = SolveDeltaConfig(hidden_size=256, num_heads=2, head_k_dim=64, head_v_dim=128, num_hidden_layers=2,
                              vocab_size=512, initializer_range=0.05)
    model = SolveDeltaForCausalLM(config).prepare(device).train()
    gen = torch.Generator().manual_seed(50 + rank)   # different data per rank
    ids = torch.randint(0, config.vocab_size, (2, 128), generator=gen).to(device)
    shadows = BF16ShadowWeights(model, lambda masters: torch.optim.SGD(masters, lr=0.05))
    step = SolveDeltaGraphedTrainingStep(model, ids, ids, distributed=True)
    params = list(model.parameters())
    with step.no_sync():
        step(ids, ids)
    local = [p.grad.float().clone() for p in params]
    for p in params:
        p.grad.zero_()
    step(ids, ids)
    averaged = [p.grad.float().clone() for p in params]
    worst = 0.0
    for g_local, g_avg in zip(local, averaged):
        both = [torch.zeros_like(g_local) for _ in range(world)]
        dist.all_gather(both, g_local)
        want = sum(both) / world
        scale = want.abs().max().clamp_min(1e-20)
        worst = max(worst, float(((g_avg - want).abs().max() / scale)))
    for _ in range(3):
        shadows.optimizer.step()
        step(ids, ids)
    probe = torch.stack([p.detach().float().sum() for p in params])
    probes = [torch.zeros_like(probe) for _ in range(world)]
    dist.all_gather(probes, probe)
    same = all(torch.equal(x, probes[0]) for x in probes)
    torch.save({"worst": worst, "same": same}, os.path.join(out_dir, f"rank{rank}.pt"))
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_distributed_graphed_step_averages_gradients(tmp_path):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    for rank in range(world):
        got = torch.load(os.path.join(tmp_path, f"rank{rank}.pt"))
        # the flat bucket sums BF16 gradients in BF16: one rounding of the sum
        assert got["worst"] < 1e-2, got
        assert got["same"], "ranks diverged"


def _bucketed_worker(rank, world, port, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    device = torch.device("cuda", rank)
    torch.cuda.set_device(device)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=device)
    from solvedelta_b200 import (BF16ShadowWeights, BucketedGradientAverager, SolveDeltaConfig,
                                 SolveDeltaForCausalLM, causal_lm_loss)

    torch.manual_seed(11)
    config = SolveDeltaConfig(hidden_size=256, num_heads=2, head_k_dim=64, head_v_dim=128, num_hidden_layers=2,
                              vocab_size=512, initializer_range=0.05)
    model = SolveDeltaForCausalLM(config).prepare(device).train()
    gen = torch.Generator().manual_seed(50 + rank)
    ids = torch.randint(0, config.vocab_size, (2, 128), generator=gen).to(device)
    shadows = BF16ShadowWeights(model, lambda masters: torch.optim.SGD(masters, lr=0.05))
    params = [p for p in model.parameters() if p.requires_grad]
    averager = BucketedGradientAverager(params, bucket_bytes=1 << 18)
    total = ids.shape[0] * (ids.shape[1] - 1)
    with averager.no_sync():
        causal_lm_loss(model, ids, ids, total=total).backward()
        averager.finish()
    local = [p.grad.float().clone() for p in params]
    averager.zero_grad()
    causal_lm_loss(model, ids, ids, total=total).backward()
    issued = averager.finish()
    averaged = [p.grad.float().clone() for p in params]
    worst = 0.0
    for g_local, g_avg in zip(local, averaged):
        both = [torch.zeros_like(g_local) for _ in range(world)]
        dist.all_gather(both, g_local)
        want = sum(both) / world
        scale = want.abs().max().clamp_min(1e-20)
        worst = max(worst, float(((g_avg - want).abs().max() / scale)))
    for _ in range(3):
        shadows.optimizer.step()
        causal_lm_loss(model, ids, ids, total=total).backward()
        averager.finish()
    probe = torch.stack([p.detach().float().sum() for p in params])
    probes = [torch.zeros_like(probe) for _ in range(world)]
    dist.all_gather(probes, probe)
    same = all(torch.equal(x, probes[0]) for x in probes)
    torch.save({"worst": worst, "same": same, "issued": issued, "buckets": len(averager.buckets)},
               os.path.join(out_dir, f"rank{rank}.pt"))
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_bucketed_averager_over_nccl(tmp_path):
    """Bucketed all-reduces launched from autograd hooks during an eager backward (NCCL, two GPUs)."""
    world = 2
    mp.spawn(_bucketed_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    for rank in range(world):
        got = torch.load(os.path.join(tmp_path, f"rank{rank}.pt"))
        assert got["issued"] == got["buckets"] and got["buckets"] > 2, got
        assert got["worst"] < 1e-2, got
        assert got["same"], "ranks diverged"
