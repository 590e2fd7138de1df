"""Host-side logic of the training helpers: the fixed-denominator chunked linear + cross entropy,
the FP32 master weights, and gradient averaging over a two-rank gloo group (CPU)."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp
import torch.nn.functional as F
from torch import nn

from solvedelta_b200.training import BF16ShadowWeights, allreduce_gradients, fixed_dense_linear_cross_entropy


@pytest.mark.parametrize("chunks,with_bias", [(1, False), (3, True), (8, False), (50, True)])
def test_fixed_denominator_loss_equals_cross_entropy(chunks, with_bias):
    gen = torch.Generator().manual_seed(chunks)
    x = torch.randn(3, 7, 10, dtype=torch.float64, generator=gen, requires_grad=True)
    w = torch.randn(13, 10, dtype=torch.float64, generator=gen, requires_grad=True)
    b = torch.randn(13, dtype=torch.float64, generator=gen, requires_grad=True) if with_bias else None
    target = torch.randint(0, 13, (3, 7), generator=gen)
    target[0, 2] = -100
    target[2, 6] = -100
    total = 19   # a constant of the batch shape, here the true count
    cot = torch.tensor(0.7, dtype=torch.float64)
    loss = fixed_dense_linear_cross_entropy(x, target, w, b, total=total, num_chunks=chunks)
    grads = torch.autograd.grad(loss, [t for t in (x, w, b) if t is not None], cot.float())
    ref = F.cross_entropy(F.linear(x, w, b).reshape(-1, 13), target.reshape(-1), ignore_index=-100, reduction="sum") / total
    ref_grads = torch.autograd.grad(ref, [t for t in (x, w, b) if t is not None], cot)
    assert abs(loss.item() - ref.item()) < 1e-6
    for got, want in zip(grads, ref_grads):
        assert got.shape == want.shape and got.dtype == want.dtype
        # the weight and bias gradients pass through an FP32 accumulator
        assert (got - want).abs().max().item() < 1e-6 * max(1.0, want.abs().max().item())


def test_a_device_side_count_gives_the_mean_of_cross_entropy():
    """``total`` as a 0-dim tensor (the count of valid labels) reproduces ``F.cross_entropy``'s mean, and the
    configuration refuses both fused losses at once (causallsso/config.py:133-136)."""
    from solvedelta_b200 import SolveDeltaConfig

    gen = torch.Generator().manual_seed(5)
    x = torch.randn(2, 9, 6, dtype=torch.float64, generator=gen, requires_grad=True)
    w = torch.randn(11, 6, dtype=torch.float64, generator=gen, requires_grad=True)
    target = torch.randint(0, 11, (2, 9), generator=gen)
    target[1, 3:] = -100
    count = (target != -100).sum()
    loss = fixed_dense_linear_cross_entropy(x, target, w, None, total=count, num_chunks=4)
    ref = F.cross_entropy(F.linear(x, w).reshape(-1, 11), target.reshape(-1), ignore_index=-100)
    assert abs(loss.item() - ref.item()) < 1e-6
    gx, = torch.autograd.grad(loss, [x])
    rx, = torch.autograd.grad(ref, [x])
    assert (gx - rx).abs().max().item() < 1e-6
    with pytest.raises(ValueError):
        fixed_dense_linear_cross_entropy(x, target, w, None, total=torch.ones(2))
    assert SolveDeltaConfig(fuse_cross_entropy=False, fuse_linear_cross_entropy=True).fuse_linear_cross_entropy
    with pytest.raises(ValueError):
        SolveDeltaConfig(fuse_cross_entropy=True, fuse_linear_cross_entropy=True)


def test_fixed_denominator_loss_checks_its_arguments():
    x, w = torch.randn(2, 3, 4), torch.randn(5, 4)
    t = torch.zeros(2, 3, dtype=torch.long)
    with pytest.raises(ValueError):
        fixed_dense_linear_cross_entropy(x, t, w, total=0)
    with pytest.raises(ValueError):
        fixed_dense_linear_cross_entropy(x, t[:, :2], w, total=6)
    with pytest.raises(ValueError):
        fixed_dense_linear_cross_entropy(x, t, torch.randn(5, 3), total=6)
    # no gradient requested: nothing but the loss is formed
    assert fixed_dense_linear_cross_entropy(x, t, w, total=6).requires_grad is False


def test_master_weights_own_the_update():
    torch.manual_seed(0)
    model = nn.Sequential(nn.Linear(8, 8), nn.Linear(8, 4)).to(torch.bfloat16)
    shadows = BF16ShadowWeights(model, lambda masters: torch.optim.SGD(masters, lr=0.5))
    assert all(m.dtype == torch.float32 for m in shadows.masters)
    assert shadows.nbytes == sum(p.numel() for p in model.parameters()) * 4
    before = [m.detach().clone() for m in shadows.masters]
    x = torch.randn(5, 8).to(torch.bfloat16)
    for _ in range(2):   # two accumulated micro-batches
        model(x).float().pow(2).sum().backward()
    grads = [p.grad.float().clone() for p in model.parameters()]
    shadows.optimizer.step()
    shadows.assert_current()
    for m, m0, g, p in zip(shadows.masters, before, grads, model.parameters()):
        assert torch.allclose(m, m0 - 0.5 * g)                       # the FP32 master took the full-precision step
        assert torch.equal(p.detach(), m.detach().to(torch.bfloat16))  # the model holds its BF16 rounding
        assert p.grad is not None and not p.grad.any()               # cleared in place (storage kept)
    # a change made to the masters by hand reaches the model through refresh()
    with torch.no_grad():
        shadows.masters[0].add_(1.0)
    shadows.refresh()
    assert torch.equal(model[0].weight.detach(), shadows.masters[0].detach().to(torch.bfloat16))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _allreduce_worker(rank, world, port, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    params = [nn.Parameter(torch.zeros(3, 2)), nn.Parameter(torch.zeros(5)), nn.Parameter(torch.zeros(4)),
              nn.Parameter(torch.zeros(2, dtype=torch.float64))]
    params[0].grad = torch.full((3, 2), float(rank + 1))
    params[1].grad = torch.arange(5, dtype=torch.float32) * (rank + 1)
    # params[2] has no gradient on any rank
    params[3].grad = torch.tensor([1.0, -2.0], dtype=torch.float64) * (rank + 1)
    issued = allreduce_gradients(params)
    torch.save({"issued": issued, "grads": [None if p.grad is None else p.grad for p in params]},
               os.path.join(out_dir, f"rank{rank}.pt"))
    dist.destroy_process_group()


def test_gradients_are_averaged_over_two_ranks(tmp_path):
    world = 2
    mp.spawn(_allreduce_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    for rank in range(world):
        got = torch.load(os.path.join(tmp_path, f"rank{rank}.pt"))
        assert got["issued"] == 2   # one flat bucket per gradient dtype
        g0, g1, g2, g3 = got["grads"]
        assert torch.equal(g0, torch.full((3, 2), 1.5))
        assert torch.equal(g1, torch.arange(5, dtype=torch.float32) * 1.5)
        assert g2 is None
        assert torch.equal(g3, torch.tensor([1.5, -3.0], dtype=torch.float64))


def _bucketed_worker(rank, world, port, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from solvedelta_b200 import BucketedGradientAverager

    torch.manual_seed(0)   # the same weights on every rank
    model = nn.Sequential(nn.Linear(6, 16), nn.Tanh(), nn.Linear(16, 16), nn.Tanh(), nn.Linear(16, 3))
    model[2].weight.data = model[2].weight.data.double()   # a second gradient dtype -> its own buckets
    model[2].bias.data = model[2].bias.data.double()
    averager = BucketedGradientAverager(model.parameters(), bucket_bytes=256)   # several buckets
    gen = torch.Generator().manual_seed(10 + rank)
    x = torch.randn(4, 6, generator=gen)

    def loss_of(inp):
        h = torch.tanh(model[0](inp)).double()
        h = torch.tanh(model[2](h)).float()
        return model[4](h).pow(2).sum()

    loss_of(x).backward()
    issued = averager.finish()
    first = [p.grad.clone() for p in model.parameters()]
    views = all(p.grad.data_ptr() >= b["flat"].data_ptr() for b in averager.buckets for p in b["params"])
    # accumulation: one local micro-batch without a collective, then a synchronised one
    averager.zero_grad()
    with averager.no_sync():
        loss_of(x).backward()
        assert averager.finish() == 0
    loss_of(2 * x).backward()
    averager.finish()
    second = [p.grad.clone() for p in model.parameters()]
    torch.save({"issued": issued, "buckets": len(averager.buckets), "views": views, "first": first, "second": second,
                "x": x}, os.path.join(out_dir, f"rank{rank}.pt"))
    dist.destroy_process_group()


def test_bucketed_averager_overlaps_nothing_it_should_not(tmp_path):
    """Two gloo ranks: gradients that live in the buckets equal the plain average of the per-rank
    gradients, for one step and for an accumulated pair of micro-batches."""
    world = 2
    mp.spawn(_bucketed_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    got = [torch.load(os.path.join(tmp_path, f"rank{r}.pt")) for r in range(world)]
    torch.manual_seed(0)
    model = nn.Sequential(nn.Linear(6, 16), nn.Tanh(), nn.Linear(16, 16), nn.Tanh(), nn.Linear(16, 3))
    model[2].weight.data = model[2].weight.data.double()
    model[2].bias.data = model[2].bias.data.double()

    def grads_of(inputs):
        for p in model.parameters():
            p.grad = None
        for inp in inputs:
            h = torch.tanh(model[0](inp)).double()
            h = torch.tanh(model[2](h)).float()
            model[4](h).pow(2).sum().backward()
        return [p.grad.clone() for p in model.parameters()]

    per_rank_first = [grads_of([g["x"]]) for g in got]
    # second step: every rank accumulated its local x micro-batch, then the all-reduce summed (local x + 2x) over ranks
    per_rank_second = [grads_of([g["x"], 2 * g["x"]]) for g in got]
    for g in got:
        assert g["issued"] == g["buckets"] and g["buckets"] >= 3 and g["views"]
        for i, (a, b) in enumerate(zip(per_rank_first[0], per_rank_first[1])):
            assert torch.allclose(g["first"][i], (a + b) / 2, rtol=1e-5, atol=1e-6)
        for i, (a, b) in enumerate(zip(per_rank_second[0], per_rank_second[1])):
            assert torch.allclose(g["second"][i], (a + b) / 2, rtol=1e-5, atol=1e-6)


def test_allreduce_is_a_no_op_without_a_group():
    p = nn.Parameter(torch.zeros(2))
    p.grad = torch.ones(2)
    assert allreduce_gradients([p]) == 0 and torch.equal(p.grad, torch.ones(2))
