"""Host-side behaviour of the block glue entries (no GPU): what they refuse, and what they leave to the caller."""
import pytest
import torch

from solvedelta_b200 import fused_cross_entropy
from solvedelta_b200.mixer_ops import add_rmsnorm, add_rmsnorm_reverse_supported, pack_rows, small_linear, swiglu


def test_reverse_widths_of_add_rmsnorm():
    assert [w for w in (128, 256, 384, 512, 1024, 2048, 2304, 4096) if add_rmsnorm_reverse_supported(w)] == [
        256, 512, 1024, 2048]


def test_entries_refuse_cpu_tensors():
    x = torch.zeros(2, 256, dtype=torch.bfloat16)
    with pytest.raises(TypeError):
        add_rmsnorm(x, x, torch.ones(256), 1e-6)
    with pytest.raises(TypeError):
        swiglu(x)
    with pytest.raises(TypeError):
        fused_cross_entropy(x, torch.zeros(2, dtype=torch.long))


def test_layouts_left_to_the_caller():
    x = torch.zeros(1, 64, dtype=torch.bfloat16)
    w = torch.zeros(32, 64, dtype=torch.bfloat16)
    with torch.no_grad():
        assert small_linear(x, w) is None                      # not on a GPU
    assert small_linear(x.requires_grad_(), w) is None         # gradients recorded
    assert pack_rows([x], (64,), (1, 64), torch.device("cpu")) is None


def test_model_blocks_fall_back_off_the_gpu():
    """The fused paths are chosen by layout: a CPU model runs on the PyTorch norms and activation."""
    from solvedelta_b200 import SolveDeltaConfig
    from solvedelta_b200.modeling import SolveDeltaBlock, SolveDeltaMLP

    assert not SolveDeltaBlock.fuses(torch.zeros(1, 4, 256))
    assert not SolveDeltaBlock.fuses(torch.zeros(1, 4, 256, dtype=torch.bfloat16))
    mlp = SolveDeltaMLP(hidden_size=32, intermediate_size=64)
    y = mlp(torch.randn(2, 3, 32))
    gate, value = mlp.gate_up_proj(torch.zeros(2, 3, 32)).chunk(2, dim=-1)
    assert y.shape == (2, 3, 32) and gate.shape == value.shape
    assert SolveDeltaConfig().fuse_cross_entropy
