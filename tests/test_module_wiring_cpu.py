"""The kernel-backed modules on a machine without a GPU: they are drop-ins for the stock PyTorch modules (same
parameters, same state-dict keys, same CPU results), which is what makes checkpoints interchangeable
(role of ScaFFold/unet/group_norm.py:540-684, conv3d.py adapters and tests/test_groupnorm_wiring_edge.py)."""
import pytest
import torch
import torch.nn as nn
import torch.nn.functional as F

from scaffold_b200.ops.conv3d import Conv3d, ConvTranspose3d
from scaffold_b200.ops.group_norm import GroupNorm
from scaffold_b200.ops.pool import MaxPool3d


def test_groupnorm_is_a_stock_groupnorm_with_an_optional_fused_relu():
    torch.manual_seed(0)
    x = torch.randn(2, 16, 4, 5, 6)
    ours, stock = GroupNorm(4, 16, activation="relu"), nn.GroupNorm(4, 16)
    with torch.no_grad():
        ours.weight.copy_(torch.rand(16) + 0.5)
        ours.bias.copy_(torch.randn(16))
    stock.load_state_dict(ours.state_dict())                      # same keys, no buffers
    assert list(ours.state_dict()) == ["weight", "bias"]
    assert torch.allclose(ours(x), F.relu(stock(x)), atol=1e-6)
    plain = GroupNorm(4, 16)
    plain.load_state_dict(ours.state_dict())
    assert torch.allclose(plain(x), stock(x), atol=1e-6)          # no activation: identical to the stock module
    assert "activation=relu" in repr(ours)
    with pytest.raises(ValueError, match="activation must be None or 'relu'"):
        GroupNorm(4, 16, activation="gelu")
    assert ours.kernel_supported() and not GroupNorm(8, 24).kernel_supported()   # 3 channels per group: ATen formula
    assert not GroupNorm(4, 16, affine=False).kernel_supported()


def test_groupnorm_keeps_dtype_and_memory_format_on_the_fallback_path():
    x = torch.randn(1, 8, 4, 4, 4).to(memory_format=torch.channels_last_3d)
    y = GroupNorm(2, 8, activation="relu")(x)
    assert y.dtype == x.dtype and y.shape == x.shape and (y >= 0).all()
    yb = GroupNorm(2, 8)(x.to(torch.bfloat16))
    assert yb.dtype == torch.bfloat16


def test_convolutions_match_the_stock_modules_on_cpu():
    torch.manual_seed(1)
    x = torch.randn(1, 6, 5, 6, 7)
    ours, stock = Conv3d(6, 10, kernel_size=3, padding=1, bias=False), nn.Conv3d(6, 10, kernel_size=3, padding=1, bias=False)
    stock.load_state_dict(ours.state_dict())
    assert list(ours.state_dict()) == ["weight"] and torch.allclose(ours(x), stock(x), atol=1e-6)
    head, stock_head = Conv3d(6, 4, kernel_size=1), nn.Conv3d(6, 4, kernel_size=1)
    stock_head.load_state_dict(head.state_dict())
    assert torch.allclose(head(x), stock_head(x), atol=1e-6)
    up, stock_up = ConvTranspose3d(6, 3, kernel_size=2, stride=2), nn.ConvTranspose3d(6, 3, kernel_size=2, stride=2)
    stock_up.load_state_dict(up.state_dict())
    assert torch.allclose(up(x), stock_up(x), atol=1e-6) and up(x).shape == (1, 3, 10, 12, 14)
    # gradients flow through the fallback path
    xg = x.clone().requires_grad_(True)
    ours(xg).sum().backward()
    assert xg.grad is not None and ours.weight.grad is not None


def test_maxpool_matches_the_stock_module_on_cpu():
    x = torch.randn(1, 4, 6, 6, 7)
    assert torch.equal(MaxPool3d(2)(x), nn.MaxPool3d(2)(x))
