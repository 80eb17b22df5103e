"""The U-Net's structure without memory (meta device): parameter counts of the benchmark scales, state-dict keys,
width parameter, CPU forward shape, and agreement with the symbolic shape calculator
(roles of ScaFFold/unet/unet_model.py and model-analysis/unet_shapes.py)."""
import pytest
import torch

from scaffold_b200.analysis import unet_shapes as U
from scaffold_b200.models.unet import UNet


def _count(model):
    return sum(p.numel() for p in model.parameters())


@pytest.mark.parametrize("layers,n_classes,expected", [(4, 6, 90_302_342), (4, 9, 90_302_537), (5, 6, 361_896_838)])
def test_parameter_counts_of_the_benchmark_scales(layers, n_classes, expected):
    with torch.device("meta"):
        model = UNet(3, n_classes, layers=layers, base_width=64)
    assert _count(model) == expected


def test_state_dict_layout_and_width_parameter():
    with torch.device("meta"):
        m64 = UNet(3, 6, layers=2, base_width=64)
        m16 = UNet(3, 6, layers=2, base_width=16)
    keys = list(m64.state_dict())
    assert keys[0] == "down_list.0.double_conv.0.weight" and keys[-1].startswith("up_list.") and len(keys) == 36
    assert [k for k in keys if k.endswith(".bias") and ".double_conv.0" in k] == []      # 3x3x3 convs carry no bias
    assert list(m16.state_dict()) == keys                                                 # width changes sizes only
    assert m64.state_dict()["down_list.0.double_conv.0.weight"].shape == (64, 3, 3, 3, 3)
    assert m16.state_dict()["down_list.0.double_conv.0.weight"].shape == (16, 3, 3, 3, 3)
    assert _count(m16) < _count(m64) / 10


def test_cpu_forward_shape_and_symbolic_trace_agree():
    torch.manual_seed(0)
    model = UNet(3, 5, layers=2, base_width=8)
    x = torch.rand(1, 3, 16, 16, 16)
    y = model(x)
    assert y.shape == (1, 5, 16, 16, 16) and torch.isfinite(y).all()
    tr = U.trace_unet(4, 2, 1, n_categories=4, base_width=8)            # scale 4 = 16^3, two levels below the stem
    convs = [o for o in tr.ops if o.kind in ("conv3", "conv1", "convT")]
    n_modules = sum(1 for m in model.modules() if isinstance(m, (torch.nn.Conv3d, torch.nn.ConvTranspose3d)))
    assert len(convs) == n_modules
