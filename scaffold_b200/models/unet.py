"""3-D U-Net for volumetric segmentation.

Topology and state-dict keys match the reference model
(ScaFFold/unet/unet_model.py:27-162, ScaFFold/unet/unet_parts.py:32-240):
``down_list[0]`` is a ``DoubleConv`` stem, ``down_list[i>0]`` are
``MaxPool3d(2) -> DoubleConv``, ``up_list[:-1]`` are ``ConvTranspose3d(k2,s2) ->
concat(skip, up) -> DoubleConv`` and ``up_list[-1]`` is the 1x1x1 head. The
``DoubleConv`` keeps ``nn.Sequential`` slots 0,1,3,4 (2 and 5 are ``Identity``
place-holders of the ReLUs now fused into the GroupNorm), so checkpoints of
either implementation load into the other.

Differences that do not change the function: the base width is a parameter
(reference: fixed 64), and on the CUDA path the skip concat is read by the
first convolution of the decoder block as two channel segments instead of
being written out.
"""
from __future__ import annotations

from typing import List

import torch
import torch.nn as nn
import torch.nn.functional as F
import torch.utils.checkpoint

from ..ops.conv3d import Conv3d, ConvTranspose3d
from ..ops.group_norm import GroupNorm
from ..ops.layout import use_cuda_kernels
from ..ops.pool import MaxPool3d
from ..utils.perf import annotate


class _FirstConvSequential(nn.Sequential):
    """``nn.Sequential`` whose first module may take a list of tensors (fused concat)."""

    def forward(self, x):
        for m in self:
            x = m(x)
        return x


class DoubleConv(nn.Module):
    """(conv3 -> GroupNorm+ReLU) x 2"""

    def __init__(self, in_channels: int, out_channels: int, group_norm_groups: int, mid_channels: int = None):
        super().__init__()
        mid = mid_channels or out_channels
        self.double_conv = _FirstConvSequential(
            Conv3d(in_channels, mid, kernel_size=3, padding=1, bias=False),
            GroupNorm(group_norm_groups, mid, activation="relu"),
            nn.Identity(),
            Conv3d(mid, out_channels, kernel_size=3, padding=1, bias=False),
            GroupNorm(group_norm_groups, out_channels, activation="relu"),
            nn.Identity(),
        )

        # each convolution feeds a GroupNorm: its kernel can hand the statistics over and save that pass
        self.double_conv[0].gn_groups_hint = group_norm_groups
        self.double_conv[3].gn_groups_hint = group_norm_groups

    @annotate("DoubleConv.forward")
    def forward(self, x):
        return self.double_conv(x)


class Down(nn.Module):
    def __init__(self, in_channels: int, out_channels: int, group_norm_groups: int):
        super().__init__()
        self.maxpool_conv = nn.Sequential(MaxPool3d(2), DoubleConv(in_channels, out_channels, group_norm_groups))

    @annotate("Down.forward")
    def forward(self, x):
        return self.maxpool_conv(x)


class Up(nn.Module):
    def __init__(self, in_channels: int, out_channels: int, group_norm_groups: int, trilinear: bool = False):
        super().__init__()
        if trilinear:
            self.up = nn.Upsample(scale_factor=2, mode="trilinear", align_corners=True)
            self.conv = DoubleConv(in_channels, out_channels, group_norm_groups, in_channels // 2)
        else:
            self.up = ConvTranspose3d(in_channels, in_channels // 2, kernel_size=2, stride=2)
            self.conv = DoubleConv(in_channels, out_channels, group_norm_groups)

    @annotate("Up.forward")
    def forward(self, x1, x2):
        x1 = self.up(x1)
        dz, dy, dx = (x2.size(i) - x1.size(i) for i in (2, 3, 4))
        if dx or dy or dz:
            x1 = F.pad(x1, [dx // 2, dx - dx // 2, dy // 2, dy - dy // 2, dz // 2, dz - dz // 2])
        if use_cuda_kernels(x2):
            return self.conv([x2, x1])  # read as two channel segments, never concatenated
        dev = x2.device.type
        dtype = torch.get_autocast_dtype(dev) if dev in ("cpu", "cuda") and torch.is_autocast_enabled(dev) else x2.dtype
        return self.conv(torch.cat([x2.to(dtype), x1.to(dtype)], dim=1))


class OutConv(nn.Module):
    def __init__(self, in_channels: int, out_channels: int):
        super().__init__()
        self.conv = Conv3d(in_channels, out_channels, kernel_size=1)

    @annotate("OutConv.forward")
    def forward(self, x):
        return self.conv(x)


class UNet(nn.Module):
    """``UNet(n_channels, n_classes, trilinear=False, layers=4, group_norm_groups=8, base_width=64)``"""

    def __init__(self, n_channels: int, n_classes: int, trilinear: bool = False, layers: int = 4,
                 group_norm_groups: int = 8, base_width: int = 64):
        super().__init__()
        if layers < 1:
            raise ValueError(
                f"UNet requires layers >= 1, got layers={layers}. layers is derived as problem_scale - "
                "unet_bottleneck_dim, so problem_scale must be strictly greater than unet_bottleneck_dim.")
        self.n_channels, self.n_classes = n_channels, n_classes
        self.trilinear, self.layers = trilinear, layers
        self.group_norm_groups = group_norm_groups
        self.base_width = base_width
        self.checkpointing = False
        self._spatial = None  # parallel.spatial.SpatialContext of a sharded run (see set_spatial)
        factor = 2 if trilinear else 1
        g = group_norm_groups

        c = base_width
        downs: List[nn.Module] = [DoubleConv(n_channels, c, g)]
        for _ in range(layers - 1):
            downs.append(Down(c, 2 * c, g))
            c *= 2
        downs.append(Down(c, (2 * c) // factor, g))
        c *= 2
        self.down_list = nn.ModuleList(downs)

        ups: List[nn.Module] = []
        for _ in range(layers - 1):
            ups.append(Up(c, (c // 2) // factor, g, trilinear))
            c //= 2
        ups.append(Up(c, c // 2, g, trilinear))
        c //= 2
        ups.append(OutConv(c, n_classes))
        self.up_list = nn.ModuleList(ups)

    def _run(self, block, *inputs):
        if self.checkpointing and torch.is_grad_enabled():
            return torch.utils.checkpoint.checkpoint(block, *inputs, use_reentrant=False)
        return block(*inputs)

    def set_spatial(self, ctx) -> None:
        """A volume split along H or W is processed with that axis exchanged with depth ('kernel space'):
        the input is transposed on the way in and the logits on the way out (views, no copies)."""
        self._spatial = ctx

    def _swap(self, t: torch.Tensor) -> torch.Tensor:
        sp = self._spatial
        return t if sp is None or sp.lead_swap is None else sp.to_kernel_space(t)

    def features(self, x: torch.Tensor) -> torch.Tensor:
        """Everything up to (not including) the 1x1x1 head (in kernel space on a sharded run)."""
        x = self._swap(x)
        if x.is_cuda and not x.is_contiguous():
            x = x.contiguous()  # the input staging kernel reads a dense NCDHW tensor
        skips = [self._run(self.down_list[0], x)]
        for i in range(1, self.layers + 1):
            skips.append(self._run(self.down_list[i], skips[-1]))
        skips.reverse()
        out = skips[0]
        for i in range(len(self.up_list) - 1):
            out = self._run(self.up_list[i], out, skips[i + 1])
        return out

    @annotate("UNet.forward")
    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self._swap(self._run(self.up_list[-1], self.features(x)))

    def forward_padded_logits(self, x: torch.Tensor) -> torch.Tensor:
        """CUDA path: voxel-major bf16 logits ``[N, D, H, W, pad16(n_classes)]`` for the fused loss, in kernel
        space (the caller exchanges the labels' axes the same way, ``SpatialContext.to_kernel_space``)."""
        return self.up_list[-1].conv.forward_padded(self.features(x))

    def use_checkpointing(self) -> None:
        self.checkpointing = True
