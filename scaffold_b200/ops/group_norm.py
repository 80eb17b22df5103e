"""GroupNorm with a fused ReLU; drop-in for ``nn.GroupNorm`` (same parameters, no buffers).

On CUDA/bf16 the forward and backward run the channels-last kernels of
``csrc/group_norm.cu`` (two streaming passes each). When the module is given a
spatial process group (``set_spatial``), the statistics span all shards of the
volume, so a sharded run normalises exactly like an unsharded one; the
reference keeps them per shard (ScaFFold/unet/group_norm.py:610-613), which
``stats="per_shard"`` reproduces. The output keeps the input's dtype and memory
format, and the ReLU is applied on every path (ScaFFold/unet/group_norm.py:662-684).
"""
from __future__ import annotations

import logging
from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import gn_kernels as gk
from .layout import from_vm, to_vm, use_cuda_kernels


class _GnFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, groups, eps, relu, spatial, partials):
        w32, b32 = weight.detach().float().contiguous(), bias.detach().float().contiguous()
        fin = None
        if partials is not None:
            # the producing convolution left (count, mean, M2) partials of this very tensor: no statistics pass
            part, splits, pg = partials
            if pg == groups and part.numel() == x.shape[0] * splits * groups * 3:
                fin = gk.gn_finalize(part, x.shape[0], groups, splits)
        if spatial is None:
            y, mean, rstd = gk.gn_forward(x, w32, b32, groups, eps, relu, fin=fin)
        else:
            y, mean, rstd = spatial.gn_forward(x, w32, b32, groups, eps, relu, fin=fin)
        ctx.save_for_backward(x, w32, b32, mean, rstd)
        ctx.cfg = (groups, eps, relu, spatial)
        return y

    @staticmethod
    def backward(ctx, gy):
        x, w32, b32, mean, rstd = ctx.saved_tensors
        groups, eps, relu, spatial = ctx.cfg
        gy = gy.contiguous()
        if spatial is None:
            dx, dw, db = gk.gn_backward(gy, x, w32, b32, mean, rstd, groups, eps, relu)
        else:
            dx, dw, db = spatial.gn_backward(gy, x, w32, b32, mean, rstd, groups, eps, relu)
        return dx, dw, db, None, None, None, None, None


class GroupNorm(nn.GroupNorm):
    """``nn.GroupNorm`` + optional fused ``activation="relu"``."""

    def __init__(self, num_groups: int, num_channels: int, eps: float = 1e-5, affine: bool = True,
                 activation: Optional[str] = None, device=None, dtype=None):
        super().__init__(num_groups, num_channels, eps=eps, affine=affine, device=device, dtype=dtype)
        if activation not in (None, "relu"):
            raise ValueError(f"activation must be None or 'relu'; got {activation!r}")
        self.activation = activation
        self._spatial = None  # parallel.spatial.SpatialContext, set by the model wrapper
        self._warned = False

    def set_spatial(self, ctx) -> None:
        self._spatial = ctx

    def extra_repr(self) -> str:
        return super().extra_repr() + f", activation={self.activation}"

    def kernel_supported(self) -> bool:
        """True when ``csrc/group_norm.cu`` covers this (channels, groups) pair: C a multiple of 8 up to 2048 and a
        group that is a whole number of channel octets (or 2 / 4 channels). Other pairs run the ATen formula."""
        return self.affine and gk.supported(self.num_channels, self.num_groups)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        relu = self.activation == "relu"
        if use_cuda_kernels(x) and x.dim() == 5 and self.kernel_supported():
            partials = getattr(x, "_sb_gn_partials", None)  # left by the convolution that produced x, if it could
            y = _GnFn.apply(to_vm(x), self.weight, self.bias, self.num_groups, self.eps, relu, self._spatial, partials)
            return from_vm(y)
        if x.is_cuda and use_cuda_kernels(x) and not self._warned:
            self._warned = True
            logging.getLogger("scaffold").warning(
                "GroupNorm(%d groups, %d channels) is outside the sm_100a kernels' range; this layer runs ATen",
                self.num_groups, self.num_channels)
        if self._spatial is not None and self._spatial.size > 1 and self._spatial.gn_global:
            y = self._spatial.group_norm_reference(x, self.num_groups, self.weight, self.bias, self.eps)
        else:
            y = F.group_norm(x.float() if x.dtype == torch.bfloat16 and not x.is_cuda else x, self.num_groups,
                             self.weight, self.bias, self.eps).to(x.dtype)
        return F.relu(y) if relu else y
