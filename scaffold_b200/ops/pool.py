"""2x2x2 max-pool module (``nn.MaxPool3d(2)`` drop-in) with a channels-last sm_100a kernel."""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from .layout import from_vm, to_vm, use_cuda_kernels


class MaxPool3d(nn.MaxPool3d):
    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if use_cuda_kernels(x) and self.kernel_size in (2, (2, 2, 2)):
            from . import pool_kernels as pk
            return from_vm(pk.MaxPool2Fn.apply(to_vm(x)))  # a missing native library raises; no silent ATen path
        return F.max_pool3d(x, self.kernel_size, self.stride, self.padding, self.dilation, self.ceil_mode)
