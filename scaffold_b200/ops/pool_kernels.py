"""Launchers of the channels-last 2x2x2 max-pool kernels (``csrc/pool.cu``)."""
from __future__ import annotations

import ctypes as C

import torch

from . import _lib

_P = C.c_void_p
_lib.register("sb_maxpool2_fwd", [_P, _P, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, _P], C.c_int)
_lib.register("sb_maxpool2_bwd", [_P, _P, _P, _P, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, _P], C.c_int)


def available() -> bool:
    return hasattr(_lib.lib(), "sb_maxpool2_fwd")


def maxpool2_fwd(x: torch.Tensor) -> torch.Tensor:
    n, d, h, w, c = x.shape
    y = torch.empty((n, d // 2, h // 2, w // 2, c), dtype=x.dtype, device=x.device)
    _lib.check(_lib.lib().sb_maxpool2_fwd(x.data_ptr(), y.data_ptr(), n, d, h, w, c, _lib.stream_ptr()),
               "sb_maxpool2_fwd")
    return y


def maxpool2_bwd(gy: torch.Tensor, x: torch.Tensor, y: torch.Tensor) -> torch.Tensor:
    n, d, h, w, c = x.shape
    gx = torch.empty_like(x)
    _lib.check(_lib.lib().sb_maxpool2_bwd(gy.data_ptr(), x.data_ptr(), y.data_ptr(), gx.data_ptr(), n, d, h, w, c,
                                          _lib.stream_ptr()), "sb_maxpool2_bwd")
    return gx


class MaxPool2Fn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        y = maxpool2_fwd(x)
        ctx.save_for_backward(x, y)
        return y

    @staticmethod
    def backward(ctx, gy):
        x, y = ctx.saved_tensors
        return maxpool2_bwd(gy.contiguous(), x, y)
