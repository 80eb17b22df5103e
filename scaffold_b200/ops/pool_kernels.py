"""Launchers of the channels-last 2x2x2 max-pool kernels (``csrc/pool.cu``)."""
from __future__ import annotations

import ctypes as C
import os

import torch

from . import _lib

_P = C.c_void_p
_lib.register("sb_maxpool2_fwd", [_P, _P, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, _P], C.c_int)
_lib.register("sb_maxpool2_bwd", [_P, _P, _P, _P, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, _P], C.c_int)
_lib.register("sb_maxpool2_fwd_idx", [_P, _P, _P, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, _P], C.c_int)
_lib.register("sb_maxpool2_bwd_idx", [_P, _P, _P, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, _P], C.c_int)


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


def maxpool2_fwd_idx(x: torch.Tensor):
    """Forward that also returns the index words (one byte per output element: which of the eight inputs won)."""
    n, d, h, w, c = x.shape
    y = torch.empty((n, d // 2, h // 2, w // 2, c), dtype=x.dtype, device=x.device)
    idx = torch.empty((n, d // 2, h // 2, w // 2, c // 8), dtype=torch.int64, device=x.device)
    _lib.check(_lib.lib().sb_maxpool2_fwd_idx(x.data_ptr(), y.data_ptr(), idx.data_ptr(), n, d, h, w, c,
                                              _lib.stream_ptr()), "sb_maxpool2_fwd_idx")
    return y, idx


def maxpool2_bwd_idx(gy: torch.Tensor, idx: torch.Tensor, in_shape) -> torch.Tensor:
    """Backward from the index words: reads ``gy`` and ``idx`` (3/16 of a volume), writes the input gradient."""
    n, d, h, w, c = in_shape
    gx = torch.empty(tuple(in_shape), dtype=gy.dtype, device=gy.device)
    _lib.check(_lib.lib().sb_maxpool2_bwd_idx(gy.data_ptr(), idx.data_ptr(), gx.data_ptr(), n, d, h, w, c,
                                              _lib.stream_ptr()), "sb_maxpool2_bwd_idx")
    return gx


# SCAFFOLD_POOL_INDEX=0: backward recomputes the winners from x and y instead of reading index words (A/B switch)
_USE_INDEX = os.environ.get("SCAFFOLD_POOL_INDEX", "1") != "0"


class MaxPool2Fn(torch.autograd.Function):
    """Keeps the index words for backward, not the input and output tensors."""

    @staticmethod
    def forward(ctx, x):
        ctx.in_shape = tuple(x.shape)
        if _USE_INDEX:
            y, idx = maxpool2_fwd_idx(x)
            ctx.save_for_backward(idx)
        else:
            y = maxpool2_fwd(x)
            ctx.save_for_backward(x, y)
        return y

    @staticmethod
    def backward(ctx, gy):
        saved = ctx.saved_tensors  # read once: activation checkpointing unpacks on access
        if len(saved) == 1:
            return maxpool2_bwd_idx(gy.contiguous(), saved[0], ctx.in_shape)
        x, y = saved
        return maxpool2_bwd(gy.contiguous(), x, y)
