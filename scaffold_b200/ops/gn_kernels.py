"""Launchers of the channels-last GroupNorm(+ReLU) kernels (``csrc/group_norm.cu``).

Tensors are voxel-major ``[N, D, H, W, C]`` bf16; affine parameters and
statistics are fp32. ``peer_parts`` lets a spatially sharded run merge the
neighbours' partial statistics (device pointers into their memory) so the
result equals the unsharded normalisation.
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Optional, Sequence

import torch

from . import _lib

_lib.register("sb_gn_nsplit", [C.c_int, C.c_longlong, C.c_int], C.c_int)
_lib.register("sb_gn_supported", [C.c_int, C.c_int], C.c_int)


def supported(channels: int, groups: int) -> bool:
    """Host-side statement of what the kernels cover (same rule as ``gn_channels_ok`` in ``csrc/group_norm.cu``)."""
    if channels < 8 or channels % 8 or channels > 2048 or groups < 1 or groups > 256 or channels % groups:
        return False
    cg = channels // groups
    if (8 % cg) if cg < 8 else (cg % 8):
        return False
    return not (cg < 8 and 8 // cg > 4)


class SbGnArgs(C.Structure):
    _fields_ = [
        ("x", C.c_void_p), ("dy", C.c_void_p), ("y", C.c_void_p),
        ("w", C.c_void_p), ("b", C.c_void_p),
        ("mean", C.c_void_p), ("rstd", C.c_void_p),
        ("part", C.c_void_p),
        ("parts", C.c_void_p * 8),
        ("n_parts", C.c_int),
        ("dw", C.c_void_p), ("db", C.c_void_p),
        ("N", C.c_int), ("C", C.c_int), ("G", C.c_int),
        ("S", C.c_longlong), ("S_total", C.c_longlong),
        ("nsplit", C.c_int),
        ("eps", C.c_float),
        ("relu", C.c_int),
        ("wait_flags", C.c_void_p),
        ("wait_epoch", C.c_uint),
        ("wait_s", C.c_double),
        ("status", C.c_void_p),
        ("fin", C.c_void_p),
    ]


for _n in ("sb_gn_stats", "sb_gn_apply", "sb_gn_bwd_partial", "sb_gn_bwd_dx"):
    _lib.register(_n, [C.POINTER(SbGnArgs), C.c_void_p], C.c_int)
_lib.register("sb_gn_stats_finalize", [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p], C.c_int)
_lib.register("sb_gn_bwd_finalize", [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p], C.c_int)
_lib.register("sb_gn_share", [C.c_void_p, C.c_longlong, C.POINTER(C.c_void_p), C.POINTER(C.c_void_p), C.c_int,
                              C.c_uint, C.c_void_p], C.c_int)


# SCAFFOLD_GN_FUSED_FINALIZE=0 collapses the partial statistics in a launch of its own (the A/B switch of the
# last-block hand-over inside the statistics kernels)
_FUSED_FINALIZE = os.environ.get("SCAFFOLD_GN_FUSED_FINALIZE", "1") != "0"


def _base(x: torch.Tensor, w, b, groups: int, eps: float, relu: bool, shards: int, nsplit: int = 0) -> SbGnArgs:
    n, d, h, wd, c = x.shape
    a = SbGnArgs()
    a.x = x.data_ptr()
    a.w, a.b = w.data_ptr(), b.data_ptr()
    a.N, a.C, a.G = n, c, groups
    a.S = d * h * wd
    a.S_total = a.S * shards
    a.nsplit = nsplit or _lib.lib().sb_gn_nsplit(n, a.S, c)
    a.eps = eps
    a.relu = 1 if relu else 0
    return a


def partial_numel_fwd(x: torch.Tensor, groups: int) -> int:
    n, d, h, w, c = x.shape
    return n * _lib.lib().sb_gn_nsplit(n, d * h * w, c) * groups * 3


def partial_numel_bwd(x: torch.Tensor) -> int:
    n, d, h, w, c = x.shape
    return n * _lib.lib().sb_gn_nsplit(n, d * h * w, c) * c * 2


def gn_stats(x, w, b, groups, eps, relu, part: Optional[torch.Tensor] = None,
             fin: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Pass 1: this rank's (count, mean, M2) per (n, group), shape ``[N*G*3]`` (what peers exchange)."""
    a = _base(x, w, b, groups, eps, relu, 1)
    if part is None:
        part = torch.empty(partial_numel_fwd(x, groups), dtype=torch.float32, device=x.device)
    a.part = part.data_ptr()
    a.n_parts = 1
    a.parts[0] = part.data_ptr()
    if fin is None:
        fin = torch.empty(x.shape[0] * groups * 3, dtype=torch.float32, device=x.device)
    fused = _FUSED_FINALIZE and x.shape[0] * groups <= 32
    if fused:
        a.fin = fin.data_ptr()  # the last block of the launch collapses the partials: no separate finalize launch
    _lib.check(_lib.lib().sb_gn_stats(C.byref(a), _lib.stream_ptr()), "sb_gn_stats")
    if not fused:
        _lib.check(_lib.lib().sb_gn_stats_finalize(part.data_ptr(), fin.data_ptr(), x.shape[0], groups, a.nsplit,
                                                   _lib.stream_ptr()), "sb_gn_stats_finalize")
    return fin


def gn_finalize(part: torch.Tensor, n: int, groups: int, nsplit: int) -> torch.Tensor:
    """Collapse ``[N, nsplit, G, 3]`` partial statistics (from ``sb_gn_stats`` or from a convolution's epilogue)
    into the ``[N*G*3]`` block that ``gn_apply`` merges."""
    fin = torch.empty(n * groups * 3, dtype=torch.float32, device=part.device)
    _lib.check(_lib.lib().sb_gn_stats_finalize(part.data_ptr(), fin.data_ptr(), n, groups, nsplit, _lib.stream_ptr()),
               "sb_gn_stats_finalize")
    return fin


def _set_wait(a: SbGnArgs, wait, device) -> None:
    if wait is not None:
        a.wait_flags, a.wait_epoch = wait[0], wait[1]
        a.wait_s = float(wait[2]) if len(wait) > 2 else 2.0  # optional third entry: limit in seconds
        a.status = _lib.status_tensor(device).data_ptr()


def gn_apply(x, w, b, groups, eps, relu, parts: Sequence[int], shards: int = 1, wait=None):
    """Pass 2: merge ``parts`` (device pointers, own first) and normalise.

    ``wait`` = (pointer to ``len(parts)`` flag words, epoch): the kernel first waits until every
    flag reached the epoch (peers push their statistics and then raise the flag)."""
    a = _base(x, w, b, groups, eps, relu, shards, nsplit=1)
    _set_wait(a, wait, x.device)
    n = x.shape[0]
    y = torch.empty_like(x)
    mean = torch.empty((n, groups), dtype=torch.float32, device=x.device)
    rstd = torch.empty((n, groups), dtype=torch.float32, device=x.device)
    a.y, a.mean, a.rstd = y.data_ptr(), mean.data_ptr(), rstd.data_ptr()
    a.n_parts = len(parts)
    for i, p in enumerate(parts):
        a.parts[i] = p
    _lib.check(_lib.lib().sb_gn_apply(C.byref(a), _lib.stream_ptr()), "sb_gn_apply")
    return y, mean, rstd


def gn_forward(x, w, b, groups: int, eps: float = 1e-5, relu: bool = True, fin: Optional[torch.Tensor] = None):
    """``fin``: this tensor's finalised statistics when its producer already computed them (pass 1 is skipped)."""
    part = fin if fin is not None else gn_stats(x, w, b, groups, eps, relu)
    return gn_apply(x, w, b, groups, eps, relu, [part.data_ptr()])


def gn_bwd_partial(dy, x, w, b, mean, rstd, groups, eps, relu, part: Optional[torch.Tensor] = None,
                   fin: Optional[torch.Tensor] = None):
    """Backward pass 1: this rank's per-(n, channel) sums ``[N*C*2]`` (what peers exchange)."""
    a = _base(x, w, b, groups, eps, relu, 1)
    a.dy = dy.data_ptr()
    a.mean, a.rstd = mean.data_ptr(), rstd.data_ptr()
    if part is None:
        part = torch.empty(partial_numel_bwd(x), dtype=torch.float32, device=x.device)
    a.part = part.data_ptr()
    a.n_parts = 1
    a.parts[0] = part.data_ptr()
    if fin is None:
        fin = torch.empty(x.shape[0] * x.shape[4] * 2, dtype=torch.float32, device=x.device)
    # The hand-over to the last block pays only while that one block has a handful of outputs to collapse: N*C
    # per-channel sums would make it a serial tail (measured: +1.6 ms per step), so they keep their own launch.
    fused = _FUSED_FINALIZE and x.shape[0] * x.shape[4] <= 32
    if fused:
        a.fin = fin.data_ptr()
    _lib.check(_lib.lib().sb_gn_bwd_partial(C.byref(a), _lib.stream_ptr()), "sb_gn_bwd_partial")
    if not fused:
        _lib.check(_lib.lib().sb_gn_bwd_finalize(part.data_ptr(), fin.data_ptr(), x.shape[0], x.shape[4], a.nsplit,
                                                 _lib.stream_ptr()), "sb_gn_bwd_finalize")
    return fin


def gn_bwd_dx(dy, x, w, b, mean, rstd, groups, eps, relu, parts: Sequence[int], shards: int = 1, wait=None):
    a = _base(x, w, b, groups, eps, relu, shards, nsplit=1)
    _set_wait(a, wait, x.device)
    a.dy = dy.data_ptr()
    a.mean, a.rstd = mean.data_ptr(), rstd.data_ptr()
    dx = torch.empty_like(x)
    c = x.shape[4]
    dw = torch.empty(c, dtype=torch.float32, device=x.device)
    db = torch.empty(c, dtype=torch.float32, device=x.device)
    a.y, a.dw, a.db = dx.data_ptr(), dw.data_ptr(), db.data_ptr()
    a.n_parts = len(parts)
    for i, p in enumerate(parts):
        a.parts[i] = p
    _lib.check(_lib.lib().sb_gn_bwd_dx(C.byref(a), _lib.stream_ptr()), "sb_gn_bwd_dx")
    return dx, dw, db


def gn_backward(dy, x, w, b, mean, rstd, groups: int, eps: float = 1e-5, relu: bool = True):
    part = gn_bwd_partial(dy, x, w, b, mean, rstd, groups, eps, relu)
    return gn_bwd_dx(dy, x, w, b, mean, rstd, groups, eps, relu, [part.data_ptr()])
