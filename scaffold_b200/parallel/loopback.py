"""Single-GPU bring-up of the multi-rank protocols: several spatial 'ranks' on ONE GPU, their channel objects
wired to each other's buffers inside one process (used by the loopback tests and the smoke run).

The fused multi-GPU kernels address their peers through plain device pointers, so on a single device
rank A's push can land in rank B's arena and vice versa. The producers (push / share kernels, which
never wait) are launched first for both ranks and complete in stream order; only then run the
consumers, whose flag waits are therefore already satisfied. No two launches ever wait on each other.
"""
from __future__ import annotations

import torch

from .halo import SLOTS, HaloChannel, StatsChannel
from .peer import PeerBuffer


def _buffers(nbytes: int, world: int):
    bufs = [PeerBuffer(nbytes) for _ in range(world)]  # no process group: each is a plain local allocation
    ptrs = [b.local for b in bufs]
    for b in bufs:
        b.ptrs = list(ptrs)
    return bufs


def halo_pair(world: int = 2, arena_mb: int = 16, wait_seconds: float = 0.5):
    """``world`` HaloChannel objects acting as consecutive depth shards of one volume, all on this device."""
    face_bytes = (arena_mb << 20) // (SLOTS * 2) // 256 * 256
    arenas = _buffers(face_bytes * SLOTS * 2, world)
    flags = _buffers(4096, world)
    chans = []
    for r in range(world):
        c = object.__new__(HaloChannel)
        c.group, c.rank, c.world = None, r, world
        c.neigh = [r - 1 if r > 0 else None, r + 1 if r + 1 < world else None]
        c.face_bytes = face_bytes
        c.arena, c.flags = arenas[r], flags[r]
        c.arena_t = c.arena.tensor(torch.uint8)
        c.counter = torch.zeros(1, dtype=torch.int32, device="cuda")
        c.seq = 0
        c.wait_seconds = wait_seconds
        chans.append(c)
    return chans


def stats_pair(world: int = 2):
    data = _buffers(SLOTS * world * StatsChannel.SLOT_FLOATS * 4, world)
    flags = _buffers(4096, world)
    chans = []
    for r in range(world):
        c = object.__new__(StatsChannel)
        c.group, c.rank, c.world = None, r, world
        c.data, c.flags = data[r], flags[r]
        c.seq = 0
        chans.append(c)
    return chans


def allreduce(tensors, scale: float = 1.0, ctas: int = 8, wait_seconds: float = 0.5) -> None:
    """Sum ``tensors`` (equal-length fp32 views of PeerBuffer allocations, one per emulated rank) in place with the
    gradient all-reduce protocol, all ranks in ONE cooperative launch (``sb_grad_allreduce_loopback``)."""
    import ctypes as C

    from ..ops import _lib
    world = len(tensors)
    flags = _buffers(4096, world)
    _P = C.c_void_p
    fn = _lib.lib().sb_grad_allreduce_loopback
    fn.argtypes = [C.POINTER(_P), C.POINTER(_P), C.c_int, C.c_longlong, C.c_longlong, C.c_uint, C.c_float, C.c_int,
                   C.c_double, _P, _P]
    fn.restype = C.c_int
    barr = (_P * world)(*[t.data_ptr() for t in tensors])
    farr = (_P * world)(*[f.local for f in flags])
    _lib.check(fn(barr, farr, world, 0, tensors[0].numel(), 1, float(scale), ctas, wait_seconds,
                  _lib.status_tensor(tensors[0].device).data_ptr(), torch.cuda.current_stream().cuda_stream),
               "sb_grad_allreduce_loopback")
    torch.cuda.current_stream().synchronize()
    for f in flags:
        f.close()
