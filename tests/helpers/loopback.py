"""Two spatial 'ranks' on ONE GPU: channel objects wired to each other's buffers inside one process.

The fused multi-GPU kernels address their peers through plain device pointers, so on a single device
rank A's push can land in rank B's arena and vice versa. The producers (push / share kernels, which
never wait) are launched first for both ranks and complete in stream order; only then run the
consumers, whose flag waits are therefore already satisfied. No two launches ever wait on each other.
"""
from __future__ import annotations

import torch

from scaffold_b200.parallel.halo import SLOTS, HaloChannel, StatsChannel
from scaffold_b200.parallel.peer import PeerBuffer


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
