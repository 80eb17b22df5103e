"""Fused halo exchange over peer memory for a volume split along one axis (the kernels' depth axis;
a volume split along H or W reaches this module with that axis already exchanged with depth, see
``SpatialContext.lead_swap``).

``HaloChannel`` owns, per rank, a landing arena and a block of flag words that
the spatial neighbours can address (:class:`PeerBuffer`). A halo exchange is one
small kernel per rank (``csrc/halo.cu``): it stores this rank's boundary planes
straight into the neighbours' arenas over NVLink and then publishes an epoch in
their flag words. The consumer is the convolution itself: its plane producer
waits (bounded) on the flag only when it reaches plane -1 or plane D and then
reads the landed slab with an ordinary TMA load from local memory; interior
planes never wait, and the activation is never copied into a padded tensor.

Slots: both neighbours execute the same layer sequence and each needs the
other's slab to finish a layer, so they are never more than one exchange apart;
four rotating slots keep a slab alive until its reader is done.
"""
from __future__ import annotations

import ctypes as C
from typing import List, Optional, Sequence

import torch
import torch.distributed as dist

from ..ops import _lib
from .peer import PeerBuffer

_P = C.c_void_p
_lib.register("sb_halo_push", [C.POINTER(C.c_longlong), C.c_int, C.c_int, C.c_uint, _P, _P])
_lib.register("sb_halo_accum", [_P, _P, C.c_longlong, C.c_longlong, C.c_longlong, C.c_int, C.c_int, C.c_int, C.c_int,
                                _P, C.c_uint, C.c_double, _P, _P])

SLOTS = 4


class Landing:
    """One exchange: where the neighbours' planes land on this rank and which flags guard them."""

    def __init__(self, chan: "HaloChannel", slot: int, epoch: int, views, wait_seconds: float):
        self.chan, self.slot, self.epoch, self.views, self.wait_seconds = chan, slot, epoch, views, wait_seconds

    def land_ptr(self, source: int, face: int):
        v = self.views[source][face] if source < len(self.views) else None
        return v.data_ptr() if v is not None else None

    def flag_ptr(self, face: int):
        return self.chan.flag_addr(self.chan.rank, self.slot, face) if self.chan.neigh[face] is not None else None

    def clone(self):
        """Private copies of the landed slabs (for the backward pass); None at the volume boundary."""
        return [[v.clone() if v is not None else None for v in pair] for pair in self.views]


class HaloChannel:
    def __init__(self, layout, group, arena_mb: int = 256, wait_seconds: float = 2.0):
        if not self.eligible(layout):
            raise ValueError("the fused halo channel handles a volume split along exactly one axis")
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        self.neigh = [self.rank - 1 if self.rank > 0 else None, self.rank + 1 if self.rank + 1 < self.world else None]
        self.face_bytes = (arena_mb << 20) // (SLOTS * 2) // 256 * 256
        self.arena = PeerBuffer(self.face_bytes * SLOTS * 2, group)
        self.flags = PeerBuffer(4096, group)
        self.arena_t = self.arena.tensor(torch.uint8)
        self.counter = torch.zeros(1, dtype=torch.int32, device="cuda")
        self.seq = 0
        self.wait_seconds = wait_seconds

    @staticmethod
    def eligible(layout) -> bool:
        """Exactly one split axis: the ranks of the spatial group are then the line of neighbours along it."""
        return sum(1 for n in layout.num_shards if n > 1) == 1

    def flag_addr(self, rank: int, slot: int, face: int) -> int:
        return self.flags.ptrs[rank] + 4 * (slot * 2 + face)

    def _region(self, rank: int, slot: int, face: int) -> int:
        return self.arena.ptrs[rank] + (slot * 2 + face) * self.face_bytes

    def exchange(self, lo_planes: Sequence[torch.Tensor], hi_planes: Sequence[torch.Tensor]) -> Landing:
        """Push ``lo_planes[s]`` / ``hi_planes[s]`` (views ``[N, H, W, C_s]`` of the first / last local plane
        of every source) to the low / high neighbour; returns where their planes land here."""
        slot, epoch = self.seq % SLOTS, self.seq + 1
        self.seq += 1
        n = lo_planes[0].shape[0]
        copies: List[int] = []
        views = []
        off = 0
        for s, (lo, hi) in enumerate(zip(lo_planes, hi_planes)):
            plane_bytes = lo.shape[1] * lo.shape[2] * lo.shape[3] * lo.element_size()
            if off + n * plane_bytes > self.face_bytes:
                raise RuntimeError(f"halo slab of {off + n * plane_bytes} bytes exceeds the landing arena "
                                   f"({self.face_bytes} bytes per face); raise halo_arena_mb")
            for face, plane in ((0, lo), (1, hi)):
                nb = self.neigh[face]
                if nb is None:
                    continue
                if plane.stride(3) != 1 or plane.stride(2) != plane.shape[3] or plane.stride(1) != plane.shape[2] * plane.shape[3]:
                    raise ValueError("boundary planes must be dense [N, H, W, C] views of a voxel-major tensor")
                # my low plane becomes the low neighbour's HIGH halo (and vice versa)
                dst = self._region(nb, slot, 1 - face) + off
                copies += [plane.data_ptr(), dst, plane.stride(0) * plane.element_size(), plane_bytes, plane_bytes,
                           self.flag_addr(nb, slot, 1 - face)]
            pair = []
            for face in (0, 1):
                if self.neigh[face] is None:
                    pair.append(None)
                    continue
                base = (slot * 2 + face) * self.face_bytes + off
                v = self.arena_t[base: base + n * plane_bytes].view(lo.dtype).view(n, 1, *lo.shape[1:])
                pair.append(v)
            views.append(pair)
            off += (n * plane_bytes + 255) // 256 * 256
        if copies:
            arr = (C.c_longlong * len(copies))(*copies)
            _lib.check(_lib.lib().sb_halo_push(arr, len(copies) // 6, n, epoch, self.counter.data_ptr(),
                                               _lib.stream_ptr()), "sb_halo_push")
        return Landing(self, slot, epoch, views, self.wait_seconds)

    def accumulate(self, grads: Sequence[torch.Tensor], landing: Landing, slab_ld: int) -> None:
        """Add the landed gradient slabs into the boundary planes of ``grads`` ([N, D, H, W, C_i] each)."""
        c_off = 0
        slab_view = landing.views[0]
        for g in grads:
            n, d, h, w, c = g.shape
            for face, plane_index in ((0, 0), (1, d - 1)):
                if self.neigh[face] is None:
                    continue
                dst = g[:, plane_index]
                slab = slab_view[face]
                _lib.check(_lib.lib().sb_halo_accum(dst.data_ptr(), slab.data_ptr(), g.stride(0), slab.stride(0),
                                                    h * w, c, slab_ld, c_off, n,
                                                    self.flag_addr(self.rank, landing.slot, face), landing.epoch,
                                                    float(self.wait_seconds),
                                                    _lib.status_tensor(g.device).data_ptr(), _lib.stream_ptr()),
                           "sb_halo_accum")
            c_off += c

    def close(self) -> None:
        self.flags.close()
        self.arena.close()


class StatsChannel:
    """Cross-shard GroupNorm statistics over peer memory.

    ``share(fin)`` launches one tiny kernel that stores this rank's finalised statistics into every
    rank's landing slot and raises their flags; it returns the LOCAL pointers of all ranks' slots (own
    first) and the flag block the merging kernel waits on. No collective library call is involved.
    """

    SLOT_FLOATS = 1 << 14  # 64 KiB per (slot, rank): N * C * 2 floats of the backward statistics fit

    def __init__(self, group):
        self.group = group
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self.data = PeerBuffer(SLOTS * self.world * self.SLOT_FLOATS * 4, group)
        self.flags = PeerBuffer(4096, group)
        self.seq = 0

    def _slot_ptr(self, on_rank: int, slot: int, from_rank: int) -> int:
        return self.data.ptrs[on_rank] + 4 * self.SLOT_FLOATS * (slot * self.world + from_rank)

    def _flag_ptr(self, on_rank: int, slot: int, position: int) -> int:
        return self.flags.ptrs[on_rank] + 4 * (slot * self.world + position)

    def _position(self, on_rank: int, from_rank: int) -> int:
        """Index of ``from_rank`` in ``on_rank``'s merge order: own first, the others in rank order."""
        if from_rank == on_rank:
            return 0
        return from_rank + 1 if from_rank < on_rank else from_rank

    def share(self, fin: torch.Tensor):
        if fin.numel() > self.SLOT_FLOATS:
            raise RuntimeError(f"statistics block of {fin.numel()} floats exceeds the slot ({self.SLOT_FLOATS})")
        slot, epoch = self.seq % SLOTS, self.seq + 1
        self.seq += 1
        dst = (_P * self.world)(*[self._slot_ptr(r, slot, self.rank) for r in range(self.world)])
        flg = (_P * self.world)(*[self._flag_ptr(r, slot, self._position(r, self.rank)) for r in range(self.world)])
        _lib.check(_lib.lib().sb_gn_share(fin.data_ptr(), fin.numel(), dst, flg, self.world, epoch,
                                          _lib.stream_ptr()), "sb_gn_share")
        order = [self.rank] + [r for r in range(self.world) if r != self.rank]
        parts = [self._slot_ptr(self.rank, slot, r) for r in order]
        return parts, (self._flag_ptr(self.rank, slot, 0), epoch)

    def close(self) -> None:
        self.flags.close()
        self.data.close()
