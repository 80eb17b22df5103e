"""Fused gradient all-reduce over peer memory (``csrc/peer.cu``).

The flat fp32 gradient buffer of every rank lives in a :class:`PeerBuffer`; one
kernel per rank sums it across ranks with P2P loads, applies the replica scale
and pushes the result back with P2P stores, synchronising through flag words in
peer memory (bounded waits). No NCCL call is involved in the reduction itself.
"""
from __future__ import annotations

import ctypes as C

import torch
import torch.distributed as dist

from ..ops import _lib
from .peer import PeerBuffer

_P = C.c_void_p
_lib.register("sb_grad_allreduce", [C.POINTER(_P), C.POINTER(_P), C.c_int, C.c_int, C.c_longlong, C.c_longlong,
                                    C.c_uint, C.c_float, C.c_int, C.c_double, _P, _P])


class FusedAllReduce:
    MAX_RANKS = 8

    def __init__(self, numel: int, group=None, ctas: int = 0, wait_seconds: float = 2.0):
        world = dist.get_world_size(group)
        if world > self.MAX_RANKS:
            raise RuntimeError(f"fused all-reduce supports up to {self.MAX_RANKS} ranks on one NVLink domain")
        self.group = group
        self.world, self.rank = world, dist.get_rank(group)
        self.numel = int(numel)
        self.data = PeerBuffer(self.numel * 4, group)
        self.flags = PeerBuffer(4096, group)
        self.grad = self.data.tensor(torch.float32)[: self.numel]
        self.epoch = 0
        self.ctas, self.wait_seconds = ctas, wait_seconds
        self._bufs, self._flags = self.data.ptr_array(), self.flags.ptr_array()

    def all_reduce_(self, offset: int = 0, count: int = None, scale: float = 1.0, ctas: int = None) -> None:
        """Sum elements ``[offset, offset+count)`` of every rank's buffer in place (result x ``scale``).
        ``ctas`` overrides the grid size of this call (0 / None: the full-width default)."""
        count = self.numel - offset if count is None else count
        self.epoch += 1
        status = _lib.status_tensor(self.grad.device)
        _lib.check(_lib.lib().sb_grad_allreduce(self._bufs, self._flags, self.rank, self.world, offset, count,
                                                self.epoch, float(scale), int(ctas if ctas else self.ctas),
                                                float(self.wait_seconds),
                                                status.data_ptr(), _lib.stream_ptr()), "sb_grad_allreduce")

    def close(self) -> None:
        self.flags.close()
        self.data.close()
