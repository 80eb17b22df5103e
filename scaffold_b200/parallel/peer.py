"""Peer-visible device buffers: one allocation per rank, mapped into every rank of a group through CUDA IPC.

``PeerBuffer(nbytes, group)`` allocates ``nbytes`` on this GPU (outside the
caching allocator, so the allocation can be exported), exchanges IPC handles
over the process group and opens every peer's allocation. ``ptrs[r]`` is a
device pointer, valid on THIS GPU, to rank ``r``'s buffer (own entry = the local
allocation); the fused kernels read and write peers through these with plain
loads and stores over NVLink. ``tensor(dtype)`` views the local allocation as a
torch tensor without copying.
"""
from __future__ import annotations

import ctypes as C
from typing import List, Optional

import torch
import torch.distributed as dist

from ..ops import _lib

_P = C.c_void_p
_lib.register("sb_peer_alloc", [C.POINTER(_P), C.c_longlong])
_lib.register("sb_peer_free", [_P])
_lib.register("sb_peer_handle_bytes", [], C.c_int)
_lib.register("sb_peer_get_handle", [_P, _P])
_lib.register("sb_peer_open_handle", [_P, C.POINTER(_P)])
_lib.register("sb_peer_close_handle", [_P])


class _RawCudaArray:
    def __init__(self, ptr: int, nbytes: int, owner):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3}
        self._owner = owner


class PeerBuffer:
    def __init__(self, nbytes: int, group=None, device: Optional[torch.device] = None):
        self.nbytes = int((nbytes + 255) // 256 * 256)
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        L = _lib.lib()
        local = _P()
        _lib.check(L.sb_peer_alloc(C.byref(local), self.nbytes), "sb_peer_alloc")
        self.local = local.value
        self._opened: List[int] = []
        self.ptrs: List[int] = [self.local]
        if self.world > 1:
            hb = L.sb_peer_handle_bytes()
            buf = C.create_string_buffer(hb)
            _lib.check(L.sb_peer_get_handle(self.local, buf), "sb_peer_get_handle")
            handles = [None] * self.world
            dist.all_gather_object(handles, bytes(buf.raw), group=group)
            self.ptrs = []
            for r, h in enumerate(handles):
                if r == self.rank:
                    self.ptrs.append(self.local)
                    continue
                out = _P()
                hbuf = C.create_string_buffer(h, hb)
                _lib.check(L.sb_peer_open_handle(hbuf, C.byref(out)), f"sb_peer_open_handle(rank {r})")
                self._opened.append(out.value)
                self.ptrs.append(out.value)
            dist.barrier(group=group)

    def tensor(self, dtype=torch.float32) -> torch.Tensor:
        raw = torch.as_tensor(_RawCudaArray(self.local, self.nbytes, self), device="cuda")
        return raw.view(dtype)

    def ptr_array(self):
        return (_P * len(self.ptrs))(*self.ptrs)

    def close(self) -> None:
        L = _lib.lib()
        for p in self._opened:
            L.sb_peer_close_handle(p)
        self._opened = []
        if self.local:
            L.sb_peer_free(self.local)
            self.local = 0
