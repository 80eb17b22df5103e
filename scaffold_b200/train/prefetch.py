"""Host-to-device prefetch of training batches.

``DevicePrefetcher`` wraps any iterable of batches (dicts, tuples or lists of tensors, as the data loader
yields them from pinned memory) and hands out batches that already live on the GPU: while step *i* runs,
the copy of batch *i+1* is in flight on a side stream, so the PCIe transfer (about 1 ms for a 2 x 128^3
batch) leaves the step's critical path. Every batch is still copied exactly once, from the host memory
the loader produced. The reference moves each batch synchronously at the top of the step
(ScaFFold/utils/trainer.py:575-583).
"""
from __future__ import annotations

import time
from typing import Any, Iterable, Iterator, List

import torch


def _flatten(obj: Any, out: List[torch.Tensor]) -> Any:
    """Replace every tensor by its index in ``out`` (structure is kept for ``_rebuild``)."""
    if torch.is_tensor(obj):
        out.append(obj)
        return ("__tensor__", len(out) - 1)
    if isinstance(obj, dict):
        return {k: _flatten(v, out) for k, v in obj.items()}
    if isinstance(obj, (list, tuple)):
        return type(obj)(_flatten(v, out) for v in obj)
    return obj


def _rebuild(spec: Any, tensors: List[torch.Tensor]) -> Any:
    if isinstance(spec, tuple) and len(spec) == 2 and spec[0] == "__tensor__":
        return tensors[spec[1]]
    if isinstance(spec, dict):
        return {k: _rebuild(v, tensors) for k, v in spec.items()}
    if isinstance(spec, (list, tuple)):
        return type(spec)(_rebuild(v, tensors) for v in spec)
    return spec


class DevicePrefetcher:
    """Two persistent sets of device buffers: batch i+1 is copied into the idle set while step i reads the other.
    (Fresh allocations per batch on a side stream made the caching allocator fall back to device mallocs.)
    A yielded batch is valid until the iteration after the next one begins: consume it, do not keep it."""

    def __init__(self, batches: Iterable, device):
        self.batches = batches
        self.device = torch.device(device)
        self.wait_s = 0.0  # host time spent waiting for the wrapped loader to hand over a batch

    def __len__(self):
        return len(self.batches)

    def __iter__(self) -> Iterator:
        if self.device.type != "cuda":
            it = iter(self.batches)
            while True:
                t0 = time.perf_counter()
                try:
                    batch = next(it)
                except StopIteration:
                    return
                finally:
                    self.wait_s += time.perf_counter() - t0
                yield batch
        copy_stream = torch.cuda.Stream(device=self.device)
        it = iter(self.batches)
        slots: List[List[torch.Tensor]] = [[], []]
        free_ev = [None, None]  # recorded on the compute stream when the consumer came back for the next batch

        def load(k: int):
            t0 = time.perf_counter()
            try:
                host = next(it)
            except StopIteration:
                return None
            finally:
                self.wait_s += time.perf_counter() - t0
            src: List[torch.Tensor] = []
            spec = _flatten(host, src)
            bufs = slots[k]
            if len(bufs) != len(src) or any(b.shape != t.shape or b.dtype != t.dtype for b, t in zip(bufs, src)):
                bufs = slots[k] = [torch.empty(t.shape, dtype=t.dtype, device=self.device) for t in src]
                free_ev[k] = None
            with torch.cuda.stream(copy_stream):
                if free_ev[k] is not None:
                    copy_stream.wait_event(free_ev[k])  # the step that read this set has been passed
                for b, t in zip(bufs, src):
                    b.copy_(t, non_blocking=True)
            return _rebuild(spec, bufs)

        k = 0
        nxt = load(k)
        while nxt is not None:
            cur, cur_k = nxt, k
            main = torch.cuda.current_stream(self.device)
            main.wait_stream(copy_stream)   # batch i is complete before the step reads it
            k ^= 1
            nxt = load(k)                   # batch i+1 starts copying under step i
            yield cur
            ev = torch.cuda.Event()
            ev.record(torch.cuda.current_stream(self.device))
            free_ev[cur_k] = ev
