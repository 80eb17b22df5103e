"""Gradient reduction across ranks (data-parallel replicas AND spatial shards).

Every rank holds the full weights; after backward each rank has the gradient
of its own samples / its own sub-volume. The reducer sums the flat fp32
gradient buffer over all ranks; the optimizer then applies ``1 / ddp_ranks``
(sum over spatial shards, mean over replicas), the scaling DistConvDDP
produces in the reference (ScaFFold/worker.py:81-97, ScaFFold/unet/conv3d.py:66-71).

Backends: ``"fused"`` reduces through peer memory with the kernel of
``csrc/grad_allreduce.cu`` when it is available for the launch, ``"nccl"`` (and
every CPU/gloo run) calls ``torch.distributed.all_reduce`` on buckets of the
flat buffer.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist


class GradReducer:
    def __init__(self, layout, flat=None, params=None, backend: str = "nccl", bucket_mb: int = 256):
        self.layout = layout
        self.flat = flat
        self.params = list(params) if params is not None else None
        self.backend = backend
        self.bucket_elems = bucket_mb * (1 << 20) // 4
        self.world = layout.world_size if layout is not None else 1
        self._fused = None
        if backend == "fused" and self.world > 1 and flat is not None:
            try:
                from .fused_allreduce import FusedAllReduce
                self._fused = FusedAllReduce(flat.numel)
                flat.rehome_grad(self._fused.grad)  # gradients now accumulate straight into peer-visible memory
            except Exception as exc:  # documented degradation: the NCCL path is always correct
                import logging
                logging.getLogger("scaffold").warning("fused gradient all-reduce unavailable (%s); using NCCL", exc)
                self._fused = None

    @property
    def scale(self) -> float:
        return self.layout.grad_scale() if self.layout is not None else 1.0

    def reduce(self) -> None:
        """Sum gradients over all ranks (call after backward, before the optimizer step)."""
        if self.world == 1:
            return
        if self._fused is not None:
            self._fused.all_reduce_()
            return
        if self.flat is not None:
            g = self.flat.grad
            for o in range(0, g.numel(), self.bucket_elems):
                dist.all_reduce(g[o:o + self.bucket_elems])
            return
        for p in self.params:
            if p.grad is not None:
                dist.all_reduce(p.grad)
