"""Gradient reduction across ranks (data-parallel replicas AND spatial shards).

Every rank holds the full weights; after backward each rank has the gradient
of its own samples / its own sub-volume. The reducer sums the flat fp32
gradient buffer over all ranks; the optimizer then applies ``1 / ddp_ranks``
(sum over spatial shards, mean over replicas), the scaling DistConvDDP
produces in the reference (ScaFFold/worker.py:81-97, ScaFFold/unet/conv3d.py:66-71).

Backends: ``"fused"`` reduces through peer memory with the kernel of
``csrc/peer.cu``; ``"nccl"`` (and every CPU/gloo run) calls
``torch.distributed.all_reduce`` on buckets of the flat buffer. A ``"fused"``
request that cannot be served (peer mapping refused, more than 8 ranks) is an
error unless ``allow_fallback`` is set, in which case the reducer logs the reason
and uses NCCL; ``effective_backend`` says which of the two runs.

Overlap: on CUDA the flat buffer is cut into buckets in the order backward
fills it (last layer first). A bucket is counted down by autograd's
post-accumulate hook or, for the convolutions that add their weight gradient
straight into the flat buffer, by ``notify_grad_written``; when its last
gradient has been enqueued the bucket's reduction is launched on a side stream
behind an event, so it runs under the rest of backward. ``reduce()`` launches
whatever is left and joins the side stream. Measured on 2 B200s (scale 7, 361 MB
of gradients, 6 buckets of 32 MB): the time left in ``reduce()`` after backward
falls from 0.89 ms to 0.12 ms, but the kernels it runs beside slow down by most
of that, so the step gains 0.2 ms (29.25 -> 29.04 ms) with the full-width grid
and nothing or less with small grids (16 CTAs: slower than no overlap, because
the last bucket finishes late; 48: +-0; 148: -0.1 ms). Hence ``overlap_ctas = 0``
(the full-width default of the kernel): get in, finish, get out.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist


class GradReducer:
    def __init__(self, layout, flat=None, params=None, backend: str = "nccl", bucket_mb: int = 256,
                 overlap: bool = False, overlap_bucket_mb: int = 32, allow_fallback: bool = False,
                 overlap_ctas: int = 0):
        self.layout = layout
        self.flat = flat
        self.params = list(params) if params is not None else None
        self.backend = backend
        self.bucket_elems = bucket_mb * (1 << 20) // 4
        self.world = layout.world_size if layout is not None else 1
        self.overlap_ctas = int(overlap_ctas)
        self._fused = None
        if backend == "fused" and self.world > 1 and flat is not None and flat.grad.is_cuda:
            try:
                from .fused_allreduce import FusedAllReduce
                self._fused = FusedAllReduce(flat.numel)
                flat.rehome_grad(self._fused.grad)  # gradients now accumulate straight into peer-visible memory
            except Exception as exc:
                if not allow_fallback:
                    raise RuntimeError(
                        f"grad_allreduce='fused' was requested but the peer-memory reducer could not be set up "
                        f"({type(exc).__name__}: {exc}); choose grad_allreduce='nccl' or set allow_fallback") from exc
                import logging
                logging.getLogger("scaffold").warning("fused gradient all-reduce unavailable (%s); using NCCL", exc)
                self._fused = None
        self._buckets = None
        self._comm = None
        if overlap and self.world > 1 and flat is not None and flat.grad.is_cuda:
            self._setup_overlap(overlap_bucket_mb * (1 << 20) // 4)

    # -- bucketed overlap with backward ---------------------------------------
    def _setup_overlap(self, bucket_elems: int) -> None:
        flat = self.flat
        ends = list(flat.offsets[1:]) + [flat.numel]
        self._buckets, self._bucket_of = [], {}
        hi = flat.numel
        members = []
        # walk the parameters from the last one (whose gradient arrives first) to the first
        for i in range(len(flat.params) - 1, -1, -1):
            members.append(i)
            lo = flat.offsets[i]
            if hi - lo >= bucket_elems or i == 0:
                b = {"lo": lo, "hi": hi, "n": len(members), "pending": len(members), "launched": False,
                     "seen": set()}
                for m in members:
                    self._bucket_of[id(flat.params[m])] = b
                self._buckets.append(b)
                hi, members = lo, []
        self._comm = torch.cuda.Stream(device=flat.grad.device)
        self._handles = []
        for p in flat.params:
            p.register_post_accumulate_grad_hook(self._on_grad)
        from ..ops.layout import add_grad_written_listener
        add_grad_written_listener(self._on_grad)  # gradients the kernels wrote into the flat buffer themselves

    def _on_grad(self, p) -> None:
        """One gradient of this step is in the flat buffer (its kernels are enqueued on the current stream).
        A parameter is counted once per step: autograd may also run its accumulate hook for a weight whose
        gradient the convolution wrote directly (``notify_grad_written`` came first, when the data was there)."""
        b = self._bucket_of.get(id(p))
        if b is None or b["launched"] or id(p) in b["seen"]:
            return
        b["seen"].add(id(p))
        b["pending"] -= 1
        if b["pending"] == 0:
            self._launch(b)

    def _launch(self, b) -> None:
        b["launched"] = True
        ev = torch.cuda.Event()
        ev.record()
        with torch.cuda.stream(self._comm):
            self._comm.wait_event(ev)
            if self._fused is not None:
                self._fused.all_reduce_(b["lo"], b["hi"] - b["lo"], ctas=self.overlap_ctas)
            else:
                self._handles.append(dist.all_reduce(self.flat.grad[b["lo"]:b["hi"]], async_op=True))

    def _finish_overlap(self) -> None:
        for b in self._buckets:
            if not b["launched"]:  # parameters that received no gradient this step
                self._launch(b)
        for h in self._handles:
            h.wait()
        self._handles = []
        torch.cuda.current_stream().wait_stream(self._comm)
        for b in self._buckets:
            b["pending"], b["launched"] = b["n"], False
            b["seen"].clear()

    @property
    def effective_backend(self) -> str:
        """'none' (one rank), 'fused' (peer-memory kernel) or 'nccl' / 'gloo' (library all-reduce)."""
        if self.world == 1:
            return "none"
        if self._fused is not None:
            return "fused"
        return dist.get_backend() if dist.is_initialized() else "nccl"

    @property
    def scale(self) -> float:
        return self.layout.grad_scale() if self.layout is not None else 1.0

    def reduce(self) -> None:
        """Sum gradients over all ranks (call after backward, before the optimizer step)."""
        if self.world == 1:
            return
        if self._buckets is not None:
            self._finish_overlap()
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
