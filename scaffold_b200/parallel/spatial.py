"""Spatial (domain-decomposition) parallelism: halo exchange, cross-shard GroupNorm, spatial sums.

A ``SpatialContext`` binds a :class:`ParallelLayout` to the communication
primitives the sharded modules need. Semantics follow what the reference gets
from DistConv (ScaFFold/unet/conv3d.py:748-841, 53-71): a 3x3x3 convolution on
a sharded volume needs a one-voxel halo on both faces of every split dim
(neighbour data, zeros at the volume boundary); backward returns the halo
gradients to their owners, which ACCUMULATE them into their boundary planes;
the weight gradient is taken against the halo'd input; k2s2 transposed conv,
pooling, concat and the 1x1x1 head are shard-local.

Transport: ``torch.distributed`` point-to-point (gloo on CPU, NCCL on GPU) of
contiguous boundary slabs. On a single-node NVLink box the CUDA path can use
peer memory instead (``halo_backend="fused"``, :mod:`scaffold_b200.parallel.peer`).

Any single split axis runs the fused (in-kernel) halo: the kernels fold the halo of their depth
axis, so when the volume is split along H or W instead, the model works in *kernel space*, the
volume with that axis exchanged with depth (``lead_swap``). Convolution, pooling, normalisation
and the voxel-wise loss are symmetric under such an exchange once the weights' tap axes are
exchanged the same way, so the modules read their parameters through a transposed view and the
state dict keeps the ordinary layout. ``dims`` / ``neighbours`` below speak kernel space.

GroupNorm statistics are global over the volume by default (``gn_stats:
global``): per-(sample, group) count/sum/sumsq (CPU) or Welford partials (CUDA)
are combined over the spatial group, so a sharded run normalises exactly like
the unsharded one. ``gn_stats: per_shard`` reproduces the reference
(ScaFFold/unet/group_norm.py:610-613).
"""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch
import torch.distributed as dist
import torch.nn.functional as F


class SpatialContext:
    def __init__(self, layout, gn_stats: str = "global", halo_backend: str = "nccl"):
        self.layout = layout
        self.size = layout.spatial_size
        self.group = layout.spatial_group
        self.gn_global = gn_stats == "global"
        self.halo_backend = halo_backend
        split = layout.sharded_dims()  # tensor dims (NCDHW numbering) of the volume that are split
        self.halo_channel = None
        self.stats_channel = None
        # One split axis other than depth on the kernel path: exchange it with depth (see the module docstring).
        self.lead_swap: Optional[int] = None
        fused_ok = (halo_backend == "fused" and self.size > 1 and torch.cuda.is_available()
                    and dist.is_initialized() and dist.get_backend() == "nccl")
        if fused_ok and len(split) == 1 and split[0] != 2:
            self.lead_swap = split[0]
        self.dims: List[int] = [2] if self.lead_swap is not None else split  # kernel-space dims that are split
        if (halo_backend == "fused" and self.size > 1 and self.size <= 8 and self.gn_global
                and torch.cuda.is_available() and dist.get_backend() == "nccl"):
            from .halo import StatsChannel
            self.stats_channel = StatsChannel(self.group)  # collective
        if halo_backend == "fused" and self.size > 1 and torch.cuda.is_available() and dist.get_backend() == "nccl":
            from .halo import HaloChannel
            if HaloChannel.eligible(layout):
                self.halo_channel = HaloChannel(layout, self.group)  # collective: every rank of the group

    # -- small reductions -------------------------------------------------------
    def all_reduce_sum(self, t: torch.Tensor) -> torch.Tensor:
        if self.size > 1:
            dist.all_reduce(t, group=self.group)
        return t

    # -- halo exchange -------------------------------------------------------------
    def volume_dim(self, dim: int) -> int:
        """Axis of the stored volume behind kernel-space axis ``dim``."""
        k = self.lead_swap
        if k is None:
            return dim
        return k if dim == 2 else (2 if dim == k else dim)

    def to_kernel_space(self, t: torch.Tensor, first_spatial: int = 2) -> torch.Tensor:
        """Exchange the split axis with depth (a view); ``first_spatial`` is the position of D in ``t``."""
        if self.lead_swap is None:
            return t
        return t.transpose(first_spatial, first_spatial + self.lead_swap - 2)

    from_kernel_space = to_kernel_space  # the exchange is its own inverse

    def neighbours(self, dim: int) -> Tuple[Optional[int], Optional[int]]:
        d = self.volume_dim(dim)
        return self.layout.neighbour(d, -1), self.layout.neighbour(d, +1)

    def _exchange(self, send_lo: torch.Tensor, send_hi: torch.Tensor, dim: int):
        """Send my low/high boundary slabs to the -/+ neighbours; returns what they sent (zeros at the boundary)."""
        lo, hi = self.neighbours(dim)
        recv_lo = torch.zeros(send_lo.shape, dtype=send_lo.dtype, device=send_lo.device)
        recv_hi = torch.zeros(send_hi.shape, dtype=send_hi.dtype, device=send_hi.device)
        ops = []
        if lo is not None:
            ops += [dist.P2POp(dist.isend, send_lo.contiguous(), lo), dist.P2POp(dist.irecv, recv_lo, lo)]
        if hi is not None:
            ops += [dist.P2POp(dist.isend, send_hi.contiguous(), hi), dist.P2POp(dist.irecv, recv_hi, hi)]
        if ops:
            for w in dist.batch_isend_irecv(ops):
                w.wait()
        return recv_lo, recv_hi

    def halo_pad(self, x: torch.Tensor, halo: int = 1) -> torch.Tensor:
        """NCDHW tensor -> the same with ``halo`` planes added on both faces of every split dim (autograd-aware)."""
        if self.size == 1 or not self.dims or halo == 0:
            return x
        for d in self.dims:
            x = _HaloPad.apply(x, self, d, halo)
        return x

    def conv_padding(self, ksize: int) -> Tuple[int, int, int]:
        """Padding of a 'same' conv whose input already carries the halo on the split dims."""
        p = ksize // 2
        return tuple(0 if d in self.dims else p for d in (2, 3, 4))

    # -- GroupNorm with global statistics (CPU / reference path) --------------------
    def group_norm_reference(self, x: torch.Tensor, groups: int, weight, bias, eps: float) -> torch.Tensor:
        n, c = x.shape[:2]
        xf = x.float().reshape(n, groups, -1)
        stats = torch.stack([xf.sum(-1), (xf * xf).sum(-1)])
        cnt = torch.tensor(float(xf.shape[-1]), device=x.device)
        stats = _AllReduceSumBoth.apply(stats, self)
        cnt = cnt * self.size
        mean = stats[0] / cnt
        var = (stats[1] / cnt - mean * mean).clamp_min(0.0)
        y = (xf - mean[..., None]) * torch.rsqrt(var + eps)[..., None]
        y = y.reshape(x.shape)
        shape = (1, c) + (1,) * (x.dim() - 2)
        return (y * weight.float().reshape(shape) + bias.float().reshape(shape)).to(x.dtype)

    # -- GroupNorm kernels with peer statistics (CUDA path) ---------------------------
    def gn_forward(self, x, w32, b32, groups, eps, relu, fin=None):
        """``fin``: this shard's finalised statistics when the producing convolution already computed them."""
        from ..ops import gn_kernels as gk
        if self.size == 1 or not self.gn_global:
            return gk.gn_forward(x, w32, b32, groups, eps, relu, fin=fin)
        if fin is None:
            fin = gk.gn_stats(x, w32, b32, groups, eps, relu)
        if self.stats_channel is not None:
            parts, wait = self.stats_channel.share(fin)
            return gk.gn_apply(x, w32, b32, groups, eps, relu, parts, shards=self.size, wait=wait)
        parts = self._gather_small(fin)
        return gk.gn_apply(x, w32, b32, groups, eps, relu, [p.data_ptr() for p in parts], shards=self.size)

    def gn_backward(self, gy, x, w32, b32, mean, rstd, groups, eps, relu):
        from ..ops import gn_kernels as gk
        if self.size == 1 or not self.gn_global:
            return gk.gn_backward(gy, x, w32, b32, mean, rstd, groups, eps, relu)
        fin = gk.gn_bwd_partial(gy, x, w32, b32, mean, rstd, groups, eps, relu)
        if self.stats_channel is not None:
            parts, wait = self.stats_channel.share(fin)
            return gk.gn_bwd_dx(gy, x, w32, b32, mean, rstd, groups, eps, relu, parts, shards=self.size, wait=wait)
        parts = self._gather_small(fin)
        return gk.gn_bwd_dx(gy, x, w32, b32, mean, rstd, groups, eps, relu, [p.data_ptr() for p in parts],
                            shards=self.size)

    def _gather_small(self, own: torch.Tensor) -> List[torch.Tensor]:
        """The spatial peers' copies of a small statistics tensor, own first, the rest in rank order."""
        others = [torch.empty_like(own) for _ in range(self.size)]
        dist.all_gather(others, own, group=self.group)
        me = self.layout.shard_id
        self._keep = others  # the kernels read these asynchronously
        return [others[me]] + [o for i, o in enumerate(others) if i != me]


class _AllReduceSumBoth(torch.autograd.Function):
    """Sum over the spatial group in forward AND backward (the statistics feed every shard's output)."""

    @staticmethod
    def forward(ctx, t, spatial):
        ctx.spatial = spatial
        out = t.clone()
        spatial.all_reduce_sum(out)
        return out

    @staticmethod
    def backward(ctx, g):
        g = g.clone()
        ctx.spatial.all_reduce_sum(g)
        return g, None


class _HaloPad(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, spatial, dim, halo):
        ctx.spatial, ctx.dim, ctx.halo = spatial, dim, halo
        n = x.shape[dim]
        if n < 2 * halo:
            raise ValueError(f"shard extent {n} along dim {dim} is thinner than twice the halo ({halo})")
        lo = x.narrow(dim, 0, halo)
        hi = x.narrow(dim, n - halo, halo)
        from_lo, from_hi = spatial._exchange(lo, hi, dim)
        return torch.cat([from_lo, x, from_hi], dim=dim)

    @staticmethod
    def backward(ctx, g):
        spatial, dim, halo = ctx.spatial, ctx.dim, ctx.halo
        n = g.shape[dim] - 2 * halo
        g_lo = g.narrow(dim, 0, halo)            # belongs to the - neighbour's high boundary
        g_hi = g.narrow(dim, n + halo, halo)     # belongs to the + neighbour's low boundary
        from_lo, from_hi = spatial._exchange(g_lo, g_hi, dim)
        gx = g.narrow(dim, halo, n).clone()
        gx.narrow(dim, 0, halo).add_(from_lo)
        gx.narrow(dim, n - halo, halo).add_(from_hi)
        return gx, None, None, None
