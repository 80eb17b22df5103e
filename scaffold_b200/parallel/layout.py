"""Parallel layout: data-parallel replicas x spatial shards of the volume.

``ParallelLayout`` is this framework's equivalent of DistConv's
``ParallelStrategy`` as the reference uses it (ScaFFold/worker.py:236-240,
ScaFFold/utils/trainer.py:128-168,340-363): ranks form a row-major mesh
``(ddp, *num_shards)``, i.e. ``rank = ddp_ind * prod(num_shards) + shard_id``
with ``shard_id`` row-major over ``num_shards``. Weights are replicated on
every rank; a gradient is summed over the spatial shards of a replica and
averaged over the replicas (ScaFFold/unet/conv3d.py:66-71).

Process groups (created collectively, same order on every rank):
``ddp_group`` (same shard, all replicas), ``spatial_group`` (all shards of one
replica) and one group per sharded dim (the line of neighbours along it).
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Sequence, Tuple

from ..utils.sharding import (normalize_sharding, shard_id_to_indices, shard_indices_to_id, total_shards)


class ParallelLayout:
    def __init__(self, num_shards: Sequence[int] = (1, 1, 1), shard_dims: Sequence[int] = (2, 3, 4),
                 world_size: int = 1, rank: int = 0, make_groups: bool = True):
        self.num_shards, self.shard_dim = normalize_sharding(num_shards, shard_dims)
        self.world_size, self.rank = int(world_size), int(rank)
        self.spatial_size = total_shards(self.num_shards)
        if self.world_size % self.spatial_size != 0:
            raise ValueError(
                f"world size {self.world_size} is not a multiple of prod(dc_num_shards)={self.spatial_size}")
        self.ddp_ranks = self.world_size // self.spatial_size
        self.ddp_ind = self.rank // self.spatial_size
        self.shard_id = self.rank % self.spatial_size
        self.shard_ind = shard_id_to_indices(self.shard_id, self.num_shards)
        self.distconv_dim_names = tuple(f"dc{d}" for d in self.shard_dim)
        self.ddp_group = None
        self.spatial_group = None
        self.dim_groups: Dict[int, object] = {}
        if make_groups and self.world_size > 1:
            self._make_groups()

    # -- rank arithmetic ----------------------------------------------------
    def rank_of(self, ddp_ind: int, shard_indices: Sequence[int]) -> int:
        return ddp_ind * self.spatial_size + shard_indices_to_id(shard_indices, self.num_shards)

    def shard_to_rank(self, shard_indices: Sequence[int], periodic: bool = False) -> Optional[int]:
        """Rank (within this replica) that owns the shard at ``shard_indices``; None outside the volume."""
        idx = list(shard_indices)
        for k, n in enumerate(self.num_shards):
            if not 0 <= idx[k] < n:
                if not periodic:
                    return None
                idx[k] %= n
        return self.rank_of(self.ddp_ind, idx)

    def neighbour(self, dim: int, direction: int) -> Optional[int]:
        """Rank of the spatial neighbour along tensor dim ``dim`` (-1 / +1), None at the volume boundary."""
        k = self.shard_dim.index(dim)
        idx = list(self.shard_ind)
        idx[k] += direction
        return self.shard_to_rank(idx)

    def spatial_ranks(self) -> List[int]:
        base = self.ddp_ind * self.spatial_size
        return list(range(base, base + self.spatial_size))

    def ddp_peer_ranks(self) -> List[int]:
        return [r * self.spatial_size + self.shard_id for r in range(self.ddp_ranks)]

    def sharded_dims(self) -> List[int]:
        return [d for d, n in zip(self.shard_dim, self.num_shards) if n > 1]

    def grad_scale(self) -> float:
        """Factor applied to a gradient summed over ALL ranks: sum over shards, mean over replicas."""
        return 1.0 / self.ddp_ranks

    # -- groups -------------------------------------------------------------
    def _make_groups(self) -> None:
        import torch.distributed as dist
        sp, dp = self.spatial_size, self.ddp_ranks
        for shard in range(sp):
            ranks = [r * sp + shard for r in range(dp)]
            g = dist.new_group(ranks) if dp > 1 else None
            if shard == self.shard_id:
                self.ddp_group = g
        for rep in range(dp):
            ranks = list(range(rep * sp, (rep + 1) * sp))
            g = dist.new_group(ranks) if sp > 1 else None
            if rep == self.ddp_ind:
                self.spatial_group = g
        for k, (d, n) in enumerate(zip(self.shard_dim, self.num_shards)):
            if n == 1:
                continue
            # one group per line of shards along dim d, for every replica
            others = [range(m) for j, m in enumerate(self.num_shards) if j != k]
            import itertools
            for rep in range(dp):
                for fixed in itertools.product(*others):
                    ranks = []
                    for i in range(n):
                        idx = list(fixed)
                        idx.insert(k, i)
                        ranks.append(rep * sp + shard_indices_to_id(idx, self.num_shards))
                    g = dist.new_group(ranks)
                    if self.rank in ranks:
                        self.dim_groups[d] = g

    def __repr__(self) -> str:
        return (f"ParallelLayout(world={self.world_size}, rank={self.rank}, ddp={self.ddp_ranks}x, "
                f"shards={self.num_shards} on dims {self.shard_dim}, ddp_ind={self.ddp_ind}, shard_ind={self.shard_ind})")
