"""Spatial sharding arithmetic shared by the dataset writer, the loader and the parallel layout.

Conventions (ScaFFold/utils/spatial_sharding.py:19-133): ``dc_shard_dims`` name
tensor dims in NCDHW numbering (2 = D, 3 = H, 4 = W); shard ids are row-major
over ``dc_num_shards`` in the order the dims are listed; extents are split the
way ``torch.chunk`` splits them (ceil-sized chunks, the tail may be short or
empty); shard files carry the suffix ``_shard%06d``.
"""
from __future__ import annotations

import math
from typing import List, Sequence, Tuple

SPATIAL_DIMS = (2, 3, 4)


def normalize_sharding(num_shards: Sequence[int], shard_dims: Sequence[int]) -> Tuple[Tuple[int, ...], Tuple[int, ...]]:
    num_shards, shard_dims = tuple(int(v) for v in num_shards), tuple(int(v) for v in shard_dims)
    if len(num_shards) != len(shard_dims):
        raise ValueError(f"num_shards {num_shards} and shard_dims {shard_dims} must have the same length")
    if len(set(shard_dims)) != len(shard_dims):
        raise ValueError(f"shard_dims {shard_dims} repeats a dimension")
    for d in shard_dims:
        if d not in SPATIAL_DIMS:
            raise ValueError(f"shard dim {d} is not spatial; batch (0) and channel (1) are never sharded")
    for n in num_shards:
        if n < 1:
            raise ValueError(f"shard counts must be >= 1; got {num_shards}")
    return num_shards, shard_dims


def canonical_sharding(num_shards: Sequence[int], shard_dims: Sequence[int]):
    """Sort by dim so that equivalent layouts written in a different order compare equal."""
    num_shards, shard_dims = normalize_sharding(num_shards, shard_dims)
    pairs = sorted(zip(shard_dims, num_shards))
    return tuple(n for _, n in pairs), tuple(d for d, _ in pairs)


def total_shards(num_shards: Sequence[int]) -> int:
    return math.prod(int(n) for n in num_shards)


def shard_id_to_indices(shard_id: int, num_shards: Sequence[int]) -> Tuple[int, ...]:
    if not 0 <= shard_id < total_shards(num_shards):
        raise ValueError(f"shard id {shard_id} out of range for {tuple(num_shards)}")
    idx: List[int] = []
    for n in reversed(tuple(num_shards)):
        idx.append(shard_id % n)
        shard_id //= n
    return tuple(reversed(idx))


def shard_indices_to_id(indices: Sequence[int], num_shards: Sequence[int]) -> int:
    sid = 0
    for i, n in zip(indices, num_shards):
        if not 0 <= i < n:
            raise ValueError(f"shard index {tuple(indices)} out of range for {tuple(num_shards)}")
        sid = sid * n + i
    return sid


def chunk_slice(extent: int, parts: int, index: int) -> slice:
    """The ``index``-th piece of ``torch.chunk(range(extent), parts)`` (may be empty)."""
    step = -(-extent // parts)
    start = min(index * step, extent)
    return slice(start, min(start + step, extent))


def spatial_slices(shape_dhw: Sequence[int], num_shards: Sequence[int], shard_dims: Sequence[int],
                   shard_id: int) -> Tuple[slice, slice, slice]:
    """(D, H, W) slices of shard ``shard_id`` of a volume of extent ``shape_dhw``."""
    num_shards, shard_dims = normalize_sharding(num_shards, shard_dims)
    idx = shard_id_to_indices(shard_id, num_shards)
    out = [slice(0, int(e)) for e in shape_dhw]
    for i, n, d in zip(idx, num_shards, shard_dims):
        out[d - 2] = chunk_slice(int(shape_dhw[d - 2]), n, i)
    return tuple(out)


def shard_file_suffix(shard_id: int) -> str:
    return f"_shard{shard_id:06d}"
