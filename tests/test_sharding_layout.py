"""Spatial sharding arithmetic and the rank <-> (replica, shard) mapping (CPU only)."""
import pytest
import torch

from scaffold_b200.parallel.layout import ParallelLayout
from scaffold_b200.utils import sharding as S


def test_shard_id_roundtrip_and_row_major():
    ns = (2, 3, 2)
    ids = [S.shard_indices_to_id(S.shard_id_to_indices(i, ns), ns) for i in range(12)]
    assert ids == list(range(12))
    assert S.shard_id_to_indices(1, ns) == (0, 0, 1) and S.shard_id_to_indices(2, ns) == (0, 1, 0)


@pytest.mark.parametrize("extent,parts", [(16, 2), (10, 4), (7, 3), (5, 8)])
def test_chunk_slice_matches_torch_chunk(extent, parts):
    chunks = torch.arange(extent).chunk(parts)
    for i in range(parts):
        sl = S.chunk_slice(extent, parts, i)
        want = chunks[i].tolist() if i < len(chunks) else []
        assert list(range(extent))[sl] == want


def test_spatial_slices_and_suffix():
    sl = S.spatial_slices((16, 16, 16), (1, 1, 2), (2, 3, 4), 1)
    assert sl == (slice(0, 16), slice(0, 16), slice(8, 16))
    assert S.shard_file_suffix(3) == "_shard000003"
    assert S.canonical_sharding((2, 1), (4, 2)) == ((1, 2), (2, 4))
    with pytest.raises(ValueError):
        S.normalize_sharding((2,), (1,))


def test_layout_rank_mapping_and_neighbours():
    world, ns = 8, (2, 1, 2)
    seen = set()
    for r in range(world):
        lay = ParallelLayout(ns, (2, 3, 4), world, r, make_groups=False)
        assert lay.ddp_ranks == 2 and lay.spatial_size == 4
        assert lay.rank_of(lay.ddp_ind, lay.shard_ind) == r
        seen.add((lay.ddp_ind, lay.shard_ind))
        assert lay.grad_scale() == 0.5
    assert len(seen) == world
    lay = ParallelLayout(ns, (2, 3, 4), world, 5, make_groups=False)  # replica 1, shard (0,0,1)
    assert lay.shard_ind == (0, 0, 1)
    assert lay.neighbour(4, -1) == 4 and lay.neighbour(4, +1) is None
    assert lay.neighbour(2, +1) == 7 and lay.neighbour(2, -1) is None
    assert lay.sharded_dims() == [2, 4]
    with pytest.raises(ValueError):
        ParallelLayout((1, 1, 3), (2, 3, 4), 8, 0, make_groups=False)
