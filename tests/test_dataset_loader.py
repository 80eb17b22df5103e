"""The dataset loader on hand-made tiny datasets: the three on-disk formats, layout checks, id rules.

(Reading side of ScaFFold/utils/data_loading.py:40-594; the generated-dataset round trips live in test_datagen.py.)
"""
import pickle

import numpy as np
import pytest
import torch
import yaml

from scaffold_b200.data.dataset import FractalDataset, SpatialShardSpec, load_dataset_metadata
from scaffold_b200.utils.sharding import shard_file_suffix


def _dirs(root, split="training"):
    v, m = root / "volumes" / split, root / "masks" / split
    v.mkdir(parents=True)
    m.mkdir(parents=True)
    return v, m


def _volume(seed, shape=(4, 6, 8)):
    rng = np.random.default_rng(seed)
    return rng.random((3, *shape), dtype=np.float32), rng.integers(0, 4, shape).astype(np.int16)


def _write_v2(root, n=3):
    v, m = _dirs(root)
    (root / "meta.yaml").write_text(yaml.safe_dump({"dataset_format_version": 2}))
    items = {}
    for i in range(n):
        img, mask = _volume(i)
        np.save(v / f"{i}.npy", img)
        np.save(m / f"{i}_mask.npy", mask)
        items[str(i)] = (img, mask)
    return v, m, items


def test_whole_volume_format_is_sliced_on_load(tmp_path):
    v, m, items = _write_v2(tmp_path)
    whole = FractalDataset(v, m)
    assert len(whole) == 3 and whole.ids == ["0", "1", "2"] and not whole.physical
    s = whole[1]
    assert s["image"].dtype == torch.float32 and s["mask"].dtype == torch.int16
    assert torch.equal(s["image"], torch.from_numpy(items["1"][0])) and torch.equal(s["mask"], torch.from_numpy(items["1"][1]))
    assert torch.equal(whole.load_mask_only(2), torch.from_numpy(items["2"][1]))
    # two shards along W (tensor dim 4): each rank reads its half, the halves tile the volume
    halves = [FractalDataset(v, m, spatial_shard_spec=SpatialShardSpec((1, 1, 2), (2, 3, 4), (0, 0, k))) for k in (0, 1)]
    got = torch.cat([h[0]["image"] for h in halves], dim=3)
    assert torch.equal(got, torch.from_numpy(items["0"][0]))
    assert torch.equal(torch.cat([h[0]["mask"] for h in halves], dim=2), torch.from_numpy(items["0"][1]))
    assert halves[0][0]["image"].shape == (3, 4, 6, 4) and halves[0][0]["image"].is_contiguous()


def test_physical_shard_format_reads_only_its_own_files_and_checks_the_layout(tmp_path):
    v, m = _dirs(tmp_path)
    (tmp_path / "meta.yaml").write_text(yaml.safe_dump(
        {"dataset_format_version": 5, "config_subset": {"dc_num_shards": [1, 1, 2], "dc_shard_dims": [2, 3, 4]}}))
    img, mask = _volume(7)
    for k in (0, 1):
        suf = shard_file_suffix(k)
        np.save(v / f"0{suf}.npy", img[..., k * 4:(k + 1) * 4])
        np.save(m / f"0{suf}_mask.npy", mask[..., k * 4:(k + 1) * 4])
    parts = [FractalDataset(v, m, spatial_shard_spec=SpatialShardSpec((1, 1, 2), (2, 3, 4), (0, 0, k))) for k in (0, 1)]
    assert all(p.physical and p.ids == ["0"] for p in parts)
    assert torch.equal(torch.cat([p[0]["image"] for p in parts], dim=3), torch.from_numpy(img))
    # the same layout written with the dims in another order is the same layout
    FractalDataset(v, m, spatial_shard_spec=SpatialShardSpec((2, 1, 1), (4, 3, 2), (1, 0, 0)))
    # another layout cannot be cut out of physical shards
    with pytest.raises(ValueError, match="cannot be re-cut"):
        FractalDataset(v, m, spatial_shard_spec=SpatialShardSpec((2, 1, 1), (2, 3, 4), (0, 0, 0)))
    with pytest.raises(ValueError, match="cannot be re-cut"):
        FractalDataset(v, m)  # whole volumes from a two-shard dataset
    # a physical dataset without its shard metadata is refused
    (tmp_path / "meta.yaml").write_text(yaml.safe_dump({"dataset_format_version": 5}))
    with pytest.raises(RuntimeError, match="missing shard metadata"):
        FractalDataset(v, m, spatial_shard_spec=SpatialShardSpec((1, 1, 2), (2, 3, 4), (0, 0, 0)))


def test_legacy_directory_remaps_label_values_and_moves_channels_first(tmp_path):
    v, m = _dirs(tmp_path)
    rng = np.random.default_rng(3)
    img = rng.random((4, 6, 8, 3), dtype=np.float32)          # channels last, no meta.yaml
    values = [0, 17, 40, 255]                                  # arbitrary label values
    idx = rng.integers(0, 4, (4, 6, 8))
    np.save(v / "5.npy", img)
    np.save(m / "5_mask.npy", np.asarray(values)[idx].astype(np.int32))
    with open(tmp_path / "train_unique_mask_vals", "wb") as f:
        pickle.dump({"mask_values": values}, f)
    ds = FractalDataset(v, m)
    assert ds.version == 1 and load_dataset_metadata(tmp_path) == {"dataset_format_version": 1}
    s = ds[0]
    assert s["image"].shape == (3, 4, 6, 8) and torch.equal(s["image"], torch.from_numpy(np.moveaxis(img, -1, 0).copy()))
    assert torch.equal(s["mask"], torch.from_numpy(idx.astype(np.int16)))


def test_id_rules_and_damaged_metadata(tmp_path):
    v, m, _ = _write_v2(tmp_path, n=11)
    ds = FractalDataset(v, m)
    assert ds.ids == [str(i) for i in range(11)]               # numeric order, not "0, 1, 10, 2"
    (v / ".hidden.npy").write_bytes(b"")                        # dot files and other suffixes are not samples
    (v / "notes.txt").write_text("x")
    assert FractalDataset(v, m).ids == ds.ids
    (m / "4_mask.npy").unlink()
    with pytest.raises(RuntimeError, match="no mask or multiple masks"):
        FractalDataset(v, m)[4]
    (tmp_path / "meta.yaml").write_text(yaml.safe_dump({"dataset_format_version": 9}))
    with pytest.raises(RuntimeError, match="Unsupported dataset format version 9"):
        FractalDataset(v, m)
    (tmp_path / "meta.yaml").write_text("dataset_format_version: [unclosed")
    with pytest.raises(ValueError, match="could not be read"):
        FractalDataset(v, m)
    (tmp_path / "meta.yaml").write_text(yaml.safe_dump({"something": 1}))
    with pytest.raises(ValueError, match="missing a usable 'dataset_format_version'"):
        FractalDataset(v, m)
    empty_v, empty_m = _dirs(tmp_path / "other")
    with pytest.raises(RuntimeError, match="No input file found"):
        FractalDataset(empty_v, empty_m)


def test_shard_spec_normalises_and_numbers_shards_row_major():
    s = SpatialShardSpec((2, 1, 2), (2, 3, 4), (1, 0, 1))
    assert s.total == 4 and s.shard_id == 3
    assert SpatialShardSpec().total == 1 and SpatialShardSpec().shard_id == 0
