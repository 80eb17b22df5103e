"""Data generation on CPU: chaos-game oracle parity, acceptance test, voxeliser, search/instances/volumes/cache."""
import pickle
from pathlib import Path
from types import SimpleNamespace

import numpy as np
import pytest
import yaml

from scaffold_b200 import config as C
from scaffold_b200.data import cache, category_search, ifs, instances, volumes
from scaffold_b200.data.dataset import FractalDataset, SpatialShardSpec
from scaffold_b200.data.rng import derive_seed


def tiny_config(tmp_path, **kw):
    d = yaml.safe_load(C.default_config_path().read_text())
    d.update(base_run_dir=str(tmp_path / "runs"), dataset_dir=str(tmp_path / "ds"), fract_base_dir=str(tmp_path / "fr"),
             problem_scale=4, unet_bottleneck_dim=3, n_categories=2, n_instances_used_per_fractal=6, n_fracts_per_vol=3,
             datagen_device="cpu", point_num_override=400)
    d.update(kw)
    return C.Config(d)


def test_derive_seed_is_stable_and_order_sensitive():
    assert derive_seed(1, 2, 3) == derive_seed(1, 2, 3)
    assert derive_seed(1, 2, 3) != derive_seed(3, 2, 1)
    assert 0 <= derive_seed(2**40, 7) < 2**32


def test_native_orbit_matches_numpy_oracle():
    params = category_search.propose_params(523, 0, 11)
    pts, flags = ifs.orbit_points(params[None], np.array([12345], dtype=np.uint64), 300, device="cpu")
    ref, ok = ifs.orbit_numpy(params, 12345, 300)
    assert flags[0] == (0 if ok else 1)
    np.testing.assert_array_equal(pts[0], ref.astype(np.float32))
    stats = ifs.orbit_stats(params[None], np.array([12345], dtype=np.uint64), 300, device="cpu")[0]
    np.testing.assert_allclose(stats[0:3], ref.min(0))
    np.testing.assert_allclose(stats[3:6], ref.max(0))
    np.testing.assert_allclose(stats[6:9], ref.mean(0), rtol=1e-10, atol=1e-12)
    np.testing.assert_allclose(stats[9:12], ref.var(0), rtol=1e-8, atol=1e-12)


def test_acceptance_rules():
    ok = np.array([[-1, -1, -1, 1, 1, 1, 0, 0, 0, .3, .3, .3, 100, 0, 0, 0]], dtype=float)
    assert ifs.accept(ok, 1.0, 0.15)[0][0]
    low = ok.copy(); low[0, 9] = 0.01
    assert ifs.accept(low, 1.0, 0.15)[1][0] == 2
    run = ok.copy(); run[0, 13] = 1
    assert ifs.accept(run, 1.0, 0.15)[1][0] == 3
    nf = ok.copy(); nf[0, 14] = 1
    assert ifs.accept(nf, 1.0, 0.15)[1][0] == 1
    flat = ok.copy(); flat[0, 3] = -1  # zero range on x
    assert not ifs.accept(flat, 1.0, 0.15)[0][0]


def test_voxelizer_matches_numpy_and_rejects_nonfinite():
    rng = np.random.default_rng(0)
    pts = (rng.standard_normal((500, 3)) * [1.0, 0.5, 0.25]).astype(np.float32)
    occ = ifs.voxelize_cpu(pts, 16)
    idx = ifs.points_to_voxel_indices(pts, 16)
    ref = np.zeros((16, 16, 16), dtype=np.uint8)
    ref[idx[:, 0], idx[:, 1], idx[:, 2]] = 1
    np.testing.assert_array_equal(occ, ref)
    assert occ[:, :, :].any(axis=(1, 2)).sum() == 16  # the longest axis fills the grid
    bad = pts.copy(); bad[3, 1] = np.nan
    with pytest.raises(ValueError, match="non-finite"):
        ifs.voxelize_cpu(bad, 16)
    with pytest.raises(ValueError, match="non-finite"):
        ifs.points_to_voxel_indices(bad, 16)


def test_instance_weight_table_shape_and_quirks():
    w = instances.instance_weights()
    assert w.shape == (145, 12) and (w[6] == 1).all()
    assert w[0, 0] == 0.4 and w[12, 0] == 1.6 and w[13, 1] == 0.4 and w[108, 8] == 0.6 and w[144, 11] == 1.6
    assert ((w != 1).sum(1) <= 1).all()


def test_search_instances_volumes_cache_end_to_end(tmp_path):
    cfg = tiny_config(tmp_path)
    assert category_search.main(cfg) == 2
    pdir = category_search.params_dir(cfg.fract_base_dir, cfg.variance_threshold, cfg.dataset_seed)
    cats = category_search.existing_categories(pdir)
    assert sorted(cats) == [0, 1] and all(v.shape == (2, 13) for v in cats.values())
    counter = category_search.load_attempt_counter(pdir, 0)
    assert counter > 0
    assert category_search.main(cfg) == 2  # nothing left to do
    assert category_search.load_attempt_counter(pdir, 0) == counter
    n = instances.main(cfg)
    assert n == 2 * 145 and instances.main(cfg) == 0  # second call finds every file valid
    # dataset through the cache
    path = cache.get_dataset(cfg)
    assert path.parent.name == cache.config_id(cfg) and (path / "meta.yaml").exists()
    assert cache.get_dataset(cfg) == path  # reused, not regenerated
    contents = np.loadtxt(path / "volumes_contents.csv", delimiter=",", dtype=int)
    assert contents.shape == (4, 7)
    with open(path / "train_unique_mask_vals", "rb") as f:
        assert pickle.load(f)["mask_values"][0] == 0
    ds = FractalDataset(path / "volumes" / "training", path / "masks" / "training", str(path))
    item = ds[0]
    assert item["image"].shape == (3, 16, 16, 16) and item["image"].dtype.is_floating_point
    assert item["mask"].shape == (16, 16, 16) and str(item["mask"].dtype) == "torch.int16"
    assert set(np.unique(item["mask"].numpy())) <= {0, 1, 2}
    assert (item["image"].numpy()[:, item["mask"].numpy() == 0] == 0).all()
    assert ds.load_mask_only(0).equal(item["mask"])


def test_sharded_dataset_files_tile_the_whole_volume(tmp_path):
    cfg1 = tiny_config(tmp_path)
    category_search.main(cfg1)
    instances.main(cfg1)
    whole = cache.get_dataset(cfg1)
    cfg2 = tiny_config(tmp_path, dc_num_shards=[1, 1, 2])
    assert cache.config_id(cfg1) != cache.config_id(cfg2)
    sharded = cache.get_dataset(cfg2)
    full = FractalDataset(whole / "volumes" / "training", whole / "masks" / "training", str(whole))
    parts = [FractalDataset(sharded / "volumes" / "training", sharded / "masks" / "training", str(sharded),
                            SpatialShardSpec((1, 1, 2), (2, 3, 4), (0, 0, i))) for i in range(2)]
    assert full.ids == parts[0].ids == parts[1].ids
    a, b, w = parts[0][0], parts[1][0], full[0]
    assert a["image"].shape == (3, 16, 16, 8)
    import torch
    assert torch.equal(torch.cat([a["image"], b["image"]], -1), w["image"])
    assert torch.equal(torch.cat([a["mask"], b["mask"]], -1), w["mask"])
    with pytest.raises(ValueError, match="shard layout"):
        FractalDataset(sharded / "volumes" / "training", sharded / "masks" / "training", str(sharded))


def test_reference_dataset_class_reads_a_generated_sharded_dataset(tmp_path):
    """Format interchange: the reference's own ``FractalDataset`` (when its package is installed under
    ``baseline/_ref``) opens a dataset this framework wrote, meta.yaml included, and returns the same tensors."""
    import sys
    from pathlib import Path
    ref = Path(__file__).resolve().parents[1] / "baseline" / "_ref"
    if not (ref / "ScaFFold").exists():
        pytest.skip("the reference package is not installed under baseline/_ref")
    cfg = tiny_config(tmp_path, dc_num_shards=[1, 1, 2])
    category_search.main(cfg)
    instances.main(cfg)
    path = cache.get_dataset(cfg)
    import yaml
    meta = yaml.safe_load((path / "meta.yaml").read_text())
    assert meta["config_subset"]["dc_num_shards"] and meta["dataset_format_version"] == 5 and meta["code_commit"]
    sys.path.insert(0, str(ref))
    try:
        from ScaFFold.utils.data_loading import FractalDataset as RefDataset, SpatialShardSpec as RefSpec
    except Exception as exc:  # a dependency of the reference is missing here
        pytest.skip(f"reference data loader does not import: {exc}")
    finally:
        sys.path.remove(str(ref))
    import torch
    for i in range(2):
        theirs = RefDataset(str(path / "volumes" / "training"), str(path / "masks" / "training"),
                            str(path / "train_unique_mask_vals"), RefSpec((2, 3, 4), (1, 1, 2), (0, 0, i)))
        ours = FractalDataset(path / "volumes" / "training", path / "masks" / "training", str(path),
                              SpatialShardSpec((1, 1, 2), (2, 3, 4), (0, 0, i)))
        assert len(theirs) == len(ours)
        assert torch.equal(theirs[0]["image"], ours[0]["image"])
        assert torch.equal(theirs[0]["mask"].long(), ours[0]["mask"].long())


def test_cache_key_ignores_irrelevant_keys_and_canonicalises_shard_order(tmp_path):
    a = tiny_config(tmp_path)
    b = tiny_config(tmp_path, local_batch_size=4, training_seed=7)
    assert cache.config_id(a) == cache.config_id(b)
    c = tiny_config(tmp_path, dc_num_shards=[2, 1, 1], dc_shard_dims=[2, 3, 4])
    d = tiny_config(tmp_path, dc_num_shards=[1, 1, 2], dc_shard_dims=[4, 3, 2])
    assert cache.config_id(c) == cache.config_id(d)


def test_stale_staging_is_swept_but_live_staging_is_kept(tmp_path):
    idd = tmp_path / "abc"
    (idd / ".tmp_old").mkdir(parents=True)
    (idd / ".tmp_live").mkdir()
    (idd / ".tmp_live" / volumes.HEARTBEAT_FILE).write_text("x")
    import os, time
    old = time.time() - 3 * 24 * 3600
    os.utime(idd / ".tmp_old", (old, old))
    assert cache.sweep_stale_staging(idd) == 1
    assert not (idd / ".tmp_old").exists() and (idd / ".tmp_live").exists()


def test_damaged_meta_is_an_error_not_a_legacy_fallback(tmp_path):
    root = tmp_path / "d"
    (root / "volumes" / "training").mkdir(parents=True)
    (root / "masks" / "training").mkdir(parents=True)
    (root / "meta.yaml").write_text("dataset_format_version: [oops")
    with pytest.raises(ValueError, match="could not be read"):
        FractalDataset(root / "volumes" / "training", root / "masks" / "training")
    (root / "meta.yaml").write_text("something: 1\n")
    with pytest.raises(ValueError, match="missing a usable"):
        FractalDataset(root / "volumes" / "training", root / "masks" / "training")
