"""Library layout, mask scanner and seed derivation of the data generator
(roles of ScaFFold/datagen/layout.py:47-103, mask_detection.py:27-108 and the keyed seeding of the generator)."""
import logging
import pickle

import numpy as np
import pytest

from scaffold_b200.data import layout, mask_scan, rng


def test_library_paths_are_keyed_by_threshold_seed_and_point_count(tmp_path):
    root = layout.library_root(tmp_path, 0.05, 523)
    assert root == tmp_path / "var0.05" / "seed523"
    assert layout.library_root(tmp_path, 0.1, 523) != root and layout.library_root(tmp_path, 0.05, 524) != root
    assert layout.library_root(tmp_path, 0.050, 523) == root            # the same threshold written differently
    assert layout.params_dir(tmp_path, 0.05, 523) == root / "3DIFS_param"
    inst = layout.instances_dir(tmp_path, 0.05, 523, 100000)
    assert inst == root / "instances" / "np100000"
    assert layout.category_name(7) == "000007"
    assert layout.instance_path(inst, 7, 12) == inst / "000007" / "000007_0012.npy"


def test_legacy_tree_is_reported_not_reused(tmp_path, caplog):
    layout.warn_if_legacy_layout(tmp_path, logging.getLogger("t"))      # nothing there: silent
    assert not caplog.records
    (tmp_path / "3DIFS_param").mkdir()
    with caplog.at_level(logging.WARNING):
        layout.warn_if_legacy_layout(tmp_path, logging.getLogger("t"))
    assert any("legacy fractal layout" in r.getMessage() for r in caplog.records)
    layout.warn_if_legacy_layout(tmp_path, None)                        # no logger: still no error


@pytest.mark.parametrize("workers", [1, 2])
def test_mask_scanner_collects_the_union_of_label_values(tmp_path, workers):
    np.save(tmp_path / "a_mask.npy", np.array([[0, 3], [3, 0]], dtype=np.int16))
    np.save(tmp_path / "b_mask.npy", np.array([[0, 5], [1, 0]], dtype=np.int16))
    (tmp_path / "notes.txt").write_text("not a mask")
    assert mask_scan.scan(tmp_path, workers=workers) == [0, 1, 3, 5]
    out = tmp_path / "vals.pkl"
    assert mask_scan.main([str(tmp_path), str(out), "--workers", str(workers)]) == 0
    assert pickle.loads(out.read_bytes()) == {"mask_values": [0, 1, 3, 5]}
    with pytest.raises(FileNotFoundError):
        mask_scan.scan(tmp_path / "nowhere", workers=1)


def test_seed_derivation_is_keyed_stable_and_gives_independent_streams():
    a, b = rng.derive_seed(523, 1, 2), rng.derive_seed(523, 2, 1)
    assert a == rng.derive_seed(523, 1, 2) and a != b                   # stable, order-sensitive
    assert 0 <= a < 2 ** 64
    g1, g2 = rng.generator(523, 1), rng.generator(523, 1)
    assert np.array_equal(g1.random(5), g2.random(5))                   # the same keys replay the same stream
    assert not np.array_equal(rng.generator(523, 1).random(5), rng.generator(523, 2).random(5))
