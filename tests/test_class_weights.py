"""Cross-entropy class weights from a sample of training masks (role of ScaFFold/utils/losses.py:42-114):
background keeps its own inverse frequency, all fractal classes share the foreground's."""
import logging

import torch

from scaffold_b200.train.trainer import compute_ce_class_weights, sample_ce_weight_indices


class _Masks:
    """A dataset that only knows its masks (the loader's ``load_mask_only`` fast path)."""

    def __init__(self, masks):
        self.masks = masks
        self.full_reads = 0

    def __len__(self):
        return len(self.masks)

    def load_mask_only(self, i):
        return self.masks[i]

    def __getitem__(self, i):
        self.full_reads += 1
        return {"mask": self.masks[i]}


def test_weights_are_total_over_background_and_total_over_foreground():
    m = torch.zeros(10, 10, dtype=torch.int16)
    m[:2] = 1                                   # 20 voxels of class 1
    m[2, :5] = 3                                # 5 voxels of class 3 -> 25 foreground, 75 background
    ds = _Masks([m] * 10)
    w = compute_ce_class_weights(ds, 4, "cpu", sample_fraction=0.5)
    assert w.shape == (5,) and w.dtype == torch.float32
    assert torch.allclose(w, torch.tensor([100 / 75] + [100 / 25] * 4))
    assert ds.full_reads == 0                   # masks only: no image was loaded for this


def test_fallbacks_are_uniform_and_logged(caplog):
    log = logging.getLogger("cw")
    only_bg = _Masks([torch.zeros(4, 4, dtype=torch.int16)] * 3)
    with caplog.at_level(logging.WARNING):
        w = compute_ce_class_weights(only_bg, 2, "cpu", 1.0, log)
    assert torch.equal(w, torch.ones(3)) and any("one kind is missing" in r.getMessage() for r in caplog.records)
    caplog.clear()
    with caplog.at_level(logging.WARNING):
        w = compute_ce_class_weights(_Masks([]), 2, "cpu", 0.1, log)
    assert torch.equal(w, torch.ones(3)) and any("training split is empty" in r.getMessage() for r in caplog.records)


def test_datasets_without_the_fast_path_are_read_through_getitem():
    class Plain:
        def __init__(self, masks):
            self.masks = masks

        def __len__(self):
            return len(self.masks)

        def __getitem__(self, i):
            return {"mask": self.masks[i]}

    m = torch.tensor([[0, 1], [2, 0]], dtype=torch.int16)
    w = compute_ce_class_weights(Plain([m, m]), 2, "cpu", 1.0)
    assert torch.allclose(w, torch.tensor([2.0, 2.0, 2.0]))


def test_sampled_indices_span_the_split_evenly():
    assert sample_ce_weight_indices(100, 0.1) == [0, 11, 22, 33, 44, 55, 66, 77, 88, 99]
    assert sample_ce_weight_indices(5, 1.0) == [0, 1, 2, 3, 4]
    assert sample_ce_weight_indices(3, 0.01) == [0]             # at least one mask
    assert sample_ce_weight_indices(0, 0.5) == []
