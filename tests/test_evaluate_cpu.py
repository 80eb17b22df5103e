"""The validation pass with a scripted engine: sample weighting over a ragged last batch, one host read at the end,
train / eval mode restored, and the CPU path of the batch prefetcher (role of ScaFFold/utils/evaluate.py:27-254)."""
import torch
import torch.nn as nn

from scaffold_b200.train.evaluate import evaluate
from scaffold_b200.train.prefetch import DevicePrefetcher


class _Engine:
    """eval_step returns a per-batch loss and per-(sample, class) Dice that depend on the batch only."""

    def __init__(self):
        self.model = nn.Linear(1, 1)
        self.device = torch.device("cpu")
        self.modes = []

    def eval_step(self, images, masks):
        self.modes.append(self.model.training)
        bs = images.shape[0]
        loss = images.reshape(bs, -1).mean()                       # mean over the batch, as a loss function returns it
        dice = torch.stack([torch.tensor([0.0, 0.2, 0.4]) + float(images[i].flatten()[0]) for i in range(bs)])
        return loss, dice


def _batches(sizes):
    out, k = [], 0
    for bs in sizes:
        img = torch.stack([torch.full((1, 2, 2, 2), float(k + i)) for i in range(bs)])
        out.append({"image": img, "mask": torch.zeros((bs, 2, 2, 2), dtype=torch.int16)})
        k += bs
    return out


def test_sums_are_sample_weighted_over_a_ragged_last_batch():
    eng = _Engine()
    eng.model.train()
    d_sum, l_sum, l_avg, n_batches, n_samples = evaluate(eng, _batches([2, 2, 1]))
    assert (n_batches, n_samples) == (3, 5)
    # sample i has value i everywhere: batch losses are 0.5, 2.5, 4.0, weighted by 2, 2, 1
    assert l_sum == 0.5 * 2 + 2.5 * 2 + 4.0 * 1 and l_avg == l_sum / 5
    # foreground Dice of sample i = mean(0.2 + i, 0.4 + i) = 0.3 + i, summed over the five samples
    assert abs(d_sum - sum(0.3 + i for i in range(5))) < 1e-6
    assert eng.modes == [False, False, False] and eng.model.training    # evaluated in eval mode, train mode restored
    eng.model.eval()
    evaluate(eng, _batches([1]))
    assert not eng.model.training                                        # an eval-mode model stays in eval mode


def test_empty_validation_split_gives_zeros_not_a_division_error():
    d_sum, l_sum, l_avg, n_batches, n_samples = evaluate(_Engine(), [])
    assert (d_sum, l_sum, l_avg, n_batches, n_samples) == (0.0, 0.0, 0.0, 0, 0)


def test_prefetcher_on_cpu_is_a_pass_through_that_counts_the_loader_wait():
    src = _batches([2, 1])
    pre = DevicePrefetcher(src, "cpu")
    got = list(pre)
    assert len(pre) == 2 and [g["image"] is s["image"] for g, s in zip(got, src)] == [True, True]
    assert pre.wait_s >= 0.0
    assert list(DevicePrefetcher([], "cpu")) == []
