"""Device-resident validation cache (scaffold_b200/data/device_cache.py)."""
import pytest
import torch

from scaffold_b200.data.device_cache import CachedEvalLoader


class _Loader:
    """Counts how often it is walked."""

    def __init__(self, n=3):
        g = torch.Generator().manual_seed(0)
        self.batches = [{"image": torch.rand((1, 3, 4, 4, 4), generator=g),
                         "mask": torch.randint(0, 5, (1, 4, 4, 4), generator=g, dtype=torch.int16)} for _ in range(n)]
        self.walks = 0

    def __len__(self):
        return len(self.batches)

    def __iter__(self):
        self.walks += 1
        return iter(self.batches)


def test_cpu_device_or_zero_budget_is_a_plain_pass_through():
    src = _Loader()
    for budget in (0, 1 << 30):
        c = CachedEvalLoader(src, "cpu", budget if budget == 0 else budget)
        a = list(c)
        b = list(c)
        assert not c.resident and len(a) == len(b) == len(c) == 3
        assert all(x["image"] is y["image"] for x, y in zip(a, src.batches))
    assert src.walks == 4  # every pass walked the loader


def test_config_key_and_cli_flag(tmp_path):
    from scaffold_b200 import cli, config as C
    from test_config_cli import base_dict
    assert C.Config(base_dict(tmp_path)).val_cache_gb == 16.0
    assert C.Config(base_dict(tmp_path, val_cache_gb=0)).val_cache_gb == 0.0
    with pytest.raises(ValueError):
        C.Config(base_dict(tmp_path, val_cache_gb=-1))
    with pytest.raises(ValueError):
        C.Config(base_dict(tmp_path, val_cache_gb="lots"))
    assert "--val-cache-gb" in cli.BENCHMARK_FLAGS


@pytest.mark.gpu
def test_second_pass_replays_device_copies_and_the_metric_does_not_change():
    from scaffold_b200.models.unet import UNet
    from scaffold_b200.ops.optim import FusedClipAdam
    from scaffold_b200.train.engine import TrainEngine
    from scaffold_b200.train.evaluate import evaluate
    g = torch.Generator().manual_seed(1)
    batches = [{"image": torch.rand((1, 3, 32, 32, 32), generator=g).pin_memory(),
                "mask": torch.randint(0, 5, (1, 32, 32, 32), generator=g, dtype=torch.int16).pin_memory()}
               for _ in range(3)]
    src = _Loader()
    src.batches = batches
    torch.manual_seed(0)
    model = UNet(3, 5, layers=2, base_width=32).cuda()
    eng = TrainEngine(model, FusedClipAdam(model.parameters(), lr=1e-3, max_norm=1.0), 5, torch.device("cuda"))
    cached = CachedEvalLoader(src, "cuda", 1 << 30)
    first = evaluate(eng, cached)
    assert cached.resident and src.walks == 1
    assert cached.cached_bytes == 3 * (3 * 32 ** 3 * 2 + 32 ** 3 * 2)   # bf16 images + int16 masks
    second = evaluate(eng, cached)
    assert src.walks == 1                                              # no host work on the replay
    replay = list(cached)
    assert replay[0]["image"].is_cuda and replay[0]["image"].dtype == torch.bfloat16
    # bf16 images are what the stem's staging kernel rounds fp32 inputs to: same metric, same loss
    assert first[0] == second[0] and first[1] == second[1]
    small = CachedEvalLoader(src, "cuda", 1000)                        # does not fit: stays on the loader
    list(small)
    list(small)
    assert not small.resident and src.walks == 3


def test_primed_loader_hands_out_the_iterator_it_created_ahead_of_time():
    from scaffold_b200.train.trainer import PrimedLoader

    class Counting:
        def __init__(self):
            self.made = 0

        def __len__(self):
            return 3

        def __iter__(self):
            self.made += 1
            return iter(range(3))

    src = Counting()
    p = PrimedLoader(src)
    assert list(p) == [0, 1, 2] and src.made == 1      # not primed: a fresh iterator
    p.prime()
    assert src.made == 2                               # created now, ahead of its use
    assert list(p) == [0, 1, 2] and src.made == 2      # ... and handed out once
    assert list(p) == [0, 1, 2] and src.made == 3
    assert len(p) == 3
