"""End-to-end plumbing on CPU/gloo at scale 4: one rank, two spatial shards, two replicas, resume."""
import csv
from pathlib import Path

import pytest

from helpers.launch import ROOT, results, torchrun_gloo

SCRIPT = ROOT / "tests" / "helpers" / "rank_scripts" / "benchmark_tiny.py"


def _run(tmp_path, nproc, shards_w, *extra):
    proc = torchrun_gloo(SCRIPT, nproc, [str(tmp_path), str(shards_w), *extra])
    assert proc.returncode == 0, proc.stdout[-3000:] + proc.stderr[-3000:]
    return results(proc.stdout)


@pytest.mark.slow
def test_two_spatial_shards_match_one_rank(tmp_path):
    one = _run(tmp_path, 1, 1)
    two = _run(tmp_path, 2, 2)
    assert one["final_epochs"] == ["2"] and two["final_epochs"] == ["2"]
    for key in ("epoch1", "epoch2"):
        a = [float(v) for v in one[key][0].split()]
        b = [float(v) for v in two[key][0].split()]
        # train loss, validation loss: fp32-level agreement; hard Dice: a few argmax near-ties may flip
        assert abs(a[0] - b[0]) <= 5e-4 * max(1.0, abs(a[0])), (key, a, b)
        assert abs(a[1] - b[1]) <= 5e-4 * max(1.0, abs(a[1])), (key, a, b)
        assert abs(a[2] - b[2]) <= 3e-3, (key, a, b)
    files = one["files"][0]
    for name in ("train_stats.csv", "checkpoints", "run_metadata.yaml", "figures"):
        assert name in files


@pytest.mark.slow
def test_two_replicas_run_and_resume(tmp_path):
    first = _run(tmp_path, 2, 1, "1", "{job_name: dp}")
    assert first["final_epochs"] == ["1"]
    run_dir = tmp_path / "run_w2_s1_dp"
    assert (run_dir / "checkpoints" / "checkpoint_last.pth").exists()
    again = _run(tmp_path, 2, 1, "3", f"{{job_name: dp, train_from_scratch: 0, restart: true, run_dir: '{run_dir}'}}")
    assert again["final_epochs"] == ["3"]
    with open(run_dir / "train_stats.csv") as f:
        epochs = [int(r["epoch"]) for r in csv.DictReader(f)]
    assert epochs == [1, 2, 3]  # the first epoch's row survived, training continued at epoch 2
    assert again["epoch1"] == first["epoch1"]


def test_device_prefetcher_passes_batches_through_on_cpu():
    import torch
    from scaffold_b200.train.prefetch import DevicePrefetcher
    batches = [{"image": torch.full((1, 2), float(i)), "mask": torch.tensor([i])} for i in range(4)]
    out = list(DevicePrefetcher(batches, "cpu"))
    assert len(out) == 4 and all(float(b["image"][0, 0]) == i for i, b in enumerate(out))
    assert len(DevicePrefetcher(batches, "cpu")) == 4


def test_engine_copies_the_loss_out_for_the_host():
    import torch
    from scaffold_b200.models.unet import UNet
    from scaffold_b200.train.engine import TrainEngine
    torch.manual_seed(0)
    model = UNet(3, 3, layers=1, base_width=8)
    eng = TrainEngine(model, torch.optim.Adam(model.parameters(), lr=1e-3), 3, "cpu", amp=False)
    with __import__("pytest").raises(RuntimeError):
        eng.read_loss()
    host = torch.zeros(1)
    loss = eng.step(torch.randn(1, 3, 8, 8, 8), torch.randint(0, 3, (1, 8, 8, 8)), loss_host=host)
    assert eng.read_loss() == float(loss)
