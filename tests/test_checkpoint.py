"""Checkpoint manager: format, atomic write, corrupt fallback, failure broadcast, state-dict interchange (CPU)."""
import torch
import torch.nn as nn
import pytest

from scaffold_b200.models.unet import UNet
from scaffold_b200.train import checkpoint as ck


def _bits():
    torch.manual_seed(0)
    model = UNet(3, 4, layers=1, base_width=8)
    opt = torch.optim.Adam(model.parameters(), lr=1e-3)
    sched = torch.optim.lr_scheduler.CosineAnnealingWarmRestarts(opt, T_0=10, T_mult=2, eta_min=1e-4)
    model(torch.randn(1, 3, 8, 8, 8)).sum().backward()
    opt.step()
    return model, opt, sched


def test_save_load_roundtrip_and_keys(tmp_path):
    model, opt, sched = _bits()
    mgr = ck.CheckpointManager(tmp_path, "checkpoints")
    assert mgr.save(3, 0.5, model, opt, sched, extras={"val_dice": 0.7, "global_step": 9}) is True
    state = torch.load(mgr.last_path, weights_only=False)
    for key in ("epoch", "val_loss_avg", "model_state_dict", "optimizer_state_dict", "grad_scaler_state_dict",
                "scheduler_state_dict", "rng_state_pytorch", "rng_state_pytorch_cuda", "rng_state_numpy",
                "rng_state_python", "val_dice", "global_step"):
        assert key in state
    assert mgr.best_path.read_bytes() == mgr.last_path.read_bytes()
    assert mgr.save(4, 0.9, model, opt, sched) is False  # not better: best keeps epoch 3
    assert torch.load(mgr.best_path, weights_only=False)["epoch"] == 3
    m2, o2, s2 = _bits()
    for p in m2.parameters():
        p.data.add_(1.0)
    info = ck.CheckpointManager(tmp_path, "checkpoints").load(m2, o2, s2)
    assert info["epoch"] == 4 and info["_loaded_from"] == ck.LAST_NAME
    for a, b in zip(model.state_dict().values(), m2.state_dict().values()):
        assert torch.equal(a, b)
    assert not list(mgr.dir.glob(f"*{ck.TMP_MARK}*"))


def test_state_dict_is_interchangeable_with_stock_modules(tmp_path):
    model, _, _ = _bits()
    sd = model.state_dict()
    assert "down_list.0.double_conv.0.weight" in sd and "down_list.1.maxpool_conv.1.double_conv.4.bias" in sd
    assert "up_list.0.up.weight" in sd and "up_list.1.conv.bias" in sd
    assert sd["up_list.0.up.weight"].shape == (16, 8, 2, 2, 2)
    stock = nn.Sequential(nn.Conv3d(3, 8, 3, padding=1, bias=False), nn.GroupNorm(8, 8))
    stock[0].load_state_dict({"weight": sd["down_list.0.double_conv.0.weight"]})
    stock[1].load_state_dict({"weight": sd["down_list.0.double_conv.1.weight"],
                              "bias": sd["down_list.0.double_conv.1.bias"]})
    assert not list(model.buffers())


def test_corrupt_last_is_quarantined_and_best_is_used(tmp_path):
    model, opt, sched = _bits()
    mgr = ck.CheckpointManager(tmp_path, "checkpoints")
    mgr.save(1, 0.5, model, opt, sched)
    mgr.last_path.write_bytes(mgr.last_path.read_bytes()[:100])  # truncated file
    info = ck.CheckpointManager(tmp_path, "checkpoints").load(*_bits())
    assert info["_loaded_from"] == ck.BEST_NAME
    assert (mgr.dir / (ck.LAST_NAME + ".corrupt")).exists()
    assert ck.CheckpointManager(tmp_path / "empty", "checkpoints").load(*_bits()) is None


def test_failed_write_raises_and_leaves_no_partial_file(tmp_path, monkeypatch):
    model, opt, sched = _bits()
    mgr = ck.CheckpointManager(tmp_path, "checkpoints")

    def half_write(obj, f, *a, **k):
        f.write(b"half")
        raise OSError("disk full")

    monkeypatch.setattr(ck.torch, "save", half_write)
    with pytest.raises(ck.CheckpointSaveError, match="disk full"):
        mgr.save(1, 0.5, model, opt, sched)
    assert not mgr.last_path.exists() and not list(mgr.dir.glob(f"*{ck.TMP_MARK}*"))


def test_async_save_reports_at_finalize(tmp_path):
    model, opt, sched = _bits()
    mgr = ck.CheckpointManager(tmp_path, "checkpoints", async_save=True)
    mgr.save(1, 0.5, model, opt, sched)
    mgr.finalize_saves()
    assert mgr.last_path.exists()
    mgr.close()


def test_snapshot_restore_puts_everything_back():
    model, opt, sched = _bits()
    snap = ck.CheckpointManager.snapshot(model, opt, sched)
    before = [p.detach().clone() for p in model.parameters()]
    r0 = torch.rand(1)
    ck.restore_rng(snap["rng"])
    for _ in range(2):
        opt.zero_grad()
        model(torch.randn(1, 3, 8, 8, 8)).sum().backward()
        opt.step()
        sched.step()
    ck.CheckpointManager.restore(snap, model, opt, sched)
    for a, b in zip(before, model.parameters()):
        assert torch.equal(a, b)
    assert torch.equal(torch.rand(1), r0) and sched.last_epoch == 0


def test_failed_write_does_not_move_the_best_mark(tmp_path, monkeypatch):
    model, opt, sched = _bits()
    mgr = ck.CheckpointManager(tmp_path, "checkpoints")
    assert mgr.save(1, 0.8, model, opt, sched) is True
    real_save = ck.torch.save

    def failing(obj, f, *a, **k):
        raise OSError("quota exceeded")

    monkeypatch.setattr(ck.torch, "save", failing)
    with pytest.raises(ck.CheckpointSaveError):
        mgr.save(2, 0.3, model, opt, sched)  # would have been the new best
    assert mgr.best_val_loss == 0.8
    monkeypatch.setattr(ck.torch, "save", real_save)
    assert mgr.save(3, 0.5, model, opt, sched) is True  # 0.5 beats the 0.8 that is really on disk
    assert torch.load(mgr.best_path, weights_only=False)["epoch"] == 3


def test_failed_async_write_rolls_the_best_mark_back(tmp_path, monkeypatch):
    model, opt, sched = _bits()
    mgr = ck.CheckpointManager(tmp_path, "checkpoints", async_save=True)
    assert mgr.save(1, 0.8, model, opt, sched) is True
    mgr.finalize_saves()

    def failing(obj, f, *a, **k):
        raise OSError("writer died")

    monkeypatch.setattr(ck.torch, "save", failing)
    assert mgr.save(2, 0.3, model, opt, sched) is True  # handed to the writer; the failure surfaces later
    with pytest.raises(ck.CheckpointSaveError, match="writer died"):
        mgr.finalize_saves()
    assert mgr.best_val_loss == 0.8
    mgr.close()


def test_ce_weight_indices_follow_the_linspace_rule():
    from scaffold_b200.train.trainer import sample_ce_weight_indices as pick
    assert pick(100, 0.1) == [0, 11, 22, 33, 44, 55, 66, 77, 88, 99]
    assert pick(10, 1.0) == list(range(10))
    assert pick(10, 0.95) == list(range(10))  # the fraction rounds up to the whole split
    assert pick(7, 0.01) == [0]
    assert pick(0, 0.1) == []
    assert pick(50, None) == [0, 12, 24, 36, 49]
