"""Reporting and instrumentation helpers: figures from train_stats.csv, scheduler metadata, the perf shim, the rank
filter of the logger (roles of ScaFFold/viz/standard_viz.py, utils/collect_scheduler_info.py, utils/perf_measure.py)."""
import io
import logging

import pytest

from scaffold_b200.utils import figures, perf, scheduler_info
from scaffold_b200.utils.log import RankFilter, mem_stats, setup_logger

CSV = ("epoch,epoch_loss,overall_loss,val_loss_epoch,val_loss_avg,train_dice,val_dice,epoch_duration,optimizer_steps,"
       "total_optimizer_steps\n1,10.0,1.5,3.0,1.2,0.1,0.30,3.4,168,168\n2,8.0,0.9,2.0,0.8,0.4,0.65,3.1,168,336\n")


def test_figures_are_written_headless_with_stable_names(tmp_path):
    (tmp_path / "train_stats.csv").write_text(CSV)
    cols = figures.read_stats(tmp_path)
    assert cols["epoch"] == [1.0, 2.0] and cols["val_dice"] == [0.30, 0.65]
    written = figures.standard_figures(tmp_path)
    assert sorted(p.stem for p in written) == ["train_loss", "val_dice", "val_loss"]
    assert all(p.parent.name == "figures" and p.exists() and p.stat().st_size > 0 for p in written)
    assert len({p.suffix for p in written}) == 1 and written[0].suffix in (".png", ".csv")
    again = figures.standard_figures(tmp_path)  # a second call overwrites in place
    assert [p.name for p in again] == [p.name for p in written]


def test_figures_fall_back_to_csv_series_without_matplotlib(tmp_path, monkeypatch):
    import builtins
    real = builtins.__import__

    def no_mpl(name, *a, **k):
        if name.startswith("matplotlib"):
            raise ImportError("no matplotlib here")
        return real(name, *a, **k)

    monkeypatch.setattr(builtins, "__import__", no_mpl)
    (tmp_path / "train_stats.csv").write_text(CSV)
    written = figures.standard_figures(tmp_path)
    assert [p.suffix for p in written] == [".csv"] * 3
    assert (tmp_path / "figures" / "val_dice.csv").read_text().splitlines() == ["epoch,val_dice", "1,0.3", "2,0.65"]


def test_scheduler_info_reads_the_allocation_it_runs_in(monkeypatch):
    for var in ("FLUX_JOB_ID", "FLUX_URI", "SLURM_JOB_ID", "WORLD_SIZE", "CUDA_VISIBLE_DEVICES", "NVIDIA_VISIBLE_DEVICES"):
        monkeypatch.delenv(var, raising=False)
    info = scheduler_info.collect_scheduler_info()
    assert info["scheduler"] == "none" and "hostname" in info and "job_id" not in info and "world_size" not in info
    monkeypatch.setenv("SLURM_JOB_ID", "4711")
    monkeypatch.setenv("SLURM_JOB_NUM_NODES", "2")
    monkeypatch.setenv("SLURM_NTASKS", "16")
    monkeypatch.setenv("WORLD_SIZE", "16")
    monkeypatch.setenv("CUDA_VISIBLE_DEVICES", "0,1")
    info = scheduler_info.collect_scheduler_info()
    assert (info["scheduler"], info["job_id"], info["nodes"], info["tasks"]) == ("slurm", "4711", "2", "16")
    assert info["world_size"] == "16" and info["cuda_visible_devices"] == "0,1"
    monkeypatch.setenv("FLUX_JOB_ID", "f123")           # a Flux allocation wins over a Slurm one
    monkeypatch.setenv("FLUX_JOB_NNODES", "4")
    assert scheduler_info.collect_scheduler_info()["scheduler"] == "flux"


def test_perf_regions_accumulate_and_metadata_round_trips(monkeypatch):
    monkeypatch.delenv("SCAFFOLD_NVTX", raising=False)
    monkeypatch.delenv("CALI_CONFIG", raising=False)
    before = perf.region_totals().get("unit_test_region", {"count": 0, "seconds": 0.0})
    with perf.region("unit_test_region"):
        with perf.region("unit_test_region"):            # nesting the same name is allowed
            pass
    after = perf.region_totals()["unit_test_region"]
    assert after["count"] == before["count"] + 2 and after["seconds"] >= before["seconds"]
    perf.end_code_region("never_opened")                 # an unmatched end is ignored, not an error
    assert "never_opened" not in perf.region_totals()
    perf.adiak_init()
    perf.adiak_value("ddp_ranks", 4)
    assert perf.metadata() == {"ddp_ranks": 4}

    @perf.annotate(fmt="fn:{}")
    def f(x):
        return x + 1
    assert f(1) == 2 and f.__name__ == "f"               # free when tracing is off, name kept


def test_profiler_is_off_by_default_bounded_when_on_and_one_rank_per_node(monkeypatch):
    monkeypatch.delenv("PROFILE_TORCH", raising=False)
    with perf.get_torch_context(0, 4) as prof:
        assert prof is None
    monkeypatch.setenv("PROFILE_TORCH", "1")
    monkeypatch.setenv("PROFILE_TORCH_ACTIVE", "0")      # clamped to the minimum
    monkeypatch.setenv("PROFILE_TORCH_WAIT", "junk")     # unreadable: default
    assert perf.profiler_schedule_args() == {"wait": 1, "warmup": 1, "active": 1, "repeat": 1}
    with perf.get_torch_context(1, 4) as prof:           # not the first rank of its node
        assert prof is None


def test_rank_filter_silences_info_off_the_root_and_stamps_the_rank():
    rec = logging.LogRecord("x", logging.INFO, __file__, 1, "m", None, None)
    assert RankFilter(0).filter(rec) and rec.rank == 0
    assert not RankFilter(3).filter(rec) and rec.rank == 3
    warn = logging.LogRecord("x", logging.WARNING, __file__, 1, "m", None, None)
    assert RankFilter(3).filter(warn)
    assert RankFilter(3, root_only=False).filter(rec)
    log = setup_logger("scaffold_test_logger", rank=2)
    stream = io.StringIO()
    log.handlers[0].setStream(stream)
    log.info("quiet")
    log.warning("loud")
    out = stream.getvalue()
    assert "quiet" not in out and "loud" in out and "[rank=2]" in out
    assert isinstance(mem_stats("cpu"), dict)
