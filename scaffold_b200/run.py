"""Drivers: ``benchmark`` (train to the target Dice) and ``generate_fractals``.

Mirrors ScaFFold/benchmark.py:27-74, ScaFFold/worker.py:143-397 and
ScaFFold/generate_fractals.py:23-45 with ``torch.distributed`` as the only
transport: rank 0 prepares the run dictionary and broadcasts it; the worker
seeds, brings up the process group (device bound first), checks the world size
against the shard layout, finds or generates the dataset, builds the model in
channels-last, sets up the parallel layout, trains under the optional profiler
and reports the figure of merit ``FOM = 1 / sum(epoch_duration)`` together with
the training throughput in voxels per second.
"""
from __future__ import annotations

import csv
import math
import os
import shutil
import socket
import time
from pathlib import Path
from typing import Any, Dict

import torch
import yaml

from .config import RunConfig
from .data import cache, category_search, instances
from .models.unet import UNet
from .parallel.layout import ParallelLayout
from .parallel.spatial import SpatialContext
from .train.trainer import Trainer
from .utils import dist as D
from .utils import perf
from .utils.log import set_seeds, setup_logger


def attach_spatial(model, spatial) -> None:
    """Hand the spatial context to every module that communicates across shards."""
    for m in model.modules():
        if hasattr(m, "set_spatial"):
            m.set_spatial(spatial)


def trace_file_name(config, rank: int, world: int, nodes: int) -> str:
    ts = time.strftime("%Y%m%d-%H%M%S")
    return (f"torch-{socket.gethostname()}-r{rank}-N{nodes}-n{world}-ps{config.problem_scale}-e{config.epochs}-"
            f"nipf{config.n_instances_used_per_fractal}-{ts}.json")


def figure_of_merit(stats_csv: Path, target_dice: float) -> Dict[str, Any]:
    """FOM = 1 / total training time; time-to-Dice = seconds until ``val_dice >= target_dice`` (None if never)."""
    total, reached, epochs = 0.0, None, 0
    with open(stats_csv) as f:
        for row in csv.DictReader(f):
            total += float(row["epoch_duration"])
            epochs += 1
            if reached is None and float(row["val_dice"]) >= target_dice:
                reached = total
    return {"FOM": (1.0 / total) if total > 0 else 0.0, "total_train_time_s": total, "time_to_dice_s": reached,
            "epochs": epochs}


def worker(run_dict: Dict[str, Any]) -> Dict[str, Any]:
    config = RunConfig(run_dict)
    set_seeds(config.dataset_seed)
    with perf.region("init_ddp"):
        device = D.initialize_dist()
    log = setup_logger("scaffold", verbose=bool(run_dict.get("verbose", False)))
    rank, world = D.get_world_rank(), D.get_world_size()
    if device.type == "cuda":
        torch.backends.cudnn.benchmark = not config.more_determinism
    total_shards = math.prod(config.dc_num_shards)
    if world % total_shards != 0:
        raise ValueError(f"world size {world} is not divisible by prod(dc_num_shards)={total_shards} "
                         f"(dc_num_shards={config.dc_num_shards})")

    with perf.region("get_dataset"):
        config.dataset_dir = str(cache.get_dataset(config, bool(config.dataset_reuse_enforce_commit_id), log))

    set_seeds(config.training_seed)
    with perf.region("init_model"):
        model = UNet(int(getattr(config, "n_channels", 3)), config.n_categories + 1, trilinear=False,
                     layers=config.unet_layers, group_norm_groups=config.group_norm_groups,
                     base_width=int(getattr(config, "unet_base_width", 64)))
        model = model.to(device=device, memory_format=torch.channels_last_3d)
        if config.activation_checkpointing:
            model.use_checkpointing()
        layout = ParallelLayout(config.dc_num_shards, config.dc_shard_dims, world, rank)
        spatial = SpatialContext(layout, gn_stats=config.gn_stats, halo_backend=config.halo_exchange)
        attach_spatial(model, spatial if layout.spatial_size > 1 else None)
        if world > 1:  # replicas start identical
            for p in model.parameters():
                torch.distributed.broadcast(p.data, 0)
    perf.adiak_value("ddp_ranks", layout.ddp_ranks)
    perf.adiak_value("total_shards", layout.spatial_size)
    log.info("%s", layout)

    trainer = Trainer(model, config, device, log, layout=layout, spatial=spatial if layout.spatial_size > 1 else None)
    nodes = max(1, world // max(1, D.get_local_size()))
    prof_ctx = perf.get_torch_context(rank, D.get_local_size())
    with prof_ctx as prof:
        with perf.region("cleanup_or_resume"):
            trainer.cleanup_or_resume()
        with perf.region("warmup"):
            trainer.warmup()
        with perf.region("train"):
            summary = trainer.train(prof)
    if prof is not None:
        try:
            prof.export_chrome_trace(str(Path(config.run_dir) / trace_file_name(config, rank, world, nodes)))
        except Exception as exc:  # a failed export must not fail the run
            log.warning("could not export the profiler trace: %s", exc)
    D.barrier()

    result = dict(summary)
    result["dataset_path"] = str(config.dataset_dir)  # the resolved dataset (cache entry) this run trained on
    if rank == 0:
        fom = figure_of_merit(Path(config.run_dir) / "train_stats.csv", float(config.target_dice))
        result.update(fom)
        perf.adiak_value("FOM", fom["FOM"])
        log.info("FOM (1 / total train time): %.6g ; total train time %.3f s ; time to Dice %.2f: %s", fom["FOM"],
                 fom["total_train_time_s"], config.target_dice,
                 "not reached" if fom["time_to_dice_s"] is None else f"{fom['time_to_dice_s']:.3f} s")
        with open(Path(config.run_dir) / "run_metadata.yaml", "w") as f:
            yaml.safe_dump({"metadata": _plain(perf.metadata()), "regions": perf.region_totals(),
                            "result": _plain(result)}, f)
        with perf.region("generate_figures"):
            try:
                from .utils.figures import standard_figures
                standard_figures(config.run_dir)
            except Exception as exc:
                log.warning("figures were not generated: %s", exc)
    return result


def _plain(d: Dict[str, Any]) -> Dict[str, Any]:
    out = {}
    for k, v in d.items():
        out[str(k)] = v if isinstance(v, (int, float, str, bool, type(None), list, dict)) else str(v)
    return out


def benchmark(kwargs: Dict[str, Any]) -> Dict[str, Any]:
    """``scaffold benchmark``: kwargs is the merged configuration dictionary produced by the CLI."""
    D.initialize_dist()

    def prepare():
        run_dir = Path(kwargs["run_dir"])
        run_dir.mkdir(parents=True, exist_ok=True)
        cfgs = kwargs.get("config")
        base = cfgs[0] if isinstance(cfgs, (list, tuple)) and cfgs else cfgs
        if base and os.path.exists(base) and not (run_dir / "base_config.yaml").exists():
            shutil.copyfile(base, run_dir / "base_config.yaml")
        run_dict = dict(kwargs)
        run_dict.setdefault("run_iter", 0)
        return run_dict

    run_dict = D.run_on_root(prepare)
    perf.adiak_init()
    for k, v in run_dict.items():
        perf.adiak_value(k, v)
    return worker(run_dict)


def generate_fractals(kwargs: Dict[str, Any]) -> None:
    """``scaffold generate_fractals``: IFS category search, then instance generation."""
    from .config import Config
    D.initialize_dist()
    log = setup_logger("scaffold", verbose=bool(kwargs.get("verbose", False)))
    config = Config(kwargs)
    D.barrier()
    category_search.main(config, log)
    D.barrier()
    instances.main(config, log)
    D.barrier()
