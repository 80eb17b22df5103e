"""Command line: ``scaffold generate_fractals`` and ``scaffold benchmark``.

Same surface as the reference CLI (ScaFFold/cli.py:1-684): repeated ``-c``
(first file = full config, later files = partial overrides), precedence
*built-in default < config file(s) < explicit flag*, run-directory rules (fresh
timestamped directory; ``--run-dir`` resumes in that directory; ``--restart``
without a directory is an error raised before anything is created), derived
keys (``unet_layers``, ``vol_size``, ``point_num``), and the run-directory
artefacts ``overrides.yaml``, ``config.yaml`` and ``restart.sh``. Decisions are
taken on rank 0 and broadcast; an error on rank 0 is re-raised on every rank.
"""
from __future__ import annotations

import argparse
import sys
from datetime import datetime
from pathlib import Path
from typing import Any, Dict, List, Optional, Set

import yaml

from . import config as C
from .utils import dist as D

BENCHMARK_FLAGS = {
    # flag -> (config key, type)
    "--base-run-dir": ("base_run_dir", str), "--fract-base-dir": ("fract_base_dir", str),
    "--dataset-dir": ("dataset_dir", str),
    "--n-categories": ("n_categories", int), "--n-instances-used-per-fractal": ("n_instances_used_per_fractal", int),
    "--problem-scale": ("problem_scale", int), "--unet-bottleneck-dim": ("unet_bottleneck_dim", int),
    "--dataset-seed": ("dataset_seed", int), "--training-seed": ("training_seed", int),
    "--local-batch-size": ("local_batch_size", int), "--warmup-batches": ("warmup_batches", int),
    "--group-norm-groups": ("group_norm_groups", int), "--dataloader-num-workers": ("dataloader_num_workers", int),
    "--optimizer": ("optimizer", str), "--epochs": ("epochs", int),
    "--starting-learning-rate": ("starting_learning_rate", float), "--min-learning-rate": ("min_learning_rate", float),
    "--T-0": ("T_0", int), "--T-mult": ("T_mult", int), "--job-name": ("job_name", str),
    "--target-dice": ("target_dice", float), "--checkpoint-interval": ("checkpoint_interval", int),
    "--unet-base-width": ("unet_base_width", int), "--gn-stats": ("gn_stats", str),
    "--grad-allreduce": ("grad_allreduce", str), "--halo-exchange": ("halo_exchange", str),
    "--grad-overlap": ("grad_overlap", int), "--allow-fallback": ("allow_fallback", int),
    "--val-cache-gb": ("val_cache_gb", float),
}
GENERATE_FLAGS = {
    "--datagen-batch-size": ("datagen_batch_size", int), "--problem-scale": ("problem_scale", int),
    "--n-categories": ("n_categories", int), "--fract-base-dir": ("fract_base_dir", str),
    "--dataset-seed": ("dataset_seed", int),
}


def build_parser() -> argparse.ArgumentParser:
    parser = argparse.ArgumentParser(prog="scaffold", description="Scale-free fractal 3D U-Net benchmark (B200)")
    sub = parser.add_subparsers(dest="command", required=True)
    default_cfg = str(C.default_config_path())

    gen = sub.add_parser("generate_fractals", help="search IFS categories and generate fractal instances")
    gen.add_argument("-c", "--config", action="append", help="config file; repeat to add partial override files")
    gen.add_argument("-v", "--verbose", action="store_true")
    for flag, (key, typ) in GENERATE_FLAGS.items():
        gen.add_argument(flag, dest=key, type=typ, default=None)

    ben = sub.add_parser("benchmark", help="train the U-Net to the target Dice and report the figure of merit")
    ben.add_argument("-c", "--config", action="append", help="config file; repeat to add partial override files")
    ben.add_argument("-v", "--verbose", action="store_true")
    for flag, (key, typ) in BENCHMARK_FLAGS.items():
        ben.add_argument(flag, dest=key, type=typ, default=None)
    ben.add_argument("--restart", action="store_true", default=None, help="resume the run named by --run-dir")
    ben.add_argument("--run-dir", dest="run_dir", type=str, default=None, help="existing run directory to resume")
    ben.add_argument("--dc-num-shards", dest="dc_num_shards", type=int, nargs="+", default=None)
    ben.add_argument("--dc-shard-dims", dest="dc_shard_dims", type=int, nargs="+", default=None)
    for p in (gen, ben):
        p.set_defaults(_default_config=default_cfg)
    return parser


def explicit_cli_keys(args: argparse.Namespace) -> Set[str]:
    """Keys the user actually typed (every option defaults to None, so non-None means explicit)."""
    skip = {"command", "config", "_default_config"}
    return {k for k, v in vars(args).items() if k not in skip and v is not None and v is not False}


def _make_fresh_run_dir(base: Path, name: str) -> Path:
    base.mkdir(parents=True, exist_ok=True)
    for k in range(1000):
        cand = base / (name if k == 0 else f"{name}-{k}")
        try:
            cand.mkdir(parents=False, exist_ok=False)
            return cand
        except FileExistsError:
            continue
    raise RuntimeError(f"could not create a unique run directory under {base}")


def resolve_run_dir(merged: Dict[str, Any]) -> Path:
    """Fresh directory, or resume in ``run_dir``; ``restart`` without a directory is rejected first."""
    restart = bool(merged.get("restart"))
    run_dir = merged.get("run_dir")
    if run_dir is not None:
        path = Path(run_dir)
        path.mkdir(parents=True, exist_ok=True)
        resuming = True
    elif restart:
        raise ValueError(
            "A restart was requested (--restart, or restart: true in the config file) but no run directory was "
            "given: pass the directory of the run to resume (e.g. '--restart --run-dir <path>'). The most recent "
            "run directory is not resolved automatically.")
    else:
        stamp = datetime.now().strftime(f"{merged.get('job_name', 'benchmark')}_%Y%m%d-%H%M%S")
        path = _make_fresh_run_dir(Path(merged["base_run_dir"]), stamp)
        resuming = False
    merged["benchmark_run_dir"] = str(path)
    merged["restart"] = resuming
    merged["run_dir"] = str(path)
    if resuming:
        merged["train_from_scratch"] = False
    return path


def missing_checkpoint_error(merged: Dict[str, Any]) -> Optional[str]:
    """A resume needs ``checkpoint_last.pth`` or ``checkpoint_best.pth`` in the run directory."""
    if not merged.get("restart"):
        return None
    ckpt = Path(merged["run_dir"]) / merged.get("checkpoint_dir", "checkpoints")
    if any((ckpt / n).exists() for n in ("checkpoint_last.pth", "checkpoint_best.pth")):
        return None
    return (f"Restart requested but no checkpoint was found in {ckpt} (looked for checkpoint_last.pth and "
            "checkpoint_best.pth). Start a fresh run, or point --run-dir at a run that saved checkpoints "
            "(checkpoint_interval > 0).")


def build_run_config(args: argparse.Namespace, argv: List[str]) -> Dict[str, Any]:
    """Rank 0: merge files and flags, derive keys, resolve the run directory, write its artefacts."""
    files = args.config or [args._default_config]
    merged = C.load_config_files(files)
    explicit = explicit_cli_keys(args)
    overrides = {k: getattr(args, k) for k in sorted(explicit)}
    merged.update(overrides)
    merged["command"] = args.command
    merged["config"] = [str(f) for f in files]
    merged["verbose"] = bool(args.verbose)
    if args.command != "benchmark":
        merged.setdefault("base_run_dir", ".")
    cfg = C.Config(merged)  # validates; raises on a bad value before any directory is created
    if args.command == "benchmark":
        path = resolve_run_dir(merged)
        resuming = bool(merged["restart"])
    merged["unet_layers"] = cfg.unet_layers
    merged["vol_size"] = cfg.vol_size
    merged["point_num"] = cfg.point_num
    if args.command != "benchmark":
        return merged
    from .utils.restart_script import create_restart_script
    from .utils.scheduler_info import collect_scheduler_info
    merged["scheduler_metadata"] = collect_scheduler_info()
    dump = {k: v for k, v in merged.items() if not k.startswith("_")}
    if not resuming:
        dump["run_dir"] = None
    with open(path / "overrides.yaml", "w") as f:
        yaml.safe_dump(overrides, f, sort_keys=True)
    with open(path / "config.yaml", "w") as f:
        yaml.safe_dump(dump, f, sort_keys=True)
    create_restart_script(path, argv)
    merged.setdefault("run_iter", 0)
    return merged


def main(argv: Optional[List[str]] = None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    args = build_parser().parse_args(argv)
    D.initialize_dist()
    D.check_launcher_world_size()
    merged = D.run_on_root(lambda: build_run_config(args, argv))
    if args.command == "benchmark":
        err = D.run_on_root(lambda: missing_checkpoint_error(merged))
        if err:
            raise FileNotFoundError(err)
        from .run import benchmark
        benchmark(merged)
    else:
        from .run import generate_fractals
        generate_fractals(merged)
    D.barrier()
    import torch.distributed as dist
    if dist.is_initialized():
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
