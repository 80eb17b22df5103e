"""Generates ``<run_dir>/restart.sh``, which resumes the run it sits in.

The command line of the original launch is rewritten so that it replays the
dumped ``config.yaml`` in place: every ``-c/--config`` is replaced by
``-c $RUN_DIR/config.yaml``, ``--base-run-dir`` and ``--job-name`` are dropped,
and ``--restart --run-dir $RUN_DIR`` is appended. The script re-activates the
virtual environment, re-exports the profiling switches that were set, and uses
the launch shape of the original job: the node and rank counts are read from the
Flux or Slurm allocation (``flux run`` / ``srun`` templates), else from the
launcher's rank variables (``torchrun`` template), else the script is a plain
single-process call. (ScaFFold/utils/create_restart_script.py:49-378.)
"""
from __future__ import annotations

import os
import shlex
import stat
import sys
from pathlib import Path
from typing import Dict, List

_DROP_WITH_VALUE = {"--base-run-dir", "--job-name", "-c", "--config", "--run-dir"}
_DROP_FLAG = {"--restart"}
_KEEP_ENV = ("PROFILE_TORCH", "PROFILE_TORCH_WAIT", "PROFILE_TORCH_WARMUP", "PROFILE_TORCH_ACTIVE", "CALI_CONFIG",
             "SCAFFOLD_NVTX")


def rewrite_argv(argv: List[str]) -> List[str]:
    out, i = [], 0
    while i < len(argv):
        a = argv[i]
        if a in _DROP_FLAG:
            i += 1
        elif a in _DROP_WITH_VALUE:
            i += 2
        elif any(a.startswith(f + "=") for f in _DROP_WITH_VALUE if f.startswith("--")):
            i += 1
        else:
            out.append(a)
            i += 1
    # the subcommand stays first; the replayed config and the resume flags follow it
    head, tail = (out[:1], out[1:]) if out else ([], [])
    return head + ["-c", "$RUN_DIR/config.yaml"] + tail + ["--restart", "--run-dir", "$RUN_DIR"]


_WORLD_VARS = ("WORLD_SIZE", "OMPI_COMM_WORLD_SIZE", "MV2_COMM_WORLD_SIZE", "PMI_SIZE", "PALS_NRANKS", "SLURM_NTASKS",
               "FLUX_JOB_SIZE")


def launch_shape(env=None, world_size: int = None) -> Dict[str, object]:
    """How the generating job was launched: ``{"scheduler", "nodes", "ranks", "per_node"}``.

    A known rank count (``world_size``, e.g. from the process group) wins over the environment. The
    scheduler is ``"flux"`` or ``"slurm"`` when the job runs inside one of their allocations, else
    ``"torchrun"`` for a multi-rank launch and ``"local"`` for a single process
    (role of ScaFFold/utils/create_restart_script.py:186-291).
    """
    env = os.environ if env is None else env

    def num(*names, default=None):
        for n in names:
            v = env.get(n)
            if v:
                try:
                    return int(str(v).split("(")[0].split(",")[0])  # Slurm writes e.g. "4(x2)"
                except ValueError:
                    continue
        return default

    if env.get("FLUX_JOB_ID"):
        sched, nodes, ranks = "flux", num("FLUX_JOB_NNODES", default=1), num("FLUX_JOB_SIZE", default=1)
    elif env.get("SLURM_JOB_ID") or env.get("SLURM_JOBID"):
        sched = "slurm"
        nodes = num("SLURM_JOB_NUM_NODES", "SLURM_NNODES", default=1)
        ranks = num("SLURM_NTASKS", "SLURM_NPROCS", default=1)
    else:
        ranks = num(*_WORLD_VARS, default=1)
        local = num("LOCAL_WORLD_SIZE", default=ranks)
        nodes = max(1, ranks // max(local, 1))
        sched = "torchrun" if ranks > 1 else "local"
    if world_size:
        ranks = int(world_size)
        if sched == "local" and ranks > 1:
            sched = "torchrun"
    nodes = max(1, int(nodes or 1))
    return {"scheduler": sched, "nodes": nodes, "ranks": int(ranks), "per_node": max(1, int(ranks) // nodes)}


def launch_lines(shape: Dict[str, object], args: str) -> List[str]:
    """The command that relaunches the CLI with the captured shape, one template per launcher."""
    cli = "python -m scaffold_b200.cli"
    nodes, ranks, per_node = shape["nodes"], shape["ranks"], shape["per_node"]
    rendezvous = "--master-addr ${MASTER_ADDR:-127.0.0.1} --master-port ${MASTER_PORT:-29500}"
    if shape["scheduler"] == "local":
        return [f"exec {cli} {args}"]
    if shape["scheduler"] == "torchrun":
        return [f"NODES={nodes}", f"RANKS_PER_NODE={per_node}",
                f'exec python -m torch.distributed.run --nnodes="$NODES" --nproc-per-node="$RANKS_PER_NODE" '
                f"{rendezvous} -m scaffold_b200.cli {args}"]
    if shape["scheduler"] == "slurm":
        # one task per GPU; the CLI reads rank and size from the SLURM_* variables
        return [f"NODES={nodes}", f"RANKS={ranks}", f"RANKS_PER_NODE={per_node}",
                'export MASTER_ADDR="${MASTER_ADDR:-$(scontrol show hostnames "$SLURM_JOB_NODELIST" | head -n 1)}"',
                'export MASTER_PORT="${MASTER_PORT:-29500}"',
                f'exec srun -N "$NODES" -n "$RANKS" --ntasks-per-node="$RANKS_PER_NODE" --gpus-per-task=1 {cli} {args}']
    return [f"NODES={nodes}", f"RANKS={ranks}", f"RANKS_PER_NODE={per_node}",
            'export MASTER_ADDR="${MASTER_ADDR:-$(flux hostlist -n 0 local 2>/dev/null || hostname)}"',
            'export MASTER_PORT="${MASTER_PORT:-29500}"',
            f'exec flux run -N "$NODES" -n "$RANKS" --gpus-per-task=1 {cli} {args}']


def render(run_dir: Path, argv: List[str], world_size: int = None, env=None) -> str:
    env = os.environ if env is None else env
    args = " ".join(a if a.startswith("$RUN_DIR") else shlex.quote(a) for a in rewrite_argv(argv))
    shape = launch_shape(env, world_size)
    lines = ["#!/bin/bash", "# Resumes the benchmark run stored in this directory "
             f"({shape['scheduler']} launch, {shape['ranks']} rank(s) on {shape['nodes']} node(s)).",
             "set -euo pipefail", 'RUN_DIR="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"']
    venv = env.get("VIRTUAL_ENV")
    if venv:
        act = shlex.quote(f"{venv}/bin/activate")
        lines += [f"if [ -f {act} ]; then source {act}; else echo 'restart.sh: virtualenv {venv} is gone' >&2; fi"]
    for var in _KEEP_ENV:
        if env.get(var):
            lines.append(f"export {var}={shlex.quote(env[var])}")
    lines.append(f"cd {shlex.quote(os.getcwd())}")
    lines += launch_lines(shape, args)
    return "\n".join(lines) + "\n"


def create_restart_script(run_dir, argv: List[str], world_size: int = None) -> Path:
    path = Path(run_dir) / "restart.sh"
    path.write_text(render(Path(run_dir), list(argv), world_size))
    path.chmod(path.stat().st_mode | stat.S_IXUSR | stat.S_IXGRP | stat.S_IXOTH)
    return path
