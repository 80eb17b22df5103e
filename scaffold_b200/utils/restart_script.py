"""Generates ``<run_dir>/restart.sh``, which resumes the run it sits in.

The command line of the original launch is rewritten so that it replays the
dumped ``config.yaml`` in place: every ``-c/--config`` is replaced by
``-c $RUN_DIR/config.yaml``, ``--base-run-dir`` and ``--job-name`` are dropped,
and ``--restart --run-dir $RUN_DIR`` is appended. The script re-activates the
virtual environment, re-exports the profiling switches that were set, and uses
the launch shape of the original job (``torchrun`` with the same rank count, or a
plain single-process call). (ScaFFold/utils/create_restart_script.py:49-378.)
"""
from __future__ import annotations

import os
import shlex
import stat
import sys
from pathlib import Path
from typing import List

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


def launch_prefix() -> str:
    world = int(os.environ.get("WORLD_SIZE", "1") or 1)
    if world > 1:
        local = int(os.environ.get("LOCAL_WORLD_SIZE", world) or world)
        nodes = max(1, world // max(local, 1))
        return (f"python -m torch.distributed.run --nnodes={nodes} --nproc-per-node={local} "
                f"--master-addr ${{MASTER_ADDR:-127.0.0.1}} --master-port ${{MASTER_PORT:-29500}} -m scaffold_b200.cli")
    return "python -m scaffold_b200.cli"


def render(run_dir: Path, argv: List[str]) -> str:
    args = " ".join(a if a.startswith("$RUN_DIR") else shlex.quote(a) for a in rewrite_argv(argv))
    lines = ["#!/bin/bash", "# Resumes the benchmark run stored in this directory.", "set -euo pipefail",
             'RUN_DIR="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"']
    venv = os.environ.get("VIRTUAL_ENV")
    if venv:
        lines.append(f"source {shlex.quote(venv)}/bin/activate")
    for var in _KEEP_ENV:
        if os.environ.get(var):
            lines.append(f"export {var}={shlex.quote(os.environ[var])}")
    lines.append(f"cd {shlex.quote(os.getcwd())}")
    lines.append(f"{launch_prefix()} {args}")
    return "\n".join(lines) + "\n"


def create_restart_script(run_dir, argv: List[str]) -> Path:
    path = Path(run_dir) / "restart.sh"
    path.write_text(render(Path(run_dir), list(argv)))
    path.chmod(path.stat().st_mode | stat.S_IXUSR | stat.S_IXGRP | stat.S_IXOTH)
    return path
