"""Scheduler metadata recorded in ``config.yaml`` (ScaFFold/utils/collect_scheduler_info.py:18-73)."""
from __future__ import annotations

import os
import socket
from typing import Any, Dict


def collect_scheduler_info() -> Dict[str, Any]:
    env = os.environ
    info: Dict[str, Any] = {"hostname": socket.gethostname(), "scheduler": "none"}
    if env.get("FLUX_JOB_ID") or env.get("FLUX_URI"):
        info.update(scheduler="flux", job_id=env.get("FLUX_JOB_ID"), nodes=env.get("FLUX_JOB_NNODES"),
                    tasks=env.get("FLUX_JOB_SIZE"))
    elif env.get("SLURM_JOB_ID"):
        info.update(scheduler="slurm", job_id=env.get("SLURM_JOB_ID"), nodes=env.get("SLURM_JOB_NUM_NODES"),
                    tasks=env.get("SLURM_NTASKS"), nodelist=env.get("SLURM_JOB_NODELIST"))
    info["world_size"] = env.get("WORLD_SIZE")
    for var in ("CUDA_VISIBLE_DEVICES", "NVIDIA_VISIBLE_DEVICES"):
        if env.get(var) is not None:
            info[var.lower()] = env[var]
    return {k: v for k, v in info.items() if v is not None}
