"""Seeding, rank-filtered logging and memory reporting.

Format and filtering follow ScaFFold/utils/utils.py:43-176: records look like
``[HH:MM:SS][file:line][rank=r][LEVEL] msg`` on stderr, only rank 0 emits below
WARNING, ``-v`` selects DEBUG.
"""
from __future__ import annotations

import logging
import random
import sys
from typing import Optional

import numpy as np
import torch

from . import dist as D


def set_seeds(seed: int) -> None:
    random.seed(seed)
    np.random.seed(seed % (2**32))
    torch.manual_seed(seed)
    if torch.cuda.is_available():
        torch.cuda.manual_seed_all(seed)


class RankFilter(logging.Filter):
    """Stamps the rank on every record and silences non-root ranks below WARNING."""

    def __init__(self, rank: int, root_only: bool = True):
        super().__init__()
        self.rank, self.root_only = rank, root_only

    def filter(self, record: logging.LogRecord) -> bool:
        record.rank = self.rank
        return not self.root_only or self.rank == 0 or record.levelno >= logging.WARNING


def setup_logger(name: str = "scaffold", verbose: bool = False, rank: Optional[int] = None) -> logging.Logger:
    rank = D.get_world_rank() if rank is None else rank
    log = logging.getLogger(name)
    log.setLevel(logging.DEBUG if verbose else logging.INFO)
    log.propagate = False
    for h in list(log.handlers):
        log.removeHandler(h)
    handler = logging.StreamHandler(sys.stderr)
    handler.setFormatter(logging.Formatter("[%(asctime)s][%(filename)s:%(lineno)d][rank=%(rank)s][%(levelname)s] %(message)s",
                                           datefmt="%H:%M:%S"))
    handler.addFilter(RankFilter(rank))
    log.addHandler(handler)
    return log


def mem_stats(device: Optional[torch.device] = None) -> dict:
    out = {}
    try:
        import psutil
        out["host_rss_gb"] = psutil.Process().memory_info().rss / 2**30
    except Exception:
        pass
    if torch.cuda.is_available() and (device is None or torch.device(device).type == "cuda"):
        out["cuda_allocated_gb"] = torch.cuda.memory_allocated(device) / 2**30
        out["cuda_reserved_gb"] = torch.cuda.memory_reserved(device) / 2**30
        out["cuda_peak_gb"] = torch.cuda.max_memory_allocated(device) / 2**30
    return out


def gather_and_print_mem(log: logging.Logger, tag: str, device=None) -> None:
    """Collect every rank's memory numbers on rank 0 and log min/max (DEBUG)."""
    if not log.isEnabledFor(logging.DEBUG):
        return
    stats = D.allgather_obj(mem_stats(device))
    if D.get_world_rank() != 0:
        return
    keys = sorted({k for s in stats for k in s})
    parts = [f"{k}: min {min(s.get(k, 0.0) for s in stats):.2f} max {max(s.get(k, 0.0) for s in stats):.2f}" for k in keys]
    log.debug("[mem:%s] %s", tag, "; ".join(parts))
