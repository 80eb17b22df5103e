"""Tracing and profiling shim.

Same switches and region names as the reference's Caliper/Adiak/torch.profiler
shim (ScaFFold/utils/perf_measure.py:19-168), mapped to what a B200 box has:

* code regions and function annotations become NVTX ranges (visible to any
  CUDA profiler) when ``SCAFFOLD_NVTX=1`` or ``CALI_CONFIG`` is set, and are
  always accumulated as host wall-clock totals available through
  ``region_totals()``;
* ``adiak_value`` key/values are collected into a metadata dict that the worker
  writes next to the run's config;
* ``PROFILE_TORCH`` (1/true/on/yes) enables a bounded ``torch.profiler``
  schedule on one rank per node, tunable with ``PROFILE_TORCH_WAIT`` /
  ``_WARMUP`` / ``_ACTIVE`` / ``_RECORD_SHAPES`` / ``_WITH_STACK``.
"""
from __future__ import annotations

import functools
import os
import time
from collections import defaultdict
from contextlib import contextmanager, nullcontext
from typing import Any, Dict

_TRUE = {"1", "true", "on", "yes"}
_metadata: Dict[str, Any] = {}
_totals: Dict[str, float] = defaultdict(float)
_counts: Dict[str, int] = defaultdict(int)
_open: Dict[str, list] = defaultdict(list)


def _nvtx_enabled() -> bool:
    return os.environ.get("SCAFFOLD_NVTX", "0").lower() in _TRUE or bool(os.environ.get("CALI_CONFIG"))


def _nvtx():
    if not _nvtx_enabled():
        return None
    try:
        import torch
        if torch.cuda.is_available():
            return torch.cuda.nvtx
    except Exception:
        pass
    return None


def begin_code_region(name: str) -> None:
    nv = _nvtx()
    if nv is not None:
        nv.range_push(name)
    _open[name].append(time.perf_counter())


def end_code_region(name: str) -> None:
    if _open[name]:
        _totals[name] += time.perf_counter() - _open[name].pop()
        _counts[name] += 1
    nv = _nvtx()
    if nv is not None:
        nv.range_pop()


@contextmanager
def region(name: str):
    begin_code_region(name)
    try:
        yield
    finally:
        end_code_region(name)


def annotate(name: str = None, fmt: str = None):
    """Decorator: wraps the call in an NVTX range when tracing is on; free otherwise."""
    def deco(fn):
        label = name or (fmt.format(fn.__name__) if fmt else fn.__qualname__)

        @functools.wraps(fn)
        def wrapper(*a, **k):
            nv = _nvtx()
            if nv is None:
                return fn(*a, **k)
            nv.range_push(label)
            try:
                return fn(*a, **k)
            finally:
                nv.range_pop()
        return wrapper
    return deco


def region_totals() -> Dict[str, Dict[str, float]]:
    return {k: {"seconds": v, "count": _counts[k]} for k, v in _totals.items()}


def adiak_init(*_a, **_k) -> None:
    _metadata.clear()


def adiak_value(key: str, value: Any) -> None:
    _metadata[key] = value


def metadata() -> Dict[str, Any]:
    return dict(_metadata)


def profile_torch_enabled() -> bool:
    return os.environ.get("PROFILE_TORCH", "").strip().lower() in _TRUE


def _env_int(name: str, default: int, minimum: int) -> int:
    try:
        return max(minimum, int(os.environ.get(name, default)))
    except ValueError:
        return default


def profiler_schedule_args() -> Dict[str, int]:
    """Bounded schedule: the trace never grows with the length of the run."""
    return dict(wait=_env_int("PROFILE_TORCH_WAIT", 1, 1), warmup=_env_int("PROFILE_TORCH_WARMUP", 1, 0),
                active=_env_int("PROFILE_TORCH_ACTIVE", 3, 1), repeat=1)


def get_torch_context(rank: int = 0, ranks_per_node: int = 1):
    """A ``torch.profiler.profile`` for one rank per node when ``PROFILE_TORCH`` is on, else a null context."""
    if not profile_torch_enabled() or rank % max(1, ranks_per_node) != 0:
        return nullcontext(None)
    import torch
    from torch.profiler import ProfilerActivity, profile, schedule
    acts = [ProfilerActivity.CPU]
    if torch.cuda.is_available():
        acts.append(ProfilerActivity.CUDA)
    return profile(activities=acts, schedule=schedule(**profiler_schedule_args()),
                   record_shapes=os.environ.get("PROFILE_TORCH_RECORD_SHAPES", "0").lower() in _TRUE,
                   with_stack=os.environ.get("PROFILE_TORCH_WITH_STACK", "0").lower() in _TRUE)
