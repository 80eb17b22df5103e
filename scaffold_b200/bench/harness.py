"""Timing primitives for kernel A/B comparisons.

A comparison of two implementations on a shared, clock-drifting GPU is only as good as its pairing:
``paired_ratio`` times the two callables in alternating batches (A B A B ...), so both see the same
clock and thermal state, takes the ratio per round and stops once the 95 % confidence interval of the
geometric-mean ratio is narrower than the target (3 % by default) or a round / time limit is hit.
Batch sizes are found online (``calibrate``): each timed batch lasts a few milliseconds so that event
resolution and launch jitter are negligible. Times come from CUDA events on the launching stream; SM
clocks are sampled through NVML during every batch so that a result can also be reported as
``time x MHz`` (cycles), which is comparable across runs that met different power-cap clocks.

Role of the reference: triton_conv3d/bench/harness.py:859-1023 (interleaved pairs, online sizing, CI).
"""
from __future__ import annotations

import math
import statistics
import time
from dataclasses import dataclass, field
from typing import Callable, List, Optional

import torch

Fn = Callable[[int], object]  # called with a running call index (lets the case rotate its operands past L2)

# two-sided 95 % Student-t quantiles for n-1 degrees of freedom (n = 2 .. 30), then the normal value
_T95 = [12.706, 4.303, 3.182, 2.776, 2.571, 2.447, 2.365, 2.306, 2.262, 2.228, 2.201, 2.179, 2.160, 2.145, 2.131,
        2.120, 2.110, 2.101, 2.093, 2.086, 2.080, 2.074, 2.069, 2.064, 2.060, 2.056, 2.052, 2.048, 2.045]


def t95(n: int) -> float:
    if n < 2:
        return float("inf")
    return _T95[n - 2] if n - 2 < len(_T95) else 1.96


class ClockReader:
    """SM clock of one GPU through NVML (read-only); ``read()`` returns MHz or None when NVML is unavailable."""

    def __init__(self, index: Optional[int] = None):
        self._h = None
        try:
            import pynvml
            pynvml.nvmlInit()
            idx = torch.cuda.current_device() if index is None else index
            # torch's device index counts visible devices; map through the UUID so that masking does not matter
            uuid = str(torch.cuda.get_device_properties(idx).uuid)
            for i in range(pynvml.nvmlDeviceGetCount()):
                h = pynvml.nvmlDeviceGetHandleByIndex(i)
                u = pynvml.nvmlDeviceGetUUID(h)
                u = u.decode() if isinstance(u, bytes) else u
                if uuid in u:
                    self._h = h
                    break
            if self._h is None:
                self._h = pynvml.nvmlDeviceGetHandleByIndex(idx)
            self._nv = pynvml
        except Exception:
            self._h = None

    def read(self) -> Optional[float]:
        if self._h is None:
            return None
        try:
            return float(self._nv.nvmlDeviceGetClockInfo(self._h, self._nv.NVML_CLOCK_SM))
        except Exception:
            return None


def time_batch(fn: Fn, calls: int, start_index: int = 0) -> float:
    """Milliseconds per call of ``calls`` back-to-back calls (CUDA events, synchronised on both sides)."""
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(calls):
        fn(start_index + i)
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / calls


def calibrate(fn: Fn, target_ms: float = 4.0, warmup: int = 3, max_calls: int = 256) -> int:
    """Warm ``fn`` up and return how many calls make a batch of about ``target_ms``."""
    for i in range(warmup):
        fn(i)
    per = max(time_batch(fn, 2, warmup), 1e-4)
    return int(min(max_calls, max(1, round(target_ms / per))))


@dataclass
class Series:
    ms: List[float] = field(default_factory=list)
    mhz: List[float] = field(default_factory=list)

    @property
    def median_ms(self) -> float:
        return statistics.median(self.ms)

    @property
    def median_mhz(self) -> Optional[float]:
        return statistics.median(self.mhz) if self.mhz else None

    @property
    def mcycles(self) -> Optional[float]:
        """time x clock, in millions of SM cycles (comparable across power-cap states)."""
        m = self.median_mhz
        return None if m is None else self.median_ms * m * 1e-3


@dataclass
class Paired:
    a: Series
    b: Optional[Series]
    ratio: Optional[float] = None       # geometric mean of b / a  (> 1: a is faster)
    ci_lo: Optional[float] = None
    ci_hi: Optional[float] = None
    rounds: int = 0
    converged: bool = False

    @property
    def rel_halfwidth(self) -> Optional[float]:
        if self.ratio is None or self.ci_lo is None:
            return None
        return 0.5 * (self.ci_hi - self.ci_lo) / self.ratio


def ratio_ci(log_ratios: List[float]):
    """Geometric mean and its 95 % confidence interval from per-round log ratios."""
    n = len(log_ratios)
    mean = sum(log_ratios) / n
    if n < 2:
        return math.exp(mean), 0.0, float("inf")
    sd = statistics.stdev(log_ratios)
    half = t95(n) * sd / math.sqrt(n)
    return math.exp(mean), math.exp(mean - half), math.exp(mean + half)


def paired_ratio(fa: Fn, fb: Optional[Fn], target_rel_ci: float = 0.03, min_rounds: int = 5, max_rounds: int = 30,
                 batch_ms: float = 4.0, budget_s: float = 20.0, clocks: Optional[ClockReader] = None) -> Paired:
    """Interleaved timing of ``fa`` (ours) and ``fb`` (the other implementation; None = time ``fa`` alone)."""
    ka = calibrate(fa, batch_ms)
    kb = calibrate(fb, batch_ms) if fb is not None else 0
    sa, sb = Series(), Series() if fb is not None else None
    logs: List[float] = []
    t_start = time.time()
    out = Paired(sa, sb)
    ia = ib = 0
    for rnd in range(max_rounds):
        order = ("a", "b") if rnd % 2 == 0 else ("b", "a")  # alternate who goes first
        ta = tb = None
        for which in order:
            if which == "a":
                ta = time_batch(fa, ka, ia)
                ia += ka
                sa.ms.append(ta)
                if clocks is not None and (m := clocks.read()) is not None:
                    sa.mhz.append(m)
            elif fb is not None:
                tb = time_batch(fb, kb, ib)
                ib += kb
                sb.ms.append(tb)
                if clocks is not None and (m := clocks.read()) is not None:
                    sb.mhz.append(m)
        out.rounds = rnd + 1
        if fb is not None:
            logs.append(math.log(tb / ta))
            out.ratio, out.ci_lo, out.ci_hi = ratio_ci(logs)
            done = out.rounds >= min_rounds and out.rel_halfwidth is not None and out.rel_halfwidth < target_rel_ci
        else:
            # a single implementation: stop when the CI of its own mean time is narrow enough
            if len(sa.ms) >= 2:
                mean = sum(sa.ms) / len(sa.ms)
                half = t95(len(sa.ms)) * statistics.stdev(sa.ms) / math.sqrt(len(sa.ms))
                done = out.rounds >= min_rounds and half / mean < target_rel_ci
            else:
                done = False
        if done:
            out.converged = True
            break
        if time.time() - t_start > budget_s:
            break
    return out
