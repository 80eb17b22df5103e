"""Host-side tests of the paired benchmark loop (scaffold_b200/bench/harness.py) with a fake timer: convergence on
the confidence interval, who-goes-first alternation, the time budget, and the single-implementation mode."""
import itertools
import math

import pytest

from scaffold_b200.bench import harness as H


def _fake(monkeypatch, times_a, times_b=None, clock=None):
    """time_batch returns scripted per-call milliseconds; calibrate returns one call per batch."""
    seq = {"a": itertools.cycle(times_a), "b": itertools.cycle(times_b or [1.0])}
    order = []

    def time_batch(fn, calls, start_index=0):
        order.append(fn.tag)
        return next(seq[fn.tag])

    monkeypatch.setattr(H, "time_batch", time_batch)
    monkeypatch.setattr(H, "calibrate", lambda fn, target_ms=4.0, warmup=3, max_calls=256: 1)

    def mk(tag):
        f = lambda i: None
        f.tag = tag
        return f
    return mk("a"), mk("b"), order


def test_steady_ratio_converges_at_the_minimum_number_of_rounds(monkeypatch):
    fa, fb, order = _fake(monkeypatch, [2.0], [3.0])
    res = H.paired_ratio(fa, fb, min_rounds=5, max_rounds=30)
    assert res.converged and res.rounds == 5
    assert res.ratio == pytest.approx(1.5) and res.ci_lo == pytest.approx(1.5) and res.ci_hi == pytest.approx(1.5)
    assert res.a.median_ms == 2.0 and res.b.median_ms == 3.0
    # the implementation that goes first alternates from round to round
    assert order[:8] == ["a", "b", "b", "a", "a", "b", "b", "a"]


def test_noisy_ratio_keeps_going_until_the_interval_is_narrow_or_rounds_run_out(monkeypatch):
    fa, fb, _ = _fake(monkeypatch, [2.0, 2.6, 1.7, 2.2], [3.0])
    res = H.paired_ratio(fa, fb, target_rel_ci=0.03, min_rounds=5, max_rounds=12)
    assert not res.converged and res.rounds == 12
    assert res.ci_lo < res.ratio < res.ci_hi and res.rel_halfwidth > 0.03
    loose = H.paired_ratio(fa, fb, target_rel_ci=0.5, min_rounds=5, max_rounds=12)
    assert loose.converged and loose.rounds == 5


def test_time_budget_stops_the_loop(monkeypatch):
    fa, fb, _ = _fake(monkeypatch, [2.0, 4.0], [3.0])
    ticks = itertools.count(0.0, 10.0)                       # every look at the wall clock is 10 s later
    monkeypatch.setattr(H.time, "time", lambda: next(ticks))
    res = H.paired_ratio(fa, fb, min_rounds=5, max_rounds=30, budget_s=15.0)
    assert not res.converged and res.rounds < 5


def test_single_implementation_mode_uses_its_own_mean(monkeypatch):
    fa, _, order = _fake(monkeypatch, [2.0, 2.02, 1.98])
    res = H.paired_ratio(fa, None, min_rounds=5, max_rounds=20)
    assert res.converged and res.b is None and res.ratio is None and set(order) == {"a"}
    assert 1.98 <= res.a.median_ms <= 2.02


def test_series_cycles_and_interval_arithmetic():
    s = H.Series(ms=[1.0, 2.0, 3.0], mhz=[1000.0, 2000.0, 1500.0])
    assert s.median_ms == 2.0 and s.median_mhz == 1500.0 and s.mcycles == pytest.approx(3.0)
    assert H.Series(ms=[1.0]).mcycles is None
    g, lo, hi = H.ratio_ci([math.log(2.0)])
    assert g == pytest.approx(2.0) and lo == 0.0 and math.isinf(hi)
    g, lo, hi = H.ratio_ci([math.log(2.0), math.log(2.0), math.log(2.0)])
    assert (g, lo, hi) == pytest.approx((2.0, 2.0, 2.0))
