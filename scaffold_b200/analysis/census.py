"""Census of the convolutions a run issues, and the corpus built from it.

``ConvCensus`` wraps the launchers of ``scaffold_b200.ops.conv_kernels`` while it is active and counts
every call by (operator, direction-independent shape key). ``make_corpus`` joins a census with measured
per-kernel times (the JSON rows ``bench_kernels.py --json`` prints) into records of shape, count,
FLOPs, roofline and measured milliseconds: the data behind "which layers matter" decisions.

Role of the reference: triton_conv3d/tests/data/{conv_census,make_census,make_corpus}.py (instrumented
run -> census -> corpus joined with profiled library times).
"""
from __future__ import annotations

import json
from collections import Counter
from typing import Dict, Iterable, List, Optional

from .shapes import ConvProblem


class ConvCensus:
    """Context manager: ``with ConvCensus() as c: step(); c.counts`` -> Counter of call signatures."""

    def __init__(self):
        self.counts: Counter = Counter()
        self._saved = {}

    def _wrap(self, mod, name, key_fn):
        orig = getattr(mod, name)
        self._saved[name] = orig

        def wrapper(*a, **k):
            self.counts[key_fn(*a, **k)] += 1
            return orig(*a, **k)
        setattr(mod, name, wrapper)

    def __enter__(self):
        from ..ops import conv_kernels as ck
        self._mod = ck

        def k_same(srcs, wpack, ksize, dst_channels, *a, **k):
            n = srcs[0].shape[0]
            dims = tuple(k.get("out_dims") or srcs[0].shape[1:4])
            return ("conv_same", n, tuple(s.shape[4] for s in srcs), tuple(dst_channels), ksize, dims,
                    k.get("halo") is not None, k.get("slabs") is not None)

        def k_convT(x, wpack, cout, bias):
            return ("convT_fwd", x.shape[0], (x.shape[4],), (cout,), 2, tuple(x.shape[1:4]), False, False)

        def k_convT_d(gy, wpack, cin):
            return ("convT_dgrad", gy.shape[0], (gy.shape[4],), (cin,), 2, tuple(gy.shape[1:4]), False, False)

        def k_wgrad(gy, xs, ksize, dw, *a, **k):
            return ("conv_wgrad", gy.shape[0], tuple(x.shape[4] for x in xs), (gy.shape[4],), ksize,
                    tuple(gy.shape[1:4]), k.get("x_halo") is not None, False)

        self._wrap(ck, "conv_same", k_same)
        self._wrap(ck, "convT_fwd", k_convT)
        self._wrap(ck, "convT_dgrad", k_convT_d)
        self._wrap(ck, "conv_wgrad", k_wgrad)
        return self

    def __exit__(self, *exc):
        for name, orig in self._saved.items():
            setattr(self._mod, name, orig)
        self._saved = {}
        return False

    def records(self) -> List[Dict]:
        out = []
        for (op, n, cins, couts, k, dims, halo, slabs), cnt in sorted(self.counts.items(), key=lambda kv: -kv[1]):
            out.append({"op": op, "n": n, "cin": list(cins), "cout": list(couts), "kernel": k, "dims": list(dims),
                        "fused_halo": halo, "slab_outputs": slabs, "count": cnt})
        return out


def problem_of(rec: Dict) -> ConvProblem:
    cin, cout = sum(rec["cin"]), sum(rec["cout"])
    dims = tuple(rec["dims"])
    if rec["op"] == "convT_dgrad":  # called on the upsampled gradient
        return ConvProblem(rec["n"], cout, cin, tuple(v // 2 for v in dims), 2, True)
    if rec["op"] == "convT_fwd":
        return ConvProblem(rec["n"], cin, cout, dims, 2, True)
    return ConvProblem(rec["n"], cin, cout, dims, rec["kernel"])


def make_corpus(census: Iterable[Dict], measured: Optional[Iterable[Dict]] = None) -> List[Dict]:
    """Join census records with ``bench_kernels.py --json`` rows (matched on op kind, channels, size, batch)."""
    index = {}
    for row in measured or []:
        index[(row["op"], row["cin"], row["cout"], row["size"], row["batch"])] = row
    out = []
    for rec in census:
        p = problem_of(rec)
        direction = {"conv_same": "fwd", "conv_wgrad": "wgrad", "convT_fwd": "fwd", "convT_dgrad": "dgrad"}[rec["op"]]
        entry = dict(rec)
        entry.update(label=p.label, flops=p.flops(direction), bytes=p.bytes(direction),
                     roofline_ms=p.roofline_seconds(direction) * 1e3, route=p.route(direction))
        for kind in ("conv_fwd", "conv_dgrad", "conv_wgrad", "convT_fwd"):
            m = index.get((kind, p.cin, p.cout, p.spatial[-1], p.n))
            if m is not None and kind.endswith(direction):
                entry["measured_ms"] = m["ms"]
                entry["library_ms"] = m.get("ref_ms")
        out.append(entry)
    return out


def dump(records: List[Dict], path: str) -> None:
    with open(path, "w") as f:
        json.dump(records, f, indent=1)
