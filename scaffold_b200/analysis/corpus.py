"""Corpus fixture: every convolution of a U-Net configuration joined with measured kernel times.

``build`` takes the rows ``bench_kernels.py --sweep --json <file>`` writes and the analytic corpus of the
configuration (``shapes.scaffold_corpus``) and produces one record per distinct layer shape: how often the
shape occurs in a step, FLOPs, bytes, roofline, the kernel each direction routes to, this framework's and the
library's measured milliseconds per call, and the per-step totals. The committed fixture
``data/scaffold_corpus_scale7_b200.json`` is what tests and "which layers matter" decisions read.

    python -m scaffold_b200.analysis.corpus --sweep-json out/sweep.json \\
        --out scaffold_b200/analysis/data/scaffold_corpus_scale7_b200.json

Role of the reference: triton_conv3d/tests/data/scaffold_corpus.json and the make_corpus tooling around it.
"""
from __future__ import annotations

import argparse
import json
from collections import OrderedDict
from pathlib import Path
from typing import Dict, Iterable, List

from .shapes import ConvProblem, measured_peaks, scaffold_corpus

DATA = Path(__file__).resolve().parent / "data"
_KIND = {("conv", "fwd"): "conv_fwd", ("conv", "dgrad"): "conv_dgrad", ("conv", "wgrad"): "conv_wgrad",
         ("convT", "fwd"): "convT_fwd", ("convT", "dgrad"): "convT_dgrad"}


def build(sweep_rows: Iterable[Dict], problem_scale: int = 7, batch: int = 2, base_width: int = 64,
          n_categories: int = 8) -> Dict:
    index = {(r["op"], r["cin"], r["cout"], r["size"], r["batch"]): r for r in sweep_rows}
    layers: "OrderedDict[tuple, Dict]" = OrderedDict()
    for p in scaffold_corpus(problem_scale, 3, batch, n_categories, base_width):
        key = (p.kernel, p.transposed, p.cin, p.cout, p.spatial)
        rec = layers.get(key)
        if rec is None:
            rec = layers[key] = {"label": p.label, "names": [], "count": 0, "n": p.n, "cin": p.cin, "cout": p.cout,
                                 "spatial": list(p.spatial), "kernel": p.kernel, "transposed": p.transposed,
                                 "gemm_fwd": list(p.gemm_shape("fwd")), "directions": {}}
            fam = "convT" if p.transposed else "conv"
            for d in ("fwd", "dgrad", "wgrad"):
                entry = {"flops": p.flops(d), "bytes": p.bytes(d), "roofline_ms": p.roofline_seconds(d) * 1e3,
                         "route": p.route(d)}
                m = index.get((_KIND.get((fam, d), ""), p.cin, p.cout, p.spatial[-1], p.n)) if p.kernel != 1 else None
                if m is not None:
                    entry.update(ms=m["ms"], library_ms=m.get("ref_ms"), ratio=m.get("speedup"), ci=m.get("ci"),
                                 fraction_of_roofline=entry["roofline_ms"] / m["ms"])
                rec["directions"][d] = entry
        rec["names"].append(p.name)
        rec["count"] += 1
    tf, gbs, which = measured_peaks()
    totals = {}
    for d in ("fwd", "dgrad", "wgrad"):
        ours = sum(r["count"] * r["directions"][d]["ms"] for r in layers.values() if "ms" in r["directions"][d])
        lib = sum(r["count"] * r["directions"][d]["library_ms"] for r in layers.values()
                  if r["directions"][d].get("library_ms"))
        roof = sum(r["count"] * r["directions"][d]["roofline_ms"] for r in layers.values())
        totals[d] = {"ms_per_step": ours, "library_ms_per_step": lib, "roofline_ms_per_step": roof}
    return {"config": {"problem_scale": problem_scale, "batch": batch, "base_width": base_width,
                       "n_categories": n_categories},
            "peaks": {"bf16_tflops": tf, "hbm_gbs": gbs, "source": which},
            "totals": totals, "layers": list(layers.values())}


def load(name: str = "scaffold_corpus_scale7_b200.json") -> Dict:
    return json.loads((DATA / name).read_text())


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description="join a kernel sweep with the U-Net's convolution corpus")
    ap.add_argument("--sweep-json", required=True)
    ap.add_argument("--out", required=True)
    ap.add_argument("--problem-scale", type=int, default=7)
    ap.add_argument("--batch", type=int, default=2)
    a = ap.parse_args(argv)
    doc = build(json.loads(Path(a.sweep_json).read_text()), a.problem_scale, a.batch)
    Path(a.out).parent.mkdir(parents=True, exist_ok=True)
    Path(a.out).write_text(json.dumps(doc, indent=1))
    for d, t in doc["totals"].items():
        print(f"{d:6s}: ours {t['ms_per_step']:.2f} ms/step, library {t['library_ms_per_step']:.2f}, roofline "
              f"{t['roofline_ms_per_step']:.2f}")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
