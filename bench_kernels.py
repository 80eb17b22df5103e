#!/usr/bin/env python
"""Per-kernel benchmark: this framework's sm_100a kernels against the library path on the same tensors.

    python bench_kernels.py --op conv_fwd --cin 64 --cout 64 --size 128 [--batch 1] [--no-ref]
    python bench_kernels.py --sweep                  # the layer shapes of the scale-7 U-Net, every direction
    python bench_kernels.py --grid                   # C in {16..512} x {16,32,64,128}^3 x every op (+ GEMM ceiling)
    python bench_kernels.py --datagen                # IFS chaos game / voxeliser: GPU kernels vs the native CPU code
    torchrun --nproc-per-node N bench_kernels.py --sharded   # depth shards: fused halo / peer statistics vs NCCL + library

Ops: conv_fwd, conv_dgrad, conv_wgrad (3x3x3 'same'), convT_fwd, convT_dgrad (k2s2), gn_fwd, gn_bwd
(GroupNorm(8)+ReLU), pool_fwd, pool_bwd, loss (fused CE + Dice forward + gradient), adam (clip + Adam over
`--cin` million parameters), gemm (the tcgen05 ceiling probe: --size^3 * --batch rows, N = --cout, K = --cin).

Every comparison is PAIRED: ours and the library alternate in batches of a few milliseconds until the 95 %
confidence interval of their ratio is under 3 % (``scaffold_b200/bench/harness.py``). A line reports the median
time, the achieved TFLOP/s or GB/s, the fraction of the measured peak (MEASURED_PEAKS.json: cuBLAS bf16 burst and
copy bandwidth; fallback 1590 TFLOP/s and 6650 GB/s), time x median SM clock (Mcycles, comparable across
power-cap states) and ``library/ours`` with its interval.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

from scaffold_b200.bench import cases, gemm_probe  # noqa: E402
from scaffold_b200.bench.harness import ClockReader, paired_ratio  # noqa: E402
from scaffold_b200.ops import _lib  # noqa: E402


def peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return float(d["bf16_tflops"]), float(d["hbm_gbs"]), "measured"
    return 1590.0, 6650.0, "fallback"


def build(op, cin, cout, size, batch, ref=True, kd_fused=True, gn_groups=0) -> cases.Case:
    if op in ("conv_fwd", "conv_dgrad", "conv_wgrad"):
        return cases.conv_case(op, cin, cout, size, batch, kd_fused, ref, gn_groups if op == "conv_fwd" else 0)
    if op in ("convT_fwd", "convT_dgrad"):
        return cases.convT_case(op, cin, cout, size, batch, ref)
    if op in ("gn_fwd", "gn_bwd"):
        return cases.gn_case(op, cin, size, batch, ref)
    if op in ("pool_fwd", "pool_bwd"):
        return cases.pool_case(op, cin, size, batch, ref)
    if op == "loss":
        return cases.loss_case(cout, size, batch, ref)
    if op == "adam":
        return cases.adam_case(cin)
    if op == "gemm":
        return gemm_probe.gemm_case(batch * size ** 3, cout, cin, ref)
    raise SystemExit(f"unknown op {op}")


def run(op, cin, cout, size, batch, ref=True, kd_fused=True, clocks=None, budget_s=12.0, gn_groups=0):
    tf_peak, bw_peak, which = peaks()
    case = build(op, cin, cout, size, batch, ref, kd_fused, gn_groups)
    res = paired_ratio(case.ours, case.library if ref else None, clocks=clocks, budget_s=budget_s)
    _lib.check_status()
    ms = res.a.median_ms
    out = {"op": op, "cin": cin, "cout": cout, "size": size, "batch": batch, "label": case.label, "ms": ms,
           "rounds": res.rounds, "converged": res.converged, "peaks": which, "mhz": res.a.median_mhz,
           "mcycles": res.a.mcycles}
    if case.flops:
        out.update(tflops=case.flops / ms / 1e9, frac=case.flops / ms / 1e9 / tf_peak)
    else:
        out.update(gbs=case.bytes / ms / 1e6, frac=case.bytes / ms / 1e6 / bw_peak)
    if case.gemm:
        out["gemm"] = list(case.gemm)
    if res.b is not None:
        out.update(ref_ms=res.b.median_ms, speedup=res.ratio, ci=[res.ci_lo, res.ci_hi])
    del case
    torch.cuda.empty_cache()
    return out


def fmt(r):
    core = f"{r['op']:11s} {r['label']:26s}: {r['ms']:8.3f} ms"
    if "tflops" in r:
        core += f"  {r['tflops']:7.0f} TFLOP/s  {100 * r['frac']:5.1f}% of {r['peaks']} bf16 peak"
    else:
        core += f"  {r['gbs']:7.0f} GB/s  {100 * r['frac']:5.1f}% of {r['peaks']} copy bandwidth"
    if r.get("mcycles") is not None:
        core += f"  {r['mcycles']:7.3f} Mcyc @{r['mhz']:.0f} MHz"
    if "ref_ms" in r:
        half = 50.0 * (r["ci"][1] - r["ci"][0]) / r["speedup"]
        core += (f"  | library {r['ref_ms']:8.3f} ms -> {r['speedup']:.2f}x +-{half:.1f}%"
                 f"{'' if r['converged'] else ' (not converged)'}")
    return core


SWEEP = [(64, 64, 128), (128, 64, 128), (64, 128, 64), (128, 128, 64), (256, 128, 64), (128, 256, 32), (256, 256, 32),
         (512, 256, 32), (256, 512, 16), (512, 512, 16), (1024, 512, 16), (512, 1024, 8), (1024, 1024, 8), (3, 64, 128)]


def sweep(a, clocks):
    rows = []

    def go(*args):
        rows.append(run(*args, ref=not a.no_ref, clocks=clocks, budget_s=a.budget))
        print(fmt(rows[-1]), flush=True)
    for cin, cout, size in SWEEP:
        for op in ("conv_fwd", "conv_dgrad", "conv_wgrad"):
            if op == "conv_dgrad" and cin < 16:
                continue
            go(op, cin, cout, size, a.batch)
    for c, size in ((64, 128), (128, 64), (256, 32), (512, 16), (1024, 8)):
        for op in ("gn_fwd", "gn_bwd"):
            go(op, c, c, size, a.batch)
    for cin, cout, size in ((1024, 512, 8), (512, 256, 16), (256, 128, 32), (128, 64, 64)):
        go("convT_fwd", cin, cout, size, a.batch)
        go("convT_dgrad", cin, cout, size, a.batch)
    for c, size in ((64, 128), (128, 64), (256, 32)):
        go("pool_fwd", c, c, size, a.batch)
        go("pool_bwd", c, c, size, a.batch)
    go("loss", 64, 9, 128, a.batch)
    go("adam", 90, 0, 0, a.batch)
    return rows


def grid(a, clocks):
    """C_in = C_out in {16..512} x local extent {16, 32, 64, 128}^3, batch 1, every operator and direction, with
    the tcgen05 GEMM ceiling at each convolution's implied shape."""
    rows = []
    chans = [int(c) for c in a.grid_channels.split(",")]
    sizes = [int(s) for s in a.grid_sizes.split(",")]

    def go(*args):
        try:
            rows.append(run(*args, ref=not a.no_ref, clocks=clocks, budget_s=a.budget))
            print(fmt(rows[-1]), flush=True)
        except torch.cuda.OutOfMemoryError:
            print(f"{args[0]:11s} {args[1]}->{args[2]} @{args[3]}^3: skipped (does not fit beside its rotated copies)",
                  flush=True)
            torch.cuda.empty_cache()
    for size in sizes:
        for c in chans:
            for op in ("conv_fwd", "conv_dgrad", "conv_wgrad"):
                go(op, c, c, size, 1)
            go("gemm", c * 27, c, size, 1)
            go("gn_fwd", c, c, size, 1)
            go("gn_bwd", c, c, size, 1)
            if size <= 64 and c >= 32:
                go("convT_fwd", c, c // 2, size, 1)
                go("convT_dgrad", c, c // 2, size, 1)
    return rows


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--op", default="conv_fwd")
    ap.add_argument("--cin", type=int, default=64)
    ap.add_argument("--cout", type=int, default=64)
    ap.add_argument("--size", type=int, default=64)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--budget", type=float, default=12.0, help="seconds per point before the pairing loop gives up")
    ap.add_argument("--no-ref", action="store_true")
    ap.add_argument("--no-kd-fused", action="store_true", help="narrow-output 3x3x3 convs on the one-tap-per-MMA kernel")
    ap.add_argument("--gn-groups", type=int, default=0, help="conv_fwd: also produce GroupNorm statistics in the epilogue")
    ap.add_argument("--quick", action="store_true",
                    help="a handful of calls of our kernel only, no pairing loop (the form to run under a profiler)")
    ap.add_argument("--iters", type=int, default=0,
                    help="like --quick with 3 warm-up calls + this many calls (the fixed-iteration form of older profiles)")
    ap.add_argument("--sweep", action="store_true")
    ap.add_argument("--grid", action="store_true")
    ap.add_argument("--grid-channels", default="16,32,64,128,256,512")
    ap.add_argument("--grid-sizes", default="16,32,64,128")
    ap.add_argument("--sharded", action="store_true", help="run under torchrun: one depth shard per rank")
    ap.add_argument("--datagen", action="store_true")
    ap.add_argument("--json", default=None, help="also write the rows to this file")
    a = ap.parse_args()
    if a.sharded:
        from scaffold_b200.bench.sharded import main as sharded_main
        rows = sharded_main(a)
    elif a.datagen:
        from scaffold_b200.bench.datagen import main as datagen_main
        rows = datagen_main(a)
    else:
        clocks = ClockReader()
        if a.sweep:
            rows = sweep(a, clocks)
        elif a.grid:
            rows = grid(a, clocks)
        elif a.quick or a.iters > 0:
            case = build(a.op, a.cin, a.cout, a.size, a.batch, False, not a.no_kd_fused, a.gn_groups)
            for i in range(3 + a.iters if a.iters > 0 else 6):
                case.ours(i)
            torch.cuda.synchronize()
            _lib.check_status()
            rows = [{"op": a.op, "label": case.label, "quick": True}]
            print(f"{a.op} {case.label}: calls done", flush=True)
        else:
            rows = [run(a.op, a.cin, a.cout, a.size, a.batch, not a.no_ref, not a.no_kd_fused, clocks, a.budget,
                        a.gn_groups)]
            print(fmt(rows[-1]), flush=True)
    if a.json and int(os.environ.get("RANK", "0")) == 0:
        Path(a.json).parent.mkdir(parents=True, exist_ok=True)
        Path(a.json).write_text(json.dumps(rows))


if __name__ == "__main__":
    main()
