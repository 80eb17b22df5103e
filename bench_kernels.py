#!/usr/bin/env python
"""Per-kernel benchmark and sweep: this framework's sm_100a kernels vs the library path on the same shapes.

    python bench_kernels.py --op conv_fwd --cin 64 --cout 64 --size 128 [--batch 1] [--iters 10] [--no-ref]
    python bench_kernels.py --sweep            # the shapes of the scale-7 U-Net, every direction

Ops: conv_fwd, conv_dgrad, conv_wgrad (3x3x3 'same'), convT_fwd (k2s2), gn_fwd, gn_bwd (GroupNorm(8)+ReLU),
loss (fused CE + Dice forward + gradient), adam (clip + Adam over `--cin` million parameters).
Timing: CUDA events on the launching stream, 3 warm-up calls, operands larger than L2 or rotated between calls.
Each line reports time, achieved TFLOP/s or GB/s, the fraction of the measured peak (MEASURED_PEAKS.json: cuBLAS bf16
burst and copy bandwidth; fallback 1590 TFLOP/s and 6650 GB/s) and the library path (cuDNN / ATen) on the same shape.
"""
from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

import torch
import torch.nn.functional as F

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

from scaffold_b200.ops import _lib, conv_kernels as ck, gn_kernels as gk, loss as L  # noqa: E402


def peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return float(d["bf16_tflops"]), float(d["hbm_gbs"]), "measured"
    return 1590.0, 6650.0, "fallback"


def timeit(fn, iters, rotate=None):
    for i in range(3):
        fn(i)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(iters):
        fn(i)
    e1.record()
    torch.cuda.synchronize()
    _lib.check_status()
    return e0.elapsed_time(e1) / iters


def rot(n, make):
    return [make() for _ in range(n)]


def run(op, cin, cout, size, batch, iters, ref=True, kd_fused=True):
    tf_peak, bw_peak, which = peaks()
    n, s = batch, size
    dev = "cuda"
    out = {"op": op, "cin": cin, "cout": cout, "size": s, "batch": n}
    if op.startswith("conv_"):
        nbuf = max(2, min(4, int(3e8 // max(1, n * s ** 3 * max(cin, cout) * 2)) + 1))  # rotate operands past L2
        xs = rot(nbuf, lambda: torch.randn(n, s, s, s, max(cin, 16), device=dev).to(torch.bfloat16))
        gys = rot(nbuf, lambda: torch.randn(n, s, s, s, cout, device=dev).to(torch.bfloat16))
        w = torch.randn(cout, max(cin, 16), 3, 3, 3, device=dev) * 0.05
        wf, wd = ck.pack_weight_fwd(w), ck.pack_weight_dgrad(w)
        dw = torch.empty_like(w)
        flops = 2.0 * n * s ** 3 * max(cin, 16) * cout * 27
        if op == "conv_fwd":
            fn = lambda i: ck.conv_same([xs[i % nbuf]], wf, 3, [cout], kd_fused=kd_fused)
        elif op == "conv_dgrad":
            fn = lambda i: ck.conv_same([gys[i % nbuf]], wd, 3, [max(cin, 16)], kd_fused=kd_fused)
        else:
            fn = lambda i: ck.conv_wgrad(gys[i % nbuf], [xs[i % nbuf]], 3, dw)
        ms = timeit(fn, iters)
        out.update(ms=ms, tflops=flops / ms / 1e9, frac=flops / ms / 1e9 / tf_peak)
        if ref:
            torch.backends.cudnn.benchmark = True
            wc = w.to(torch.bfloat16).contiguous(memory_format=torch.channels_last_3d)
            xc = [x.permute(0, 4, 1, 2, 3) for x in xs]
            gc = [g.permute(0, 4, 1, 2, 3) for g in gys]
            mask = {"conv_fwd": None, "conv_dgrad": [True, False, False], "conv_wgrad": [False, True, False]}[op]
            if op == "conv_fwd":
                rfn = lambda i: F.conv3d(xc[i % nbuf], wc, padding=1)
            else:
                rfn = lambda i: torch.ops.aten.convolution_backward(gc[i % nbuf], xc[i % nbuf], wc, None, [1, 1, 1],
                                                                    [1, 1, 1], [1, 1, 1], False, [0, 0, 0], 1, mask)
            rms = timeit(rfn, iters)
            out.update(ref_ms=rms, ref_tflops=flops / rms / 1e9, speedup=rms / ms)
    elif op == "convT_fwd":
        x = torch.randn(n, s, s, s, cin, device=dev).to(torch.bfloat16)
        w = torch.randn(cin, cout, 2, 2, 2, device=dev) * 0.05
        b = torch.randn(cout, device=dev)
        wp = ck.pack_weight_convT_fwd(w)
        ms = timeit(lambda i: ck.convT_fwd(x, wp, cout, b), iters)
        nbytes = x.numel() * 2 + n * (2 * s) ** 3 * cout * 2
        out.update(ms=ms, gbs=nbytes / ms / 1e6, frac=nbytes / ms / 1e6 / bw_peak)
        if ref:
            xc, wc = x.permute(0, 4, 1, 2, 3), w.to(torch.bfloat16)
            rms = timeit(lambda i: F.conv_transpose3d(xc, wc, b.to(torch.bfloat16), stride=2), iters)
            out.update(ref_ms=rms, speedup=rms / ms)
    elif op in ("gn_fwd", "gn_bwd"):
        c = cin
        x = torch.randn(n, s, s, s, c, device=dev).to(torch.bfloat16)
        dy = torch.randn_like(x)
        w, b = torch.randn(c, device=dev), torch.randn(c, device=dev)
        y, mean, rstd = gk.gn_forward(x, w, b, 8)
        vol = x.numel() * 2
        if op == "gn_fwd":
            ms = timeit(lambda i: gk.gn_forward(x, w, b, 8), iters)
            nbytes = 3 * vol
        else:
            ms = timeit(lambda i: gk.gn_backward(dy, x, w, b, mean, rstd, 8), iters)
            nbytes = 5 * vol
        out.update(ms=ms, gbs=nbytes / ms / 1e6, frac=nbytes / ms / 1e6 / bw_peak)
        if ref:
            xc = x.permute(0, 4, 1, 2, 3).detach().requires_grad_(op == "gn_bwd")
            wb, bb = w.to(torch.bfloat16), b.to(torch.bfloat16)
            if op == "gn_fwd":
                rms = timeit(lambda i: F.relu(F.group_norm(xc, 8, wb, bb)), iters)
            else:
                dyc = dy.permute(0, 4, 1, 2, 3)

                def rfn(i):
                    xc.grad = None
                    F.relu(F.group_norm(xc, 8, wb, bb)).backward(dyc)
                rms = timeit(rfn, iters)  # library number includes its forward
            out.update(ref_ms=rms, speedup=rms / ms)
    elif op == "loss":
        c = cout
        cp = (c + 15) // 16 * 16
        lg = torch.randn(n, s, s, s, cp, device=dev).to(torch.bfloat16)
        lab = torch.randint(0, c, (n, s, s, s), device=dev, dtype=torch.int16)

        def fn(i):
            t = lg.detach().requires_grad_(True)
            L.segmentation_loss_fused(t, lab, c)[0].backward()
        ms = timeit(fn, iters)
        nbytes = lg.numel() * 2 * 3 + lab.numel() * 2 * 2
        out.update(ms=ms, gbs=nbytes / ms / 1e6, frac=nbytes / ms / 1e6 / bw_peak)
        if ref:
            lr = lg[..., :c].permute(0, 4, 1, 2, 3)

            def rfn(i):
                t = lr.detach().requires_grad_(True)
                L.segmentation_loss_reference(t, lab.long(), c)[0].backward()
            rms = timeit(rfn, iters)
            out.update(ref_ms=rms, speedup=rms / ms)
    elif op == "adam":
        from scaffold_b200.ops.optim import FusedClipAdam
        numel = cin * 1_000_000
        p = torch.nn.Parameter(torch.randn(numel, device=dev))
        opt = FusedClipAdam([p], lr=1e-3)
        opt.attach()
        p.grad.normal_()
        ms = timeit(lambda i: opt.step(), iters)
        nbytes = numel * 4 * (1 + 7)  # norm pass reads g; update reads p,g,m,v and writes p,m,v
        out.update(ms=ms, gbs=nbytes / ms / 1e6, frac=nbytes / ms / 1e6 / bw_peak)
    else:
        raise SystemExit(f"unknown op {op}")
    out["peaks"] = which
    return out


def fmt(r):
    core = f"{r['op']:10s} cin {r['cin']:4d} cout {r['cout']:4d} size {r['size']:3d} batch {r['batch']} : {r['ms']:8.3f} ms"
    if "tflops" in r:
        core += f"  {r['tflops']:7.0f} TFLOP/s  {100 * r['frac']:5.1f}% of {r['peaks']} bf16 peak"
    else:
        core += f"  {r['gbs']:7.0f} GB/s  {100 * r['frac']:5.1f}% of {r['peaks']} copy bandwidth"
    if "ref_ms" in r:
        core += f"  | library {r['ref_ms']:8.3f} ms  -> {r['speedup']:.2f}x"
    return core


SWEEP = [(64, 64, 128), (128, 64, 128), (64, 128, 64), (128, 128, 64), (256, 128, 64), (128, 256, 32), (256, 256, 32),
         (512, 256, 32), (256, 512, 16), (512, 512, 16), (1024, 512, 16), (512, 1024, 8), (1024, 1024, 8), (3, 64, 128)]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--op", default="conv_fwd")
    ap.add_argument("--cin", type=int, default=64)
    ap.add_argument("--cout", type=int, default=64)
    ap.add_argument("--size", type=int, default=64)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--no-ref", action="store_true")
    ap.add_argument("--no-kd-fused", action="store_true", help="narrow-output 3x3x3 convs on the one-tap-per-MMA kernel")
    ap.add_argument("--sweep", action="store_true")
    ap.add_argument("--json", action="store_true")
    a = ap.parse_args()
    rows = []
    if a.sweep:
        for cin, cout, size in SWEEP:
            for op in ("conv_fwd", "conv_dgrad", "conv_wgrad"):
                if op == "conv_dgrad" and cin < 16:
                    continue
                rows.append(run(op, cin, cout, size, a.batch, a.iters, not a.no_ref))
                print(fmt(rows[-1]), flush=True)
        for c, size in ((64, 128), (128, 64), (256, 32), (512, 16)):
            for op in ("gn_fwd", "gn_bwd"):
                rows.append(run(op, c, c, size, a.batch, a.iters, not a.no_ref))
                print(fmt(rows[-1]), flush=True)
        for extra in (("loss", 64, 9, 128), ("convT_fwd", 128, 64, 64), ("adam", 90, 0, 0)):
            rows.append(run(extra[0], extra[1], extra[2], extra[3], a.batch, a.iters, not a.no_ref))
            print(fmt(rows[-1]), flush=True)
    else:
        rows.append(run(a.op, a.cin, a.cout, a.size, a.batch, a.iters, not a.no_ref, not a.no_kd_fused))
        print(fmt(rows[-1]), flush=True)
    if a.json:
        print(json.dumps(rows))


if __name__ == "__main__":
    main()
