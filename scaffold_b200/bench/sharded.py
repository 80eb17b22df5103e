"""Depth-sharded kernels against the library path, one shard per rank (run under ``torch.distributed.run``).

Each point times, on every rank at once (device time, maximum over ranks):

* ``conv_fwd`` with the halo fused into the kernel: boundary planes pushed into the neighbours' landing
  slabs over NVLink (``halo_push_kernel``) + the convolution that waits on the flags only in its boundary
  tiles; against NCCL ``batch_isend_irecv`` of the slabs + ``torch.cat`` + a cuDNN convolution;
* ``gn_fwd`` with cross-shard statistics through peer memory (``gn_stats`` -> ``gn_share`` -> ``gn_apply``);
  against ATen sums + an NCCL all-reduce of the statistics + the ATen normalisation formula.

Rooflines: the convolution's FLOPs at the measured bf16 peak or its slab bytes at the measured NVLink rate
(770 GB/s per direction), whichever is slower; GroupNorm's 3 x tensor bytes at the measured copy bandwidth.
"""
from __future__ import annotations

import json
import os
from pathlib import Path

import torch
import torch.distributed as dist
import torch.nn.functional as F

NVLINK_GBS = 770.0


def _timeit(fn, iters=20, warm=3):
    for i in range(warm):
        fn(i)
    torch.cuda.synchronize()
    dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(iters):
        fn(i)
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / iters], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def main(args):
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    dist.init_process_group("nccl", device_id=dev)
    from ..ops import _lib, conv_kernels as ck, gn_kernels as gk
    from ..parallel.layout import ParallelLayout
    from ..parallel.spatial import SpatialContext

    root = Path(__file__).resolve().parents[2]
    try:
        pk = json.loads((root / "MEASURED_PEAKS.json").read_text())
        tf_peak, bw_peak, which = float(pk["bf16_tflops"]), float(pk["hbm_gbs"]), "measured"
    except Exception:
        tf_peak, bw_peak, which = 1590.0, 6650.0, "fallback"

    layout = ParallelLayout([world, 1, 1], (2, 3, 4), world, rank)
    sp = SpatialContext(layout, gn_stats="global", halo_backend="fused")
    chan, stats = sp.halo_channel, sp.stats_channel
    assert chan is not None and stats is not None
    chans = [int(c) for c in args.grid_channels.split(",")]
    sizes = [int(s) for s in args.grid_sizes.split(",")]
    rows = []
    for size in sizes:
        for c in chans:
            if size * size * size * c * 2 > (6 << 30):
                continue
            n, d, h, w = 1, size, size, size  # the LOCAL extent per shard
            x = torch.randn(n, d, h, w, c, device=dev).to(torch.bfloat16)
            wt = torch.randn(c, c, 3, 3, 3, device=dev) * 0.05
            wf = ck.pack_weight_fwd(wt)

            def fused(i):
                land = chan.exchange([x[:, 0]], [x[:, -1]])
                ck.conv_same([x], wf, 3, [c], halo=land)
            xc = x.permute(0, 4, 1, 2, 3)
            wc = wt.to(torch.bfloat16).contiguous(memory_format=torch.channels_last_3d)
            torch.backends.cudnn.benchmark = True

            def library(i):
                xp = sp.halo_pad(xc, 1)
                F.conv3d(xp, wc, padding=(0, 1, 1))
            t_f, t_l = _timeit(fused), _timeit(library)
            _lib.check_status()
            flops = 2.0 * n * d * h * w * c * c * 27
            slab = n * h * w * c * 2  # bytes per face and direction
            roof = max(flops / (tf_peak * 1e12), slab / (NVLINK_GBS * 1e9)) * 1e3
            rows.append({"op": "conv_fwd+halo", "c": c, "size": size, "shards": world, "ms": t_f, "library_ms": t_l,
                         "roofline_ms": roof, "frac": roof / t_f, "speedup": t_l / t_f, "peaks": which})
            wg, bg = torch.randn(c, device=dev), torch.randn(c, device=dev)

            def gn_fused(i):
                fin = gk.gn_stats(x, wg, bg, 8, 1e-5, True)
                parts, wait = stats.share(fin)
                gk.gn_apply(x, wg, bg, 8, 1e-5, True, parts, shards=world, wait=wait)

            def gn_library(i):
                F.relu(sp.group_norm_reference(xc, 8, wg, bg, 1e-5))
            t_f, t_l = _timeit(gn_fused), _timeit(gn_library)
            _lib.check_status()
            roof = 3 * x.numel() * 2 / (bw_peak * 1e9) * 1e3
            rows.append({"op": "gn_fwd+stats", "c": c, "size": size, "shards": world, "ms": t_f, "library_ms": t_l,
                         "roofline_ms": roof, "frac": roof / t_f, "speedup": t_l / t_f, "peaks": which})
            if rank == 0:
                for r in rows[-2:]:
                    print(f"{r['op']:14s} C={r['c']:4d} local {size}^3 x{world} shards: {r['ms']:8.3f} ms  "
                          f"{100 * r['frac']:5.1f}% of its roofline ({r['peaks']})  | NCCL + library {r['library_ms']:8.3f} ms"
                          f" -> {r['speedup']:.2f}x", flush=True)
            del x, xc
            torch.cuda.empty_cache()
    dist.barrier()
    dist.destroy_process_group()
    return rows
