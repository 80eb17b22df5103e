"""Benchmark cases: for an (op, shape) pair, the callable of this framework's kernel, the callable of the
library path on the same tensors, and the algorithmic work (FLOPs or bytes) one call does.

Operands are rotated through several copies whenever one copy is smaller than the L2 cache, so a timed
call never finds its inputs resident from the previous one.

Role of the reference: the operator x direction cases of triton_conv3d/bench/conv_bench.py:973-1560 and its
library baseline capture (triton_conv3d/bench/baseline.py).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Optional

import torch
import torch.nn.functional as F

from ..ops import conv_kernels as ck, gn_kernels as gk, loss as L

L2_BYTES = 126 << 20


@dataclass
class Case:
    op: str
    label: str
    ours: Callable[[int], object]
    library: Optional[Callable[[int], object]]
    flops: float = 0.0      # > 0: compute-bound reporting (TFLOP/s against the bf16 peak)
    bytes: float = 0.0      # > 0: bandwidth reporting (GB/s against the copy bandwidth)
    gemm: Optional[tuple] = None  # implicit-GEMM (M, N, K) of a convolution case


def _copies(bytes_per_copy: int) -> int:
    return max(2, min(6, (2 * L2_BYTES) // max(1, bytes_per_copy) + 1))


def _rot(n: int, make):
    return [make() for _ in range(n)]


def conv_case(op: str, cin: int, cout: int, size: int, batch: int, kd_fused: bool = True, library: bool = True,
              gn_groups: int = 0) -> Case:
    """``gn_groups`` > 0 (forward only): the kernel also writes the GroupNorm partial statistics of its output."""
    dev = "cuda"
    ci = max(cin, 16)
    n, s = batch, size
    nbuf = _copies(n * s ** 3 * max(ci, cout) * 2)
    xs = _rot(nbuf, lambda: torch.randn(n, s, s, s, ci, device=dev).to(torch.bfloat16))
    gys = _rot(nbuf, lambda: torch.randn(n, s, s, s, cout, device=dev).to(torch.bfloat16))
    w = torch.randn(cout, ci, 3, 3, 3, device=dev) * 0.05
    wf, wd = ck.pack_weight_fwd(w), ck.pack_weight_dgrad(w)
    dw = torch.empty_like(w)
    flops = 2.0 * n * s ** 3 * ci * cout * 27
    vox = n * s ** 3
    if op == "conv_fwd":
        ours = lambda i: ck.conv_same([xs[i % nbuf]], wf, 3, [cout], kd_fused=kd_fused, gn_groups=gn_groups,
                                      gn_sink=[] if gn_groups else None)
        gemm = (vox, cout, ci * 27)
    elif op == "conv_dgrad":
        ours = lambda i: ck.conv_same([gys[i % nbuf]], wd, 3, [ci], kd_fused=kd_fused)
        gemm = (vox, ci, cout * 27)
    elif op == "conv_wgrad":
        ours = lambda i: ck.conv_wgrad(gys[i % nbuf], [xs[i % nbuf]], 3, dw)
        gemm = (cout, ci * 27, vox)
    else:
        raise ValueError(op)
    lib = None
    if library:
        torch.backends.cudnn.benchmark = True
        wc = w.to(torch.bfloat16).contiguous(memory_format=torch.channels_last_3d)
        xc = [x.permute(0, 4, 1, 2, 3) for x in xs]
        gc = [g.permute(0, 4, 1, 2, 3) for g in gys]
        if op == "conv_fwd":
            lib = lambda i: F.conv3d(xc[i % nbuf], wc, padding=1)
        else:
            mask = [True, False, False] if op == "conv_dgrad" else [False, True, False]
            lib = lambda i: torch.ops.aten.convolution_backward(gc[i % nbuf], xc[i % nbuf], wc, None, [1, 1, 1],
                                                                [1, 1, 1], [1, 1, 1], False, [0, 0, 0], 1, mask)
    return Case(op, f"{cin}->{cout} @{size}^3 n{batch}", ours, lib, flops=flops, gemm=gemm)


def convT_case(op: str, cin: int, cout: int, size: int, batch: int, library: bool = True) -> Case:
    """k2s2 transposed convolution on a coarse grid of ``size``^3 (output 2*size)."""
    dev = "cuda"
    n, s = batch, size
    nbuf = _copies(n * (2 * s) ** 3 * cout * 2)
    xs = _rot(nbuf, lambda: torch.randn(n, s, s, s, cin, device=dev).to(torch.bfloat16))
    w = torch.randn(cin, cout, 2, 2, 2, device=dev) * 0.05
    b = torch.randn(cout, device=dev)
    nbytes = n * s ** 3 * cin * 2 + n * (2 * s) ** 3 * cout * 2
    if op == "convT_fwd":
        wp = ck.pack_weight_convT_fwd(w)
        ours = lambda i: ck.convT_fwd(xs[i % nbuf], wp, cout, b)
    elif op == "convT_dgrad":
        gys = _rot(nbuf, lambda: torch.randn(n, 2 * s, 2 * s, 2 * s, cout, device=dev).to(torch.bfloat16))
        wp = ck.pack_weight_convT_dgrad(w)
        ours = lambda i: ck.convT_dgrad(gys[i % nbuf], wp, cin)
    else:
        raise ValueError(op)
    lib = None
    if library:
        wc, bc = w.to(torch.bfloat16), b.to(torch.bfloat16)
        if op == "convT_fwd":
            xc = [x.permute(0, 4, 1, 2, 3) for x in xs]
            lib = lambda i: F.conv_transpose3d(xc[i % nbuf], wc, bc, stride=2)
        else:
            gc = [g.permute(0, 4, 1, 2, 3) for g in gys]
            lib = lambda i: F.conv3d(gc[i % nbuf], wc, stride=2)  # the adjoint of the k2s2 transposed convolution
    return Case(op, f"{cin}->{cout} @{size}^3 n{batch}", ours, lib, bytes=float(nbytes))


def gn_case(op: str, channels: int, size: int, batch: int, library: bool = True) -> Case:
    dev = "cuda"
    c, n, s = channels, batch, size
    nbuf = _copies(n * s ** 3 * c * 2)
    xs = _rot(nbuf, lambda: torch.randn(n, s, s, s, c, device=dev).to(torch.bfloat16))
    dys = _rot(nbuf, lambda: torch.randn(n, s, s, s, c, device=dev).to(torch.bfloat16))
    w, b = torch.randn(c, device=dev), torch.randn(c, device=dev)
    stats = [gk.gn_forward(x, w, b, 8)[1:] for x in xs]
    vol = n * s ** 3 * c * 2
    if op == "gn_fwd":
        ours = lambda i: gk.gn_forward(xs[i % nbuf], w, b, 8)
        nbytes = 3 * vol
    else:
        ours = lambda i: gk.gn_backward(dys[i % nbuf], xs[i % nbuf], w, b, *stats[i % nbuf], 8)
        nbytes = 5 * vol
    lib = None
    if library:
        wb, bb = w.to(torch.bfloat16), b.to(torch.bfloat16)
        xc = [x.permute(0, 4, 1, 2, 3).detach().requires_grad_(op == "gn_bwd") for x in xs]
        if op == "gn_fwd":
            lib = lambda i: F.relu(F.group_norm(xc[i % nbuf], 8, wb, bb))
        else:
            dyc = [d.permute(0, 4, 1, 2, 3) for d in dys]

            def lib(i):  # the library number includes its forward pass
                xc[i % nbuf].grad = None
                F.relu(F.group_norm(xc[i % nbuf], 8, wb, bb)).backward(dyc[i % nbuf])
    return Case(op, f"C={c} @{size}^3 n{batch}", ours, lib, bytes=float(nbytes))


def loss_case(n_classes: int, size: int, batch: int, library: bool = True) -> Case:
    dev = "cuda"
    c, n, s = n_classes, batch, size
    cp = (c + 15) // 16 * 16
    lg = torch.randn(n, s, s, s, cp, device=dev).to(torch.bfloat16)
    lab = torch.randint(0, c, (n, s, s, s), device=dev, dtype=torch.int16)

    def ours(i):
        t = lg.detach().requires_grad_(True)
        L.segmentation_loss_fused(t, lab, c)[0].backward()
    nbytes = lg.numel() * 2 * 3 + lab.numel() * 2 * 2
    lib = None
    if library:
        lr = lg[..., :c].permute(0, 4, 1, 2, 3)

        def lib(i):
            t = lr.detach().requires_grad_(True)
            L.segmentation_loss_reference(t, lab.long(), c)[0].backward()
    return Case("loss", f"{c} classes @{size}^3 n{batch}", ours, lib, bytes=float(nbytes))


def adam_case(millions: int) -> Case:
    from ..ops.optim import FusedClipAdam
    numel = millions * 1_000_000
    p = torch.nn.Parameter(torch.randn(numel, device="cuda"))
    opt = FusedClipAdam([p], lr=1e-3)
    opt.attach()
    p.grad.normal_()
    q = torch.nn.Parameter(p.detach().clone())
    q.grad = p.grad.detach().clone()
    ref = torch.optim.Adam([q], lr=1e-3, fused=True)

    def lib(i):
        torch.nn.utils.clip_grad_norm_([q], 1.0)
        ref.step()
    # the norm pass reads g; the update reads p, g, m, v and writes p, m, v
    return Case("adam", f"{millions}M parameters", lambda i: opt.step(), lib, bytes=float(numel * 4 * 8))


def pool_case(op: str, channels: int, size: int, batch: int, library: bool = True) -> Case:
    from ..ops import pool_kernels as pk
    dev = "cuda"
    c, n, s = channels, batch, size
    nbuf = _copies(n * s ** 3 * c * 2)
    xs = _rot(nbuf, lambda: torch.randn(n, s, s, s, c, device=dev).to(torch.bfloat16))
    vol = n * s ** 3 * c * 2
    # the pair the module runs: forward also writes one index byte per output element, backward reads gy + indices
    if op == "pool_fwd":
        ours = lambda i: pk.maxpool2_fwd_idx(xs[i % nbuf])
        nbytes = vol + vol // 8 + vol // 16
        lib = (lambda i: F.max_pool3d(xs[i % nbuf].permute(0, 4, 1, 2, 3), 2)) if library else None
    else:
        pairs = [pk.maxpool2_fwd_idx(x) for x in xs]
        gys = [torch.randn_like(y) for y, _ in pairs]
        shape = tuple(xs[0].shape)
        ours = lambda i: pk.maxpool2_bwd_idx(gys[i % nbuf], pairs[i % nbuf][1], shape)
        nbytes = vol + vol // 8 + vol // 16
        lib = None
    return Case(op, f"C={c} @{size}^3 n{batch}", ours, lib, bytes=float(nbytes))
