"""Tensor-core ceiling at a convolution's implied GEMM shape.

For an implicit GEMM (M, N, K) = (voxels, Cout, Cin * 27) the question "how fast could a kernel be if the
operand gather cost nothing" has two answers, both measured here on the same machine:

* ``ours``: this framework's own tcgen05 pipeline on a plain GEMM of that shape, a 1x1x1 convolution over
  M voxels with K input and N output channels (``csrc/conv_igemm.cu``): no halo, no taps;
* ``library``: cuBLAS through ``torch.matmul`` on bf16 operands of the same (M, N, K).

A 3x3x3 kernel that reaches the first number has hidden its gather completely.

Role of the reference: triton_conv3d/bench/gemm_probe.py:65-153 (matrix-core ceiling at conv-implied shapes).
"""
from __future__ import annotations

import torch

from ..ops import conv_kernels as ck
from .cases import Case, _copies, _rot


MAX_M = 1 << 19  # rows of the probe: enough tiles to fill the machine; the ceiling does not move beyond this


def gemm_case(m: int, n: int, k: int, library: bool = True) -> Case:
    """M voxels x K channels -> N channels. K and N are rounded up to multiples of 16; M is capped at
    ``MAX_M`` and rounded to whole 64 x 64 planes (the activation is a [1, M/4096, 64, 64, K] volume)."""
    k16, n16 = (k + 15) // 16 * 16, (n + 15) // 16 * 16
    m = max(4096, min(m, MAX_M) // 4096 * 4096)
    nbuf = _copies(m * k16 * 2)
    a = _rot(nbuf, lambda: torch.randn(1, m // 4096, 64, 64, k16, device="cuda").to(torch.bfloat16))
    w = torch.randn(n16, k16, 1, 1, 1, device="cuda") * 0.05
    wp = ck.pack_weight_fwd(w)
    ours = lambda i: ck.conv_same([a[i % nbuf]], wp, 1, [n16])
    lib = None
    if library:
        b = w.reshape(n16, k16).to(torch.bfloat16).t().contiguous()
        a2 = [t.reshape(m, k16) for t in a]
        lib = lambda i: torch.matmul(a2[i % nbuf], b)
    return Case("gemm", f"M={m} N={n16} K={k16}", ours, lib, flops=2.0 * m * n16 * k16, gemm=(m, n16, k16))
