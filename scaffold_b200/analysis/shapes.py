"""Shape and cost model of the convolutions this framework runs (no torch needed).

``ConvProblem`` describes one convolution the way the kernels see it and answers: how many FLOPs and
bytes per direction, the arithmetic intensity, the implicit-GEMM shape, the time a B200 needs at the
measured roofs, and which kernel ``sb_conv_fwd`` / ``sb_conv_wgrad`` route it to. Corpora list the
problems of a U-Net configuration in three forms: *logical* (the layer as the model defines it),
*sharded* (what one rank of a spatially split run computes, halo included) and *kernel* (channels
padded to what the kernels take). ``edge_cases`` are the odd shapes the tests sweep.

Role of the reference: triton_conv3d/shapes.py:110-756 (ConvProblem, corpora, edge cases), with the
MI300A roofs replaced by this machine's measured peaks (``MEASURED_PEAKS.json`` at the repository root:
cuBLAS bf16 burst and STREAM-style copy; fallback 1590 TFLOP/s and 6650 GB/s).
"""
from __future__ import annotations

import json
from dataclasses import dataclass, replace
from pathlib import Path
from typing import Dict, Iterator, Optional, Sequence, Tuple

from .unet_shapes import ShardSpec, trace_unet

Direction = str  # "fwd" | "dgrad" | "wgrad"
FALLBACK_TFLOPS, FALLBACK_GBS = 1590.0, 6650.0


def measured_peaks() -> Tuple[float, float, str]:
    """(bf16 TFLOP/s, copy GB/s, 'measured' | 'fallback')."""
    p = Path(__file__).resolve().parents[2] / "MEASURED_PEAKS.json"
    try:
        d = json.loads(p.read_text())
        return float(d["bf16_tflops"]), float(d["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_TFLOPS, FALLBACK_GBS, "fallback"


def _pad(v: int, m: int = 16) -> int:
    return (v + m - 1) // m * m


@dataclass(frozen=True)
class ConvProblem:
    n: int
    cin: int
    cout: int
    spatial: Tuple[int, int, int]          # input extents (D, H, W)
    kernel: int = 3
    transposed: bool = False               # k2s2 transposed convolution when True
    halo: Tuple[int, int, int] = (0, 0, 0)  # input carries this many extra voxels per side (sharded run)
    split_cin: Optional[Tuple[int, int]] = None  # two concatenated sources (decoder blocks)
    name: str = ""

    # -- shapes ------------------------------------------------------------------
    @property
    def out_spatial(self) -> Tuple[int, int, int]:
        if self.transposed:
            return tuple(2 * v for v in self.spatial)
        return tuple(v - 2 * h for v, h in zip(self.spatial, self.halo))

    @property
    def input_shape(self):
        return (self.n, self.cin, *self.spatial)

    @property
    def output_shape(self):
        return (self.n, self.cout, *self.out_spatial)

    @property
    def weight_shape(self):
        k = self.kernel
        return (self.cin, self.cout, k, k, k) if self.transposed else (self.cout, self.cin, k, k, k)

    @property
    def taps(self) -> int:
        return self.kernel ** 3

    def _vox(self, spatial) -> int:
        return self.n * spatial[0] * spatial[1] * spatial[2]

    # -- cost ----------------------------------------------------------------------
    def flops(self, direction: Direction = "fwd") -> int:
        """Multiply-adds x 2; the same count for every direction (each is one pass over voxels x Cin x Cout x taps)."""
        vox = self._vox(self.spatial if self.transposed else self.out_spatial)
        return 2 * vox * self.cin * self.cout * self.taps

    def bytes(self, direction: Direction = "fwd", elem: int = 2) -> int:
        """Algorithmic traffic: each operand read once, the result written once (bf16 activations)."""
        x = self._vox(self.spatial) * self.cin * elem
        y = self._vox(self.out_spatial) * self.cout * elem
        w = self.cin * self.cout * self.taps
        if direction == "fwd":
            return x + y + w * elem
        if direction == "dgrad":
            return y + x + w * elem
        return x + y + w * 4  # weight gradient is fp32

    def arithmetic_intensity(self, direction: Direction = "fwd") -> float:
        return self.flops(direction) / self.bytes(direction)

    def roofline_seconds(self, direction: Direction = "fwd") -> float:
        tf, gbs, _ = measured_peaks()
        return max(self.flops(direction) / (tf * 1e12), self.bytes(direction) / (gbs * 1e9))

    def efficiency(self, ms: float, direction: Direction = "fwd") -> float:
        """Fraction of the roofline a measured time reaches."""
        return self.roofline_seconds(direction) / (ms * 1e-3)

    def gemm_shape(self, direction: Direction = "fwd") -> Tuple[int, int, int]:
        """(M, N, K) of the implicit GEMM the kernels run."""
        vox_out = self._vox(self.out_spatial)
        if self.transposed:
            vox_in = self._vox(self.spatial)
            if direction == "fwd":
                return vox_in, 8 * self.cout, self.cin
            if direction == "dgrad":
                return vox_in, self.cin, 8 * self.cout
            return self.cin, 8 * self.cout, vox_in
        if direction == "fwd":
            return vox_out, self.cout, self.cin * self.taps
        if direction == "dgrad":
            return self._vox(self.spatial), self.cin, self.cout * self.taps
        return self.cout, self.cin * self.taps, vox_out

    # -- limits and routing ---------------------------------------------------------
    @property
    def max_elements(self) -> int:
        return max(self._vox(self.spatial) * _pad(self.cin), self._vox(self.out_spatial) * _pad(self.cout))

    @property
    def index_exceeds_int32(self) -> bool:
        """True when an element offset does not fit 31 bits (the kernels index voxels with 64-bit integers)."""
        return self.max_elements >= 2 ** 31

    def kernel_variant(self) -> "ConvProblem":
        """Channels as the kernels see them: padded to multiples of 16."""
        sc = None if self.split_cin is None else tuple(_pad(c) for c in self.split_cin)
        cin = sum(sc) if sc else _pad(self.cin)
        return replace(self, cin=cin, cout=_pad(self.cout), split_cin=sc)

    def route(self, direction: Direction = "fwd", pair: bool = True) -> str:
        """Name of the kernel that runs this problem (mirrors the dispatch in csrc/conv_igemm.cu / conv_wgrad.cu);
        ``pair=False`` gives the routing with the two-SM kernel switched off."""
        k = self.kernel_variant()
        d, h, w = k.out_spatial if direction != "dgrad" else k.spatial
        if self.transposed:
            return {"fwd": "igemm(scatter)", "dgrad": "igemm(strided)", "wgrad": "wgrad(generic)"}[direction]
        if self.kernel == 1:
            return "wgrad(generic)" if direction == "wgrad" else "igemm"
        big = w >= 16 and h >= 8
        rows_, kk_ = (k.cout, k.cin) if direction == "fwd" else (k.cin, k.cout)
        if (direction != "wgrad" and h == 8 and w == 8 and d % 2 == 0 and 2 <= d <= 8 and rows_ % 128 == 0
                and not k.split_cin and not any(self.halo)):
            return "conv_small"
        if direction == "wgrad":
            return "wgrad_plane" if big else "wgrad(generic)"
        rows, kk = (k.cout, k.cin) if direction == "fwd" else (k.cin, k.cout)
        first = (k.split_cin[0] if (k.split_cin and direction == "fwd") else kk)
        if big and pair and rows >= 128 and rows % 128 == 0 and kk % 64 == 0 and first % 64 == 0:
            return "conv_plane2(pair)"  # two-SM cta_group::2 kernel, with or without a fused halo
        if big and (rows <= 64 or rows % 64 == 0) and kk % 32 == 0 and first % 32 == 0:
            return "conv_plane3"
        return "conv_plane" if big else "igemm"

    @property
    def label(self) -> str:
        t = "T" if self.transposed else ""
        return f"{self.cin}->{self.cout} k{self.kernel}{t} @{'x'.join(map(str, self.spatial))} n{self.n}"


# ----------------------------------------------------------------------------------
# corpora
# ----------------------------------------------------------------------------------
def scaffold_corpus(problem_scale: int = 7, unet_bottleneck_dim: int = 3, batch: int = 2, n_categories: int = 8,
                    base_width: int = 64, shards: Sequence[int] = (1, 1, 1)) -> Tuple[ConvProblem, ...]:
    """Every convolution of the U-Net, logical form on one rank's sub-volume (halo'd when sharded)."""
    tr = trace_unet(problem_scale, unet_bottleneck_dim, batch, n_categories, 3, 8, shards, (2, 3, 4), base_width)
    spec = ShardSpec(tuple(shards))
    out = []
    prev = None
    for o in tr.ops:
        sp = o.local_in[2:]
        if o.kind == "conv3":
            halo = tuple(1 if s > 1 else 0 for s in spec.shards)
            sp_in = tuple(v + 2 * hh for v, hh in zip(sp, halo))
            split = None
            if prev is not None and prev.kind == "concat":
                split = (o.in_channels // 2, o.in_channels - o.in_channels // 2)
            out.append(ConvProblem(o.local_in[0], o.in_channels, o.out_channels, sp_in, 3, False, halo, split, o.name))
        elif o.kind == "convT":
            out.append(ConvProblem(o.local_in[0], o.in_channels, o.out_channels, sp, 2, True, name=o.name))
        elif o.kind == "conv1":
            out.append(ConvProblem(o.local_in[0], o.in_channels, o.out_channels, sp, 1, name=o.name))
        prev = o
    return tuple(out)


def halo_corpus(problem_scale: int = 7, batch: int = 2) -> Tuple[ConvProblem, ...]:
    """The same layers as seen by one rank of a [2,1,1] and a [2,2,1] split."""
    return scaffold_corpus(problem_scale, 3, batch, shards=(2, 1, 1)) + scaffold_corpus(problem_scale, 3, batch,
                                                                                         shards=(2, 2, 1))


def edge_cases(include_large: bool = False) -> Tuple[ConvProblem, ...]:
    """Odd shapes: ragged extents, tiny volumes, channel counts off the tile sizes, one-plane volumes."""
    cases = [
        ConvProblem(1, 3, 64, (4, 16, 16), name="stem, 3 input channels"),
        ConvProblem(1, 64, 64, (3, 12, 20), name="ragged H and W"),
        ConvProblem(2, 64, 64, (7, 24, 48), name="ragged D, W = 3 tiles"),
        ConvProblem(1, 64, 64, (1, 8, 16), name="single plane"),
        ConvProblem(1, 32, 32, (3, 12, 20), name="32 channels"),
        ConvProblem(1, 128, 48, (9, 16, 16), split_cin=(32, 96), name="48 outputs, uneven concat"),
        ConvProblem(2, 64, 128, (4, 4, 4), name="volume below one tile"),
        ConvProblem(1, 512, 128, (8, 8, 8), name="bottleneck-like"),
        ConvProblem(1, 64, 9, (2, 16, 16), 1, name="1x1x1 head, 9 classes"),
        ConvProblem(1, 128, 64, (4, 8, 16), 2, True, name="k2s2 transposed"),
        ConvProblem(1, 64, 64, (6, 16, 16), halo=(1, 0, 0), name="depth halo"),
        ConvProblem(1, 64, 64, (6, 18, 18), halo=(1, 1, 1), name="halo on all axes"),
    ]
    if include_large:
        cases.append(ConvProblem(2, 64, 64, (512, 512, 512), name="scale 9 stem level: offsets beyond 2^31"))
    return tuple(cases)


def all_problems(include_large: bool = False) -> Iterator[ConvProblem]:
    yield from scaffold_corpus()
    yield from halo_corpus()
    yield from edge_cases(include_large)


def summarize(problems: Sequence[ConvProblem]) -> Dict[str, float]:
    """Roofline time of a training step's convolutions (all three directions), in milliseconds."""
    total = {"fwd": 0.0, "dgrad": 0.0, "wgrad": 0.0}
    for p in problems:
        for d in total:
            total[d] += p.roofline_seconds(d) * 1e3
    total["all"] = sum(total.values())
    return total


def main(argv=None) -> int:
    """``python -m scaffold_b200.analysis.shapes [--problem-scale 7 --batch 2 --dc-num-shards 2 1 1]``: the corpus
    of one configuration with FLOPs, arithmetic intensity, roofline time and the kernel each direction runs on."""
    import argparse
    ap = argparse.ArgumentParser(description="Convolution corpus of a U-Net configuration with roofline and routing")
    ap.add_argument("--problem-scale", type=int, default=7)
    ap.add_argument("--unet-bottleneck-dim", type=int, default=3)
    ap.add_argument("--batch", type=int, default=2)
    ap.add_argument("--n-categories", type=int, default=8)
    ap.add_argument("--base-width", type=int, default=64)
    ap.add_argument("--dc-num-shards", type=int, nargs=3, default=[1, 1, 1])
    a = ap.parse_args(argv)
    tf, gbs, which = measured_peaks()
    print(f"roofs ({which}): {tf:.0f} TFLOP/s bf16, {gbs:.0f} GB/s")
    probs = scaffold_corpus(a.problem_scale, a.unet_bottleneck_dim, a.batch, a.n_categories, a.base_width,
                            tuple(a.dc_num_shards))
    print(f"{'layer':34s} {'problem':40s} {'GFLOP':>8s} {'AI':>7s} {'roof ms':>8s}  fwd / dgrad / wgrad kernels")
    for p in probs:
        print(f"{p.name:34s} {p.label:40s} {p.flops() / 1e9:8.1f} {p.arithmetic_intensity():7.0f} "
              f"{p.roofline_seconds() * 1e3:8.3f}  {p.route('fwd')} / {p.route('dgrad')} / {p.route('wgrad')}")
    tot = summarize(probs)
    print(f"roofline of one step's convolutions: fwd {tot['fwd']:.2f} + dgrad {tot['dgrad']:.2f} + wgrad "
          f"{tot['wgrad']:.2f} = {tot['all']:.2f} ms")
    return 0


if __name__ == "__main__":
    import sys
    sys.exit(main())
