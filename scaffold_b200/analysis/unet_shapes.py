"""Symbolic shape calculator of the 3-D U-Net (standard library only).

``trace_unet`` walks the network of ``scaffold_b200.models.unet.UNet`` for any problem scale,
bottleneck, batch size and spatial shard layout and lists every operation with its global shape, its
per-rank (local) shape, the halo'd shape a sharded 3x3x3 convolution reads, parameter counts per block,
forward FLOPs and the number of halo exchanges per step. It mirrors what the reference's calculator
reports (model-analysis/unet_shapes.py:56-663) for this implementation's layout rules: depth, height
and width are split over ``dc_num_shards`` (one entry per ``dc_shard_dims`` axis), channels never.

    python -m scaffold_b200.analysis.unet_shapes --problem-scale 7 --unet-bottleneck-dim 3 \\
        --local-batch-size 2 --dc-num-shards 2 1 1 [--json]
"""
from __future__ import annotations

import argparse
import json
import sys
from dataclasses import asdict, dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

Shape = Tuple[int, ...]


@dataclass(frozen=True)
class ShardSpec:
    """Number of shards along each of (D, H, W)."""
    shards: Tuple[int, int, int] = (1, 1, 1)

    @staticmethod
    def from_config(num_shards: Sequence[int], shard_dims: Sequence[int] = (2, 3, 4)) -> "ShardSpec":
        s = [1, 1, 1]
        for n, d in zip(num_shards, shard_dims):
            if d not in (2, 3, 4):
                raise ValueError(f"dc_shard_dims entries must be 2, 3 or 4 (D, H, W of NCDHW), got {d}")
            s[d - 2] = int(n)
        return ShardSpec(tuple(s))

    @property
    def total(self) -> int:
        return self.shards[0] * self.shards[1] * self.shards[2]

    def local(self, spatial: Sequence[int]) -> Tuple[int, int, int]:
        out = []
        for n, s in zip(spatial, self.shards):
            if n % s != 0:
                raise ValueError(f"extent {n} is not divisible by {s} shards")
            out.append(n // s)
        return tuple(out)

    def halo(self, spatial: Sequence[int], width: int) -> Tuple[int, int, int]:
        """Local extent plus ``width`` on both sides of every split axis."""
        return tuple(n + (2 * width if s > 1 else 0) for n, s in zip(self.local(spatial), self.shards))


@dataclass
class Op:
    name: str
    kind: str                      # conv3 | convT | conv1 | group_norm | max_pool | concat | loss
    block: str
    in_channels: int
    out_channels: int
    global_in: Shape               # (N, C, D, H, W)
    global_out: Shape
    local_in: Shape
    local_out: Shape
    halo_in: Optional[Shape] = None   # what a sharded 3x3x3 convolution reads
    params: int = 0
    flops_fwd: int = 0
    halo_exchanges: int = 0        # per forward pass (backward mirrors each with one gradient exchange)
    halo_bytes: int = 0            # bytes this rank sends per forward exchange (bf16)


@dataclass
class Trace:
    config: Dict[str, object]
    ops: List[Op] = field(default_factory=list)

    @property
    def params(self) -> int:
        return sum(o.params for o in self.ops)

    @property
    def flops_fwd(self) -> int:
        return sum(o.flops_fwd for o in self.ops)

    @property
    def halo_exchanges_fwd(self) -> int:
        return sum(o.halo_exchanges for o in self.ops)

    def params_per_block(self) -> Dict[str, int]:
        out: Dict[str, int] = {}
        for o in self.ops:
            out[o.block] = out.get(o.block, 0) + o.params
        return out

    def activation_bytes_local(self, elem: int = 2) -> int:
        """bf16 bytes of every op output on one rank (what a step keeps for backward, upper bound)."""
        total = 0
        for o in self.ops:
            n = 1
            for v in o.local_out:
                n *= v
            total += n * elem
        return total


class Tracer:
    def __init__(self, batch: int, shard: ShardSpec, groups: int):
        self.batch, self.shard, self.groups = batch, shard, groups
        self.ops: List[Op] = []

    def _shapes(self, c: int, spatial):
        return (self.batch, c, *spatial), (self.batch, c, *self.shard.local(spatial))

    def conv3(self, name, block, cin, cout, spatial):
        gi, li = self._shapes(cin, spatial)
        go, lo = self._shapes(cout, spatial)
        split_axes = sum(1 for s in self.shard.shards if s > 1)
        hl = self.shard.halo(spatial, 1)
        face = 0
        for ax, s in enumerate(self.shard.shards):
            if s > 1:
                other = 1
                for j, v in enumerate(self.shard.local(spatial)):
                    if j != ax:
                        other *= v
                face += 2 * other
        vox = self.batch * spatial[0] * spatial[1] * spatial[2]
        self.ops.append(Op(name, "conv3", block, cin, cout, gi, go, li, lo,
                           halo_in=(self.batch, cin, *hl) if split_axes else None,
                           params=cin * cout * 27, flops_fwd=2 * vox * cin * cout * 27,
                           halo_exchanges=1 if split_axes else 0, halo_bytes=self.batch * cin * face * 2))

    def group_norm(self, name, block, c, spatial):
        g, l = self._shapes(c, spatial)
        self.ops.append(Op(name, "group_norm", block, c, c, g, g, l, l, params=2 * c))

    def pool(self, name, block, c, spatial):
        gi, li = self._shapes(c, spatial)
        half = tuple(v // 2 for v in spatial)
        go, lo = self._shapes(c, half)
        self.ops.append(Op(name, "max_pool", block, c, c, gi, go, li, lo))
        return half

    def convT(self, name, block, cin, cout, spatial):
        gi, li = self._shapes(cin, spatial)
        dbl = tuple(v * 2 for v in spatial)
        go, lo = self._shapes(cout, dbl)
        vox = self.batch * spatial[0] * spatial[1] * spatial[2]
        self.ops.append(Op(name, "convT", block, cin, cout, gi, go, li, lo, params=cin * cout * 8 + cout,
                           flops_fwd=2 * vox * cin * cout * 8))
        return dbl

    def concat(self, name, block, c_skip, c_up, spatial):
        gi, li = self._shapes(c_skip + c_up, spatial)
        self.ops.append(Op(name, "concat", block, c_skip + c_up, c_skip + c_up, gi, gi, li, li))

    def conv1(self, name, block, cin, cout, spatial):
        gi, li = self._shapes(cin, spatial)
        go, lo = self._shapes(cout, spatial)
        vox = self.batch * spatial[0] * spatial[1] * spatial[2]
        self.ops.append(Op(name, "conv1", block, cin, cout, gi, go, li, lo, params=cin * cout + cout,
                           flops_fwd=2 * vox * cin * cout))

    def double_conv(self, block, cin, cout, spatial):
        self.conv3(f"{block}.double_conv.0", block, cin, cout, spatial)
        self.group_norm(f"{block}.double_conv.1", block, cout, spatial)
        self.conv3(f"{block}.double_conv.3", block, cout, cout, spatial)
        self.group_norm(f"{block}.double_conv.4", block, cout, spatial)


def trace_unet(problem_scale: int = 7, unet_bottleneck_dim: int = 3, local_batch_size: int = 1,
               n_categories: int = 5, n_channels: int = 3, group_norm_groups: int = 8,
               dc_num_shards: Sequence[int] = (1, 1, 1), dc_shard_dims: Sequence[int] = (2, 3, 4),
               base_width: int = 64) -> Trace:
    layers = problem_scale - unet_bottleneck_dim
    if layers < 1:
        raise ValueError("problem_scale must be strictly greater than unet_bottleneck_dim")
    shard = ShardSpec.from_config(dc_num_shards, dc_shard_dims)
    size = 2 ** problem_scale
    spatial = (size, size, size)
    bottleneck = tuple(v >> layers for v in spatial)
    for ext, s in zip(bottleneck, shard.shards):
        if ext % s != 0 or ext // s < 1:
            raise ValueError(f"bottleneck extent {ext} cannot be split into {s} shards")
    t = Tracer(local_batch_size, shard, group_norm_groups)
    c = base_width
    t.double_conv("down_list.0", n_channels, c, spatial)
    skips = [(c, spatial)]
    for i in range(1, layers + 1):
        blk = f"down_list.{i}"
        spatial = t.pool(f"{blk}.maxpool_conv.0", blk, c, spatial)
        t.double_conv(f"{blk}.maxpool_conv.1", c, 2 * c, spatial)
        t.ops[-4].block = t.ops[-3].block = t.ops[-2].block = t.ops[-1].block = blk
        c *= 2
        skips.append((c, spatial))
    skips.pop()
    for i in range(layers):
        blk = f"up_list.{i}"
        c_skip, sp_skip = skips.pop()
        spatial = t.convT(f"{blk}.up", blk, c, c // 2, spatial)
        assert spatial == sp_skip
        t.concat(f"{blk}.concat", blk, c_skip, c // 2, spatial)
        t.double_conv(f"{blk}.conv", c, c // 2, spatial)
        for o in t.ops[-4:]:
            o.block = blk
        c //= 2
    t.conv1(f"up_list.{layers}.conv", f"up_list.{layers}", c, n_categories + 1, spatial)
    cfg = dict(problem_scale=problem_scale, unet_bottleneck_dim=unet_bottleneck_dim, layers=layers,
               local_batch_size=local_batch_size, n_classes=n_categories + 1, n_channels=n_channels,
               group_norm_groups=group_norm_groups, shards=list(shard.shards), base_width=base_width,
               volume=[size] * 3)
    return Trace(cfg, t.ops)


def fmt_shape(shape: Optional[Shape]) -> str:
    return "-" if shape is None else "x".join(str(v) for v in shape)


def print_report(trace: Trace, out=sys.stdout) -> None:
    cfg = trace.config
    print(f"U-Net scale {cfg['problem_scale']} ({cfg['layers']} levels below the stem), batch {cfg['local_batch_size']} "
          f"per replica, shards (D,H,W) = {tuple(cfg['shards'])}", file=out)
    print(f"{'op':38s} {'kind':10s} {'global out':22s} {'local out':22s} {'halo in':22s} {'params':>11s} {'GFLOP':>9s}",
          file=out)
    for o in trace.ops:
        print(f"{o.name:38s} {o.kind:10s} {fmt_shape(o.global_out):22s} {fmt_shape(o.local_out):22s} "
              f"{fmt_shape(o.halo_in):22s} {o.params:11d} {o.flops_fwd / 1e9:9.2f}", file=out)
    print(f"parameters: {trace.params:,}", file=out)
    for blk, n in trace.params_per_block().items():
        print(f"  {blk:14s} {n:12,}", file=out)
    print(f"forward GFLOP (global): {trace.flops_fwd / 1e9:.1f}; training step ~3x", file=out)
    print(f"halo exchanges per step: {trace.halo_exchanges_fwd} forward + {trace.halo_exchanges_fwd} backward", file=out)
    print(f"bf16 activations kept per rank (upper bound): {trace.activation_bytes_local() / 2**30:.2f} GiB", file=out)


def main(argv=None) -> int:
    p = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    p.add_argument("--problem-scale", type=int, default=7)
    p.add_argument("--unet-bottleneck-dim", type=int, default=3)
    p.add_argument("--local-batch-size", type=int, default=1)
    p.add_argument("--n-categories", type=int, default=5, help="n_classes = this + 1")
    p.add_argument("--n-channels", type=int, default=3)
    p.add_argument("--group-norm-groups", type=int, default=8)
    p.add_argument("--dc-num-shards", type=int, nargs="+", default=[1, 1, 1])
    p.add_argument("--dc-shard-dims", type=int, nargs="+", default=[2, 3, 4])
    p.add_argument("--unet-base-width", type=int, default=64)
    p.add_argument("--json", action="store_true")
    a = p.parse_args(argv)
    tr = trace_unet(a.problem_scale, a.unet_bottleneck_dim, a.local_batch_size, a.n_categories, a.n_channels,
                    a.group_norm_groups, a.dc_num_shards, a.dc_shard_dims, a.unet_base_width)
    if a.json:
        json.dump({"config": tr.config, "params": tr.params, "flops_fwd": tr.flops_fwd,
                   "halo_exchanges_fwd": tr.halo_exchanges_fwd, "ops": [asdict(o) for o in tr.ops]}, sys.stdout)
        print()
    else:
        print_report(tr)
    return 0


if __name__ == "__main__":
    sys.exit(main())
