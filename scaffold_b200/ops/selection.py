"""Start-up report: which kernel every layer of a model runs, and which fused channels are live.

``kernel_selection(model, batch, local_dims)`` walks a shape-only copy of the network (meta
tensors: no memory, no launches) and lists, per convolution / normalisation / pooling layer, the
input shape it will see on this rank and the sm_100a kernel each direction routes to
(:meth:`scaffold_b200.analysis.shapes.ConvProblem.route` mirrors the dispatch of ``sb_conv_fwd`` /
``sb_conv_wgrad``). ``format_selection`` renders the table that the trainer logs once before
the first step together with the state of the three peer-memory channels (halo, GroupNorm
statistics, gradient all-reduce), so a run's log says what actually executes.

Role of the reference: ``kernel_selection`` / ``format_kernel_selection``
(ScaFFold/unet/_rungs.py:409-463) and the trainer's start-up log (ScaFFold/utils/trainer.py:808-830).
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import torch
import torch.nn as nn

from ..analysis.shapes import ConvProblem
from . import conv_kernels as ck
from .conv3d import Conv3d, ConvTranspose3d
from .group_norm import GroupNorm
from .pool import MaxPool3d


def _halo_mode(conv: Conv3d, spatial, src_c: Sequence[int], dims) -> str:
    if spatial is None or spatial.size == 1 or conv.kernel_size[0] != 3:
        return "-"
    d, h, w = dims
    chan = getattr(spatial, "halo_channel", None)
    if (chan is not None and h >= 8 and w >= 16 and d >= 2 and conv.bias is None and conv.out_channels % 32 == 0
            and all(c % 16 == 0 for c in src_c)):
        return "fused(" + ",".join("DHW"[a - 2] for a in spatial.dims) + ")"
    return "nccl slabs"


def kernel_selection(model: nn.Module, batch: int, local_dims: Sequence[int], spatial=None) -> List[Dict[str, str]]:
    """One row per kernel-backed layer, in execution order."""
    rows: List[Dict[str, str]] = []
    names = {m: n for n, m in model.named_modules()}
    split_first = set()  # first convolution of a decoder block reads (skip, upsampled) as two sources
    for m in model.modules():
        if hasattr(m, "up") and hasattr(m, "conv") and isinstance(getattr(m, "up"), ConvTranspose3d):
            split_first.add(m.conv.double_conv[0])
    hooks = []

    def conv_hook(mod, args):
        x = args[0]
        n, c, d, h, w = x.shape
        if isinstance(mod, ConvTranspose3d):
            p = ConvProblem(n, mod.in_channels, mod.out_channels, (d, h, w), kernel=2, transposed=True)
            halo = "-"
        else:
            split = (c // 2, c - c // 2) if mod in split_first else None
            p = ConvProblem(n, c, mod.out_channels, (d, h, w), kernel=mod.kernel_size[0], split_cin=split)
            halo = _halo_mode(mod, spatial, split or (p.kernel_variant().cin,), (d, h, w))
        fwd, dgrad = p.route("fwd", ck.PAIR_CONV), p.route("dgrad", ck.PAIR_CONV)
        if not p.transposed and c < 16:
            # the stem: its forward pass reads a copy padded to 32 channels, and the network input needs no gradient
            fwd = ConvProblem(n, 32, mod.out_channels, (d, h, w), kernel=p.kernel).route("fwd") + " (32-ch padded input)"
            dgrad = "-"
        rows.append({"layer": names[mod], "op": f"conv{'T' if p.transposed else ''} k{p.kernel} {p.cin}->{p.cout}",
                     "input": f"{n}x{d}x{h}x{w}", "fwd": fwd, "dgrad": dgrad,
                     "wgrad": p.route("wgrad"), "halo": halo})

    def gn_hook(mod, args):
        n, c, d, h, w = args[0].shape
        k = "gn_stats+gn_apply" if mod.kernel_supported() else "ATen (outside the kernels' channel range)"
        stats = "-"
        if spatial is not None and spatial.size > 1:
            stats = ("peer memory" if getattr(spatial, "stats_channel", None) is not None else "nccl all_gather") \
                if spatial.gn_global else "per shard"
        rows.append({"layer": names[mod], "op": f"GroupNorm({mod.num_groups}){'+ReLU' if mod.activation else ''} C={c}",
                     "input": f"{n}x{d}x{h}x{w}", "fwd": k, "dgrad": "gn_bwd_partial+gn_bwd_dx" if mod.kernel_supported()
                     else "ATen", "wgrad": "-", "halo": stats})

    def pool_hook(mod, args):
        n, c, d, h, w = args[0].shape
        rows.append({"layer": names[mod], "op": f"MaxPool3d(2) C={c}", "input": f"{n}x{d}x{h}x{w}",
                     "fwd": "maxpool2_fwd", "dgrad": "maxpool2_bwd", "wgrad": "-", "halo": "-"})

    for m in model.modules():
        if isinstance(m, (Conv3d, ConvTranspose3d)):
            hooks.append(m.register_forward_pre_hook(conv_hook))
        elif isinstance(m, GroupNorm):
            hooks.append(m.register_forward_pre_hook(gn_hook))
        elif isinstance(m, MaxPool3d):
            hooks.append(m.register_forward_pre_hook(pool_hook))
    try:
        _shape_walk(model, batch, local_dims)
    finally:
        for h in hooks:
            h.remove()
    return rows


def _shape_walk(model: nn.Module, batch: int, local_dims: Sequence[int]) -> None:
    """Run the model's forward on meta tensors: shapes only. Parameters are swapped for meta views
    for the duration of the call, so nothing is copied and no kernel launches."""
    from torch.func import functional_call
    meta = {k: torch.empty_like(v, device="meta") for k, v in list(model.named_parameters()) + list(model.named_buffers())}
    n_in = getattr(model, "n_channels", 3)
    x = torch.empty((batch, n_in, *local_dims), device="meta")
    saved = [(m, m._spatial) for m in model.modules() if getattr(m, "_spatial", None) is not None]
    for m, _ in saved:
        m._spatial = None  # the walk must not communicate
    try:
        with torch.no_grad():
            functional_call(model, meta, (x,))
    finally:
        for m, s in saved:
            m._spatial = s


def format_selection(rows: List[Dict[str, str]], channels: Optional[Dict[str, str]] = None) -> str:
    cols = ["layer", "op", "input", "fwd", "dgrad", "wgrad", "halo"]
    head = dict(zip(cols, ["layer", "operation", "local input", "forward", "backward-data", "weight-grad",
                           "halo / stats"]))
    width = {c: max(len(head[c]), *(len(r[c]) for r in rows)) if rows else len(head[c]) for c in cols}
    lines = ["  ".join(head[c].ljust(width[c]) for c in cols), "  ".join("-" * width[c] for c in cols)]
    lines += ["  ".join(r[c].ljust(width[c]) for c in cols) for r in rows]
    if channels:
        lines.append("")
        lines += [f"{k}: {v}" for k, v in channels.items()]
    return "\n".join(lines)


def effective_backends(engine) -> Dict[str, str]:
    """What actually runs (not what was asked for): the three peer-memory channels of a training engine."""
    sp = engine.spatial
    world = engine.layout.world_size if engine.layout is not None else 1
    red = engine.reducer
    out = {
        "grad_allreduce_effective": "none" if world == 1 else ("fused" if red._fused is not None else "nccl"),
        "grad_overlap_effective": "on" if red._buckets is not None else "off",
        "halo_exchange_effective": "none" if sp is None or sp.size == 1 else
        ("fused" if sp.halo_channel is not None else "nccl"),
        "gn_stats_effective": "local" if sp is None or sp.size == 1 else
        ("per_shard" if not sp.gn_global else ("peer" if sp.stats_channel is not None else "nccl")),
    }
    return out
