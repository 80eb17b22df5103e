"""Thin Python launchers of the tcgen05 convolution kernels.

All tensors here are *voxel-major* views: activations ``[N, D, H, W, C]`` bf16
contiguous (the memory of an NCDHW ``channels_last_3d`` tensor), packed
weights bf16, weight gradients fp32 in the parameter's own layout. Autograd,
module parameters and the CPU path live in :mod:`scaffold_b200.ops.conv3d`.
"""
from __future__ import annotations

import os

import ctypes as C
from typing import Optional, Sequence

import torch

from . import _lib


def _pad_to(v: int, m: int) -> int:
    return (v + m - 1) // m * m


def pad_channels(c: int) -> int:
    """Channel counts the kernels accept: multiples of 16."""
    return _pad_to(c, 16)


# ---------------------------------------------------------------------------
# weight packing (bf16 operand copies; the fp32 parameter stays the master)
# ---------------------------------------------------------------------------
def kd_order(pack: torch.Tensor) -> torch.Tensor:
    """Reorder a 27-tap pack from (kd, kh, kw) to (kh, kw, 2-kd): the operand of the kd-fused plane kernel."""
    rows, k = pack.shape[1:]
    return pack.view(3, 3, 3, rows, k).flip(0).permute(1, 2, 0, 3, 4).reshape(27, rows, k).contiguous()


def _attach_kd_order(pack: torch.Tensor) -> torch.Tensor:
    # the kd-fused kernel (output channels in tiles of <= 64) wants the second ordering
    if pack.shape[0] == 27 and (pack.shape[1] <= 64 or pack.shape[1] % 64 == 0) and pack.shape[2] % 32 == 0:
        pack.kd_order = kd_order(pack)
    return pack


def pack_weight_fwd(w: torch.Tensor) -> torch.Tensor:
    """[Cout, Cin, k, k, k] -> bf16 [taps, cout_pad, cin_pad] (taps = kd,kh,kw row-major)."""
    co, ci = w.shape[:2]
    taps = w.shape[2] * w.shape[3] * w.shape[4]
    out = torch.zeros(taps, pad_channels(co), pad_channels(ci), dtype=torch.bfloat16, device=w.device)
    out[:, :co, :ci] = w.reshape(co, ci, taps).permute(2, 0, 1)
    return _attach_kd_order(out)


def pack_weight_dgrad(w: torch.Tensor) -> torch.Tensor:
    """Backward-data operand: bf16 [taps, cin_pad, cout_pad], taps flipped."""
    co, ci = w.shape[:2]
    taps = w.shape[2] * w.shape[3] * w.shape[4]
    out = torch.zeros(taps, pad_channels(ci), pad_channels(co), dtype=torch.bfloat16, device=w.device)
    out[:, :ci, :co] = w.reshape(co, ci, taps).flip(2).permute(2, 1, 0)
    return _attach_kd_order(out)


class Packed:
    """bf16 operand copies of one 3x3x3 weight for one direction: ``std`` taps in (kd,kh,kw) order and / or
    ``kd`` taps in (kh,kw,2-kd) order (kd-fused kernel). Shapes ``[27, rows, k]``."""
    __slots__ = ("std", "kd", "shape")

    def __init__(self, std: Optional[torch.Tensor], kd: Optional[torch.Tensor]):
        self.std, self.kd = std, kd
        self.shape = (std if std is not None else kd).shape


# Wide-output 3x3x3 calls run on SM pairs (tcgen05 cta_group::2, csrc/conv_plane2.cu). SCAFFOLD_PAIR_CONV=0 keeps
# them on the single-CTA kernels (the A/B switch of the kernel benchmarks).
PAIR_CONV = os.environ.get("SCAFFOLD_PAIR_CONV", "1") != "0"


def pair_eligible(rows: int, k: int, out_dims: Sequence[int], first_src: Optional[int] = None) -> bool:
    """True when ``sb_conv_fwd`` runs the two-SM pair kernel for a call that passes tap-ordered weights only:
    >= 128 output rows in multiples of 128, sources in multiples of 64 channels, planes of at least 8 x 16."""
    _, h, w = out_dims
    first = k if first_src is None else first_src
    return (PAIR_CONV and w >= 16 and h >= 8 and rows >= 128 and rows % 128 == 0 and k % 64 == 0
            and first % 64 == 0)


def kd_eligible(rows: int, k: int, out_dims: Sequence[int], first_src: Optional[int] = None) -> bool:
    """True when ``sb_conv_fwd`` should get the kd-ordered weights and run the kd-fused plane kernel for this
    call (no fused halo / slabs); wide outputs go to the pair kernel instead."""
    _, h, w = out_dims
    first = k if first_src is None else first_src
    if pair_eligible(rows, k, out_dims, first_src):
        return False
    return (w >= 16 and h >= 8 and rows % 16 == 0 and (rows <= 64 or rows % 64 == 0) and k % 32 == 0
            and first % 32 == 0)


def pack_conv3(w: torch.Tensor, src_c: Sequence[int], real_c: Sequence[int], want: dict, tap_swap: int = 0) -> None:
    """Fill the requested operand layouts of a 3x3x3 weight ``[Cout, Cin, 3,3,3]`` (fp32) in one kernel.

    ``want`` maps 'fwd' / 'fwd_kd' / 'dgrad' / 'dgrad_kd' to zero-initialised bf16 buffers
    (``[27, cout_pad, cin_pad]`` for forward, ``[27, cin_pad, cout_pad]`` for backward-data); padding
    positions are never written. ``src_c`` are the (padded) channel counts of the concatenated sources,
    ``real_c`` the channels of the weight that belong to each.
    """
    a = _lib.SbPackArgs()
    wc = w.detach().contiguous().float()
    fill_pack_args(a, wc, src_c, real_c, want, tap_swap)
    _lib.check(_lib.lib().sb_pack_conv3(C.byref(a), _lib.stream_ptr()), "sb_pack_conv3")


def fill_pack_args(a, wc: torch.Tensor, src_c: Sequence[int], real_c: Sequence[int], want: dict,
                   tap_swap: int = 0) -> None:
    """Describe one packing job: ``wc`` is the contiguous fp32 weight, ``want`` the layouts to write;
    ``tap_swap`` 1 / 2 packs the weight with the (kd, kh) / (kd, kw) tap axes exchanged."""
    a.tap_swap = int(tap_swap)
    co, ci = wc.shape[:2]
    a.w = wc.data_ptr()
    a.cout, a.cin = co, ci
    a.real0, a.pad0 = (real_c[0], src_c[0]) if len(src_c) > 1 else (ci, ci)
    a.cin_pad, a.cout_pad = sum(src_c), pad_channels(co)
    if len(src_c) > 2 or (len(src_c) == 2 and real_c[1] > src_c[1]):
        raise ValueError("pack_conv3 handles at most two concatenated sources")
    for name in ("fwd", "fwd_kd", "dgrad", "dgrad_kd"):
        t = want.get(name)
        setattr(a, name, t.data_ptr() if t is not None else None)


def bias_grad(gy: torch.Tensor, n_out: int) -> torch.Tensor:
    """fp32 sum of a voxel-major bf16 gradient ``[..., C]`` over all voxels, first ``n_out`` channels."""
    c = gy.shape[-1]
    m = gy.numel() // c
    L = _lib.lib()
    out = torch.empty(n_out, dtype=torch.float32, device=gy.device)
    work = torch.empty(L.sb_colsum_blocks() * c, dtype=torch.float32, device=gy.device)
    _lib.check(L.sb_colsum(gy.data_ptr(), m, c, out.data_ptr(), n_out, work.data_ptr(), _lib.stream_ptr()), "sb_colsum")
    return out


def pack_weight_convT_fwd(w: torch.Tensor) -> torch.Tensor:
    """[Cin, Cout, 2,2,2] -> bf16 [8*Cout, Cin] (row = tap*Cout + co)."""
    ci, co = w.shape[:2]
    return w.reshape(ci, co, 8).permute(2, 1, 0).reshape(8 * co, ci).to(torch.bfloat16).contiguous()


def pack_weight_convT_dgrad(w: torch.Tensor) -> torch.Tensor:
    """[Cin, Cout, 2,2,2] -> bf16 [4, cin_pad, 2*Cout] (outer = kd*2+kh, col = kw*Cout + co)."""
    ci, co = w.shape[:2]
    out = torch.zeros(4, pad_channels(ci), 2 * co, dtype=torch.bfloat16, device=w.device)
    # w[ci, co, kd, kh, kw] -> [kd, kh, ci, kw, co]
    out[:, :ci] = w.permute(2, 3, 0, 4, 1).reshape(4, ci, 2 * co)
    return out


# ---------------------------------------------------------------------------
# launchers
# ---------------------------------------------------------------------------
def _chk_act(t: torch.Tensor) -> None:
    if t.dtype != torch.bfloat16 or not t.is_contiguous() or t.dim() != 5:
        raise ValueError(f"expected a contiguous bf16 [N,D,H,W,C] tensor, got {t.dtype} {tuple(t.shape)} "
                         f"contiguous={t.is_contiguous()}")


def conv_same(srcs: Sequence[torch.Tensor], wpack: torch.Tensor, ksize: int,
              dst_channels: Sequence[int], bias: Optional[torch.Tensor] = None,
              force_plain: bool = False, out: Optional[Sequence[torch.Tensor]] = None,
              out_dims: Optional[Sequence[int]] = None, in_off: Sequence[int] = (0, 0, 0), halo=None,
              slabs: Optional[Sequence[torch.Tensor]] = None, kd_fused: bool = True, gn_groups: int = 0,
              gn_sink: Optional[list] = None):
    """Stride-1 'same' convolution of the channel concatenation of ``srcs``.

    Returns a list of outputs, one per entry of ``dst_channels`` (the output
    channels are split in that order). ``out_dims`` (D, H, W) and ``in_off`` describe
    halo'd sources of a sharded volume: output voxel 0 sits at ``in_off`` inside the
    sources (negative offsets read zeros, which is how backward-data grows a halo).
    ``kd_fused=False`` keeps a narrow-output call on the one-tap-per-MMA plane kernel.
    ``gn_groups`` > 0 asks the kernel to also produce the GroupNorm statistics of its output (groups over
    the padded output channels); when the call can (kd-fused kernel, one destination) the triple
    ``(partials, splits, groups)`` is appended to ``gn_sink``, the input of :func:`gn_kernels.gn_finalize`.
    """
    for s in srcs:
        _chk_act(s)
    n = srcs[0].shape[0]
    d, h, w = out_dims if out_dims is not None else srcs[0].shape[1:4]
    a = _lib.SbConvArgs()
    for i in range(2):
        if i < len(srcs):
            a.src[i] = srcs[i].data_ptr()
            a.src_c[i] = srcs[i].shape[4]
            a.src_ld[i] = srcs[i].shape[4]
        else:
            a.src[i] = None
            a.src_c[i] = 0
            a.src_ld[i] = 0
    a.N, a.D, a.H, a.W = n, d, h, w
    a.in_d, a.in_h, a.in_w = srcs[0].shape[1:4]
    a.off_d, a.off_h, a.off_w = (int(v) for v in in_off)
    a.ksize = ksize
    if isinstance(wpack, Packed):
        std, kd = wpack.std, (wpack.kd if kd_fused else None)
    else:
        std, kd = wpack, (getattr(wpack, "kd_order", None) if kd_fused else None)
    if kd is not None and std is not None and pair_eligible(wpack.shape[1], wpack.shape[2], (d, h, w),
                                                            srcs[0].shape[4]):
        kd = None  # both orderings at hand: the pair kernel reads the tap-ordered one
    a.wpack = std.data_ptr() if std is not None else None
    a.cout_pad = wpack.shape[1]
    a.wpack_kd = kd.data_ptr() if kd is not None else None
    if wpack.shape[2] != sum(s.shape[4] for s in srcs):
        raise ValueError(f"packed weight K {wpack.shape[2]} != source channels {[s.shape[4] for s in srcs]}")
    outs = list(out) if out is not None else [
        torch.empty((n, d, h, w, c), dtype=torch.bfloat16, device=srcs[0].device) for c in dst_channels]
    for i in range(2):
        if i < len(outs):
            a.dst[i] = outs[i].data_ptr()
            a.dst_c[i] = outs[i].shape[4]
            a.dst_ld[i] = outs[i].shape[4]
        else:
            a.dst[i] = None
            a.dst_c[i] = 0
            a.dst_ld[i] = 0
    a.bias = _lib.ptr(bias)
    a.status = _lib.status_tensor(srcs[0].device).data_ptr()
    a.force_plain = int(force_plain) if (PAIR_CONV or int(force_plain) != 0) else 4
    if halo is not None:
        # fused depth halo: landing slabs per (source, face) and the flag words that guard them
        for si in range(len(srcs)):
            for f in range(2):
                a.halo_land[si][f] = halo.land_ptr(si, f)
        for f in range(2):
            a.halo_flag[f] = halo.flag_ptr(f)
        a.halo_epoch = halo.epoch
        a.halo_wait_s = halo.wait_seconds
    if slabs is not None:
        a.slab_out[0], a.slab_out[1] = slabs[0].data_ptr(), slabs[1].data_ptr()
        a.slab_ld = slabs[0].shape[-1]
    if gn_groups > 0 and gn_sink is not None and len(outs) == 1 and slabs is None:
        a.gn_groups = int(gn_groups)
        splits = _lib.lib().sb_conv_gn_splits(C.byref(a))
        if splits > 0:
            part = torch.empty(n * splits * gn_groups * 3, dtype=torch.float32, device=srcs[0].device)
            a.gn_part = part.data_ptr()
            gn_sink.append((part, splits, int(gn_groups)))
        else:
            a.gn_groups = 0
    need = _lib.lib().sb_conv_fwd_workspace(C.byref(a))
    if need > 0:  # kernels that split the reduction keep fp32 partial sums here
        ws = _workspace(srcs[0].device, need)
        a.workspace, a.workspace_elems = ws.data_ptr(), ws.numel()
    _lib.check(_lib.lib().sb_conv_fwd(C.byref(a), _lib.stream_ptr()), "sb_conv_fwd")
    return outs


def convT_fwd(x: torch.Tensor, wpack: torch.Tensor, cout: int, bias: Optional[torch.Tensor]) -> torch.Tensor:
    _chk_act(x)
    n, d, h, w, cin = x.shape
    y = torch.empty((n, 2 * d, 2 * h, 2 * w, cout), dtype=torch.bfloat16, device=x.device)
    a = _lib.SbConvTArgs()
    a.src, a.src_ld = x.data_ptr(), cin
    a.N, a.D, a.H, a.W = n, d, h, w
    a.cin, a.cout = cin, cout
    a.wpack, a.wrows = wpack.data_ptr(), wpack.shape[0]
    a.dst, a.dst_ld = y.data_ptr(), cout
    a.bias = _lib.ptr(bias)
    a.status = _lib.status_tensor(x.device).data_ptr()
    _lib.check(_lib.lib().sb_convT_fwd(C.byref(a), _lib.stream_ptr()), "sb_convT_fwd")
    return y


def convT_dgrad(gy: torch.Tensor, wpack: torch.Tensor, cin_store: int) -> torch.Tensor:
    """gy [N,2D,2H,2W,Cout] -> gx [N,D,H,W,cin_store]."""
    _chk_act(gy)
    n, d2, h2, w2, cout = gy.shape
    d, h, w = d2 // 2, h2 // 2, w2 // 2
    gx = torch.empty((n, d, h, w, cin_store), dtype=torch.bfloat16, device=gy.device)
    a = _lib.SbConvTArgs()
    a.src, a.src_ld = gy.data_ptr(), cout
    a.N, a.D, a.H, a.W = n, d, h, w
    a.cin, a.cout = cin_store, cout
    a.wpack, a.wrows = wpack.data_ptr(), wpack.shape[1]
    a.dst, a.dst_ld = gx.data_ptr(), cin_store
    a.bias = None
    a.status = _lib.status_tensor(gy.device).data_ptr()
    _lib.check(_lib.lib().sb_convT_dgrad(C.byref(a), _lib.stream_ptr()), "sb_convT_dgrad")
    return gx


_workspaces: dict = {}


def _workspace(device, elems: int) -> torch.Tensor:
    key = torch.device(device).index or 0
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < elems:
        ws = torch.empty(max(elems, 1 << 22), dtype=torch.float32, device=device)
        _workspaces[key] = ws
    return ws


def conv_wgrad(gy: torch.Tensor, xs: Sequence[torch.Tensor], ksize: int, dw: torch.Tensor,
               accumulate: bool = False, splits: int = 0, x_off: Sequence[int] = (0, 0, 0),
               x_halo=None, tap_swap: int = 0) -> torch.Tensor:
    """Weight gradient into ``dw`` (fp32, parameter layout).

    ksize 1/3: ``dw`` is [Cout, Cin, k,k,k]; ``gy`` and ``xs`` share the voxel grid.
    ksize 2:   k2s2 transposed conv, ``dw`` is [Cin, Cout, 2,2,2]; ``gy`` is on the fine grid.
    """
    _chk_act(gy)
    for x in xs:
        _chk_act(x)
    n, d, h, w = xs[0].shape[:4]
    if ksize != 2:
        d, h, w = gy.shape[1:4]  # x may carry a halo; the voxel grid is gy's
    a = _lib.SbWgradArgs()
    if ksize != 2:
        a.xin_d, a.xin_h, a.xin_w = xs[0].shape[1:4]
        a.xoff_d, a.xoff_h, a.xoff_w = (int(v) for v in x_off)
    a.gy, a.gy_c, a.gy_ld = gy.data_ptr(), gy.shape[4], gy.shape[4]
    for i in range(2):
        if i < len(xs):
            a.x[i], a.x_c[i], a.x_ld[i] = xs[i].data_ptr(), xs[i].shape[4], xs[i].shape[4]
        else:
            a.x[i], a.x_c[i], a.x_ld[i] = None, 0, 0
    a.N, a.D, a.H, a.W = n, d, h, w
    if x_halo is not None:
        for si, pair in enumerate(x_halo):
            for f in range(2):
                a.xhalo[si][f] = pair[f].data_ptr() if pair[f] is not None else None
    a.ksize = ksize
    a.splits = splits
    a.tap_swap = int(tap_swap) if ksize == 3 else 0
    a.accumulate = 1 if accumulate else 0
    if not (dw.dtype == torch.float32 and dw.is_contiguous()):
        raise ValueError("dw must be contiguous fp32")
    if ksize == 2:
        a.dw_cin, a.dw_cout = dw.shape[0], dw.shape[1]
    else:
        a.dw_cout, a.dw_cin = dw.shape[0], dw.shape[1]
    L = _lib.lib()
    need = L.sb_conv_wgrad_workspace(C.byref(a))
    if need < 0:
        if len(xs) == 2 and x_halo is None:
            # two narrow sources (below the kernels' 64-channel source tiles): reduce over their concatenation
            return conv_wgrad(gy, [torch.cat(list(xs), dim=4)], ksize, dw, accumulate, splits, x_off,
                              tap_swap=tap_swap)
        raise _lib.NativeError(f"sb_conv_wgrad: unsupported shape gy={tuple(gy.shape)} xs={[tuple(x.shape) for x in xs]}")
    ws = _workspace(gy.device, need)
    a.workspace, a.workspace_elems = ws.data_ptr(), ws.numel()
    a.dw = dw.data_ptr()
    a.status = _lib.status_tensor(gy.device).data_ptr()
    _lib.check(L.sb_conv_wgrad(C.byref(a), _lib.stream_ptr()), "sb_conv_wgrad")
    return dw
