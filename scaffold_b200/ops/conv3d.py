"""Convolution modules: stock parameter names, sm_100a kernels on CUDA, ATen on CPU.

``Conv3d`` / ``ConvTranspose3d`` subclass the ``torch.nn`` modules, so their
state dicts are interchangeable with the stock ones (weights ``(Cout,Cin,k,k,k)``
and ``(Cin,Cout,2,2,2)``, no buffers); packed bf16 operand copies are caches
outside the state dict, refreshed when the parameter's version changes.

On CUDA with bf16 activations (or under autocast) the forward, backward-data
and weight-gradient all run on the tcgen05 kernels of ``csrc/conv_igemm.cu`` and
``csrc/conv_wgrad.cu``; there is no library fallback on that path. A CPU tensor
(the gloo plumbing runs) takes ATen.

``Conv3d.forward`` accepts one tensor or a sequence of tensors that are read as
their channel concatenation: the U-Net skip concat is never materialised on the
CUDA path (role of ``_skip_concat``, ScaFFold/unet/unet_parts.py:76-120, and of
``FastConv3d``/``FastConvTranspose3d``, ScaFFold/unet/conv3d.py:1235-1904).
"""
from __future__ import annotations

import ctypes as C
import os
import weakref
from typing import List, Optional, Sequence, Union

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import conv_kernels as ck
from .layout import direct_grad_target, from_vm, notify_grad_written, to_vm, use_cuda_kernels, weights_epoch


# A/B switch: "0" keeps the GroupNorm statistics in their own pass instead of the convolution's epilogue
_GN_FROM_EPILOGUE = os.environ.get("SCAFFOLD_GN_FROM_EPILOGUE", "1") != "0"

_PACK_REGISTRY: "weakref.WeakSet[_PackCache]" = weakref.WeakSet()
_PACK_PLAN = {"key": None, "table": None, "n": 0, "tiles": 0, "members": []}


def repack_all() -> int:
    """Refresh every 3x3x3 operand copy that any layer has asked for so far, in ONE kernel launch.

    The optimizer calls this right after it updated the weights, so the next forward pass finds all
    packs fresh instead of launching one packing kernel per layer (role of the weight repack that
    the update kernel owes the convolutions). Returns the number of layers covered; layers that have
    not run yet, or whose weight is a non-contiguous view, keep packing lazily on first use.
    """
    from . import _lib
    members = []
    for cache in list(_PACK_REGISTRY):
        w = cache._w_ref() if cache._w_ref is not None else None
        if w is None or not w.is_cuda or not w.is_contiguous() or w.dtype != torch.float32:
            continue
        for sig in sorted({k[1] for k in cache._asked}):
            names = sorted(nm for nm, s_ in cache._asked if s_ == sig)
            bufs = {nm: cache._bufs.get((nm, sig, w.device)) for nm in names}
            if any(b is None for b in bufs.values()):
                continue
            members.append((cache, w, sig, cache._real[sig], bufs))
    if not members:
        return 0
    key = tuple((id(c), w.data_ptr(), sig, c._tap_swap, tuple((n, b.data_ptr()) for n, b in sorted(bufs.items())))
                for c, w, sig, _, bufs in members)
    plan = _PACK_PLAN
    if plan["key"] != key:
        jobs = (_lib.SbPackJob * len(members))()
        for j, (_, w, sig, real_c, bufs) in enumerate(members):
            ck.fill_pack_args(jobs[j].a, w, sig, real_c, bufs, cache._tap_swap)
        total = _lib.lib().sb_pack_conv3_plan(jobs, len(members))
        if total < 1:
            raise _lib.NativeError("sb_pack_conv3_plan refused the packing table")
        host = torch.frombuffer(bytearray(bytes(jobs)), dtype=torch.uint8)
        plan.update(key=key, table=host.to(members[0][1].device), n=len(members), tiles=int(total))
    _lib.check(_lib.lib().sb_pack_conv3_batch(plan["table"].data_ptr(), plan["n"], plan["tiles"], _lib.stream_ptr()),
               "sb_pack_conv3_batch")
    for cache, w, sig, _, bufs in members:
        cache._sync(w)
        cache._fresh.update((nm, sig) for nm in bufs)
    return len(members)


class _PackCache:
    """bf16 operand copies of one parameter, keyed by (tensor identity, version)."""

    def __init__(self):
        self._key = None
        self._w_ref = None    # the parameter these copies belong to (set on first use)
        self._real = {}       # source signature -> real channels per source
        self._tap_swap = 0    # tap-axis exchange the packs were made with (sharded runs, see Conv3d._tap_swap)
        self._vals = {}
        self._asked = set()   # (layout name, source signature) ever requested: packed together
        self._fresh = set()   # of those, the ones that hold the current weights
        self._bufs = {}       # persistent operand buffers (padding positions stay zero)

    def _sync(self, w: torch.Tensor, tap_swap: Optional[int] = None):
        # strides / tap exchange: the same parameter may be read tap-transposed (sharded runs) or directly
        if tap_swap is not None:
            self._tap_swap = int(tap_swap)
        key = (w.data_ptr(), w._version, w.device, weights_epoch(), tuple(w.stride()), self._tap_swap)
        if key != self._key:
            self._key = key
            self._vals = {}
            self._fresh = set()

    def conv3(self, w: torch.Tensor, src_c, real_c, kind: str, kd: bool, tap_swap: int = 0) -> "ck.Packed":
        """Operand copy of a 3x3x3 weight for ``kind`` in ('fwd', 'dgrad'), taps kd-ordered if ``kd``.

        Every layout this module has ever asked for with the same sources is refreshed by the same
        kernel launch, so a step packs each weight once.
        """
        self._sync(w, tap_swap)
        sig = tuple(src_c)
        name = kind + ("_kd" if kd else "")
        if (name, sig) not in self._fresh:
            self._asked.add((name, sig))
            self._real[sig] = list(real_c)
            if self._w_ref is None and isinstance(w, torch.nn.Parameter):
                self._w_ref = weakref.ref(w)
                _PACK_REGISTRY.add(self)
            group = [k for k in self._asked if k[1] == sig]
            want = {}
            co_pad, k_pad = ck.pad_channels(w.shape[0]), sum(sig)
            for nm, _ in group:
                bkey = (nm, sig, w.device)
                buf = self._bufs.get(bkey)
                if buf is None:
                    shape = (27, co_pad, k_pad) if nm.startswith("fwd") else (27, k_pad, co_pad)
                    buf = self._bufs[bkey] = torch.zeros(shape, dtype=torch.bfloat16, device=w.device)
                want[nm] = buf
            ck.pack_conv3(w, sig, real_c, want, tap_swap)
            self._fresh.update(group)
        buf = self._bufs[(name, sig, w.device)]
        return ck.Packed(None if kd else buf, buf if kd else None)

    def get(self, w: torch.Tensor, name: str, fn):
        self._sync(w)
        v = self._vals.get(name)
        if v is None:
            with torch.no_grad():
                v = fn(w.detach().float())
            self._vals[name] = v
        return v


def _pad_in_channels(w: torch.Tensor, src_channels: Sequence[int], real: Sequence[int]) -> torch.Tensor:
    """Insert zero input-channel columns so the weight matches channel-padded sources."""
    if list(src_channels) == list(real):
        return w
    parts, o = [], 0
    for sc, rc in zip(src_channels, real):
        blk = w[:, o:o + rc]
        if sc > rc:
            blk = F.pad(blk, (0, 0, 0, 0, 0, 0, 0, sc - rc))
        parts.append(blk)
        o += rc
    return torch.cat(parts, 1)


class _ConvSameFn(torch.autograd.Function):
    """k in {1,3} stride-1 'same' conv over voxel-major bf16 sources."""

    @staticmethod
    def forward(ctx, weight, bias, mod, in_off, fwd_xs, *xs):
        """``xs`` are saved for backward; ``fwd_xs`` (or None) are the same sources padded to more channels,
        read by the forward kernel only (a few-channel stem runs the kd-fused kernel on 32 padded channels)."""
        ks = weight.shape[2]
        in_off = tuple(int(v) for v in in_off)
        in_dims = tuple(xs[0].shape[1:4])
        out_dims = tuple(d - 2 * o for d, o in zip(in_dims, in_off))
        src_c = [x.shape[4] for x in xs]
        real_c = mod._real_in_channels(src_c)
        ts = mod._tap_swap() if ks == 3 else 0
        if fwd_xs is not None:
            f_src = [x.shape[4] for x in fwd_xs]
            wf = mod._cache.conv3(weight, f_src, real_c, "fwd",
                                  ck.kd_eligible(ck.pad_channels(weight.shape[0]), sum(f_src), out_dims, f_src[0]), ts)
        elif ks == 3:
            kd = ck.kd_eligible(ck.pad_channels(weight.shape[0]), sum(src_c), out_dims, src_c[0])
            wf = mod._cache.conv3(weight, src_c, real_c, "fwd", kd, ts)
        else:
            wf = mod._cache.get(weight, f"fwd{src_c}",
                                lambda w: ck.pack_weight_fwd(_pad_in_channels(w, src_c, real_c)))
        cout_pad = wf.shape[1]
        bpad = None
        if bias is not None:
            bpad = mod._cache_b.get(bias, "b", lambda b: F.pad(b, (0, cout_pad - b.shape[0])).contiguous())
        sink = []
        gn = mod.gn_groups_hint if (_GN_FROM_EPILOGUE and ks == 3 and cout_pad == weight.shape[0]) else 0
        (y,) = ck.conv_same(list(fwd_xs if fwd_xs is not None else xs), wf, ks, [cout_pad], bias=bpad,
                            out_dims=out_dims, in_off=in_off, gn_groups=gn, gn_sink=sink)
        mod._gn_partials = sink[0] if sink else None  # picked up by Conv3d.forward, handed to the GroupNorm
        ctx.mod = mod
        ctx.wparam = weight  # the caller's tensor itself: backward may add into its flat-buffer .grad
        ctx.in_off, ctx.in_dims = in_off, in_dims
        ctx.src_c, ctx.real_c = src_c, real_c
        ctx.tap_swap = ts
        ctx.has_bias = bias is not None
        ctx.save_for_backward(weight, *xs)
        return y

    @staticmethod
    def backward(ctx, gy):
        weight, *xs = ctx.saved_tensors
        mod = ctx.mod
        ks = weight.shape[2]
        gy = gy.contiguous()
        src_c, real_c = ctx.src_c, ctx.real_c
        gxs: List[Optional[torch.Tensor]] = [None] * len(xs)
        need_gx = [ctx.needs_input_grad[5 + i] for i in range(len(xs))]
        if any(need_gx):
            if ks == 3:
                # rows = input channels of the layer, K = gy's channels (Cout padded to a multiple of 16)
                kd = ck.kd_eligible(sum(src_c), gy.shape[4], ctx.in_dims)
                wd = mod._cache.conv3(weight, src_c, real_c, "dgrad", kd, ctx.tap_swap)
            else:
                wd = mod._cache.get(weight, f"dgrad{src_c}",
                                    lambda w: ck.pack_weight_dgrad(_pad_in_channels(w, src_c, real_c)))
            # a halo'd input gets a halo'd gradient: output grid = input extents, gy read at -offset
            outs = ck.conv_same([gy], wd, ks, src_c, out_dims=ctx.in_dims, in_off=[-o for o in ctx.in_off])
            for i, o in enumerate(outs):
                if need_gx[i]:
                    gxs[i] = o
        gw = gb = None
        if ctx.needs_input_grad[0]:
            direct = direct_grad_target(ctx.wparam) if list(src_c) == list(real_c) else None
            if direct is not None:
                # the ordered split-K reduce adds straight into the parameter's slice of the flat gradient buffer
                ck.conv_wgrad(gy, list(xs), ks, direct, accumulate=True, x_off=ctx.in_off, tap_swap=ctx.tap_swap)
                notify_grad_written(ctx.wparam)
            elif list(src_c) == list(real_c):
                gw = torch.empty(weight.shape, dtype=torch.float32, device=weight.device)  # contiguous whatever the parameter layout
                ck.conv_wgrad(gy, list(xs), ks, gw, x_off=ctx.in_off, tap_swap=ctx.tap_swap)
            else:
                # channel-padded sources (the 3-channel stem): gradient over padded Cin, then slice
                gw = None
                gwp = torch.empty((weight.shape[0], sum(src_c), ks, ks, ks), dtype=torch.float32, device=gy.device)
                ck.conv_wgrad(gy, list(xs), ks, gwp, x_off=ctx.in_off, tap_swap=ctx.tap_swap)
                parts, o = [], 0
                for sc, rc in zip(src_c, real_c):
                    parts.append(gwp[:, o:o + rc])
                    o += sc
                gw = torch.cat(parts, 1).contiguous()
        if ctx.has_bias and ctx.needs_input_grad[1]:
            gb = ck.bias_grad(gy, weight.shape[0])
        return (gw, gb, None, None, None, *gxs)


class _ConvHaloFn(torch.autograd.Function):
    """3x3x3 conv on a depth-sharded volume with the halo fused into the kernels (no padded copy)."""

    @staticmethod
    def forward(ctx, weight, bias, mod, chan, *xs):
        src_c = [x.shape[4] for x in xs]
        kd = ck.kd_eligible(ck.pad_channels(weight.shape[0]), sum(src_c), xs[0].shape[1:4], src_c[0])
        ts = mod._tap_swap()
        wf = mod._cache.conv3(weight, src_c, src_c, "fwd", kd, ts)
        cout_pad = wf.shape[1]
        landing = chan.exchange([x[:, 0] for x in xs], [x[:, -1] for x in xs])
        sink = []
        gn = mod.gn_groups_hint if (_GN_FROM_EPILOGUE and cout_pad == weight.shape[0]) else 0
        (y,) = ck.conv_same(list(xs), wf, 3, [cout_pad], halo=landing, gn_groups=gn, gn_sink=sink)
        mod._gn_partials = sink[0] if sink else None
        ctx.halo_saved = landing.clone()  # the arena slot is recycled; backward needs the planes again
        ctx.mod, ctx.chan, ctx.src_c = mod, chan, src_c
        ctx.wparam, ctx.tap_swap = weight, ts
        ctx.save_for_backward(weight, *xs)
        return y

    @staticmethod
    def backward(ctx, gy):
        weight, *xs = ctx.saved_tensors
        mod, chan, src_c = ctx.mod, ctx.chan, ctx.src_c
        gy = gy.contiguous()
        n, d, h, w, _ = gy.shape
        gxs: List[Optional[torch.Tensor]] = [None] * len(xs)
        if any(ctx.needs_input_grad[4 + i] for i in range(len(xs))):
            kd = ck.kd_eligible(sum(src_c), gy.shape[4], (d + 2, h, w))
            wd = mod._cache.conv3(weight, src_c, src_c, "dgrad", kd, ctx.tap_swap)
            ctot = sum(src_c)
            slabs = [torch.empty((n, 1, h, w, ctot), dtype=torch.bfloat16, device=gy.device) for _ in range(2)]
            outs = ck.conv_same([gy], wd, 3, src_c, out_dims=(d + 2, h, w), in_off=(-1, 0, 0), slabs=slabs,
                                out=[torch.empty((n, d, h, w, c), dtype=torch.bfloat16, device=gy.device)
                                     for c in src_c])
            # the halo's gradient goes home: my low slab is the low neighbour's last plane, and vice versa
            landing = chan.exchange([slabs[0][:, 0]], [slabs[1][:, 0]])
            chan.accumulate(outs, landing, ctot)
            for i, o in enumerate(outs):
                if ctx.needs_input_grad[4 + i]:
                    gxs[i] = o
        gw = None
        if ctx.needs_input_grad[0]:
            direct = direct_grad_target(ctx.wparam)
            if direct is not None:
                ck.conv_wgrad(gy, list(xs), 3, direct, accumulate=True, x_halo=ctx.halo_saved, tap_swap=ctx.tap_swap)
                notify_grad_written(ctx.wparam)
            else:
                gw = torch.empty(weight.shape, dtype=torch.float32, device=weight.device)  # contiguous whatever the parameter layout
                ck.conv_wgrad(gy, list(xs), 3, gw, x_halo=ctx.halo_saved, tap_swap=ctx.tap_swap)
        return (gw, None, None, None, *gxs)


class Conv3d(nn.Conv3d):
    """3-D convolution; drop-in for ``nn.Conv3d`` (k=1 or k=3 'same', stride 1 on the CUDA path)."""

    def __init__(self, *args, **kwargs):
        super().__init__(*args, **kwargs)
        self._cache = _PackCache()
        self._cache_b = _PackCache()
        self._spatial = None  # parallel.spatial.SpatialContext when the volume is sharded
        self.gn_groups_hint = 0   # groups of the GroupNorm that consumes this layer's output (0: none / unknown)
        self._gn_partials = None  # statistics the last forward kernel produced for that GroupNorm

    def set_spatial(self, ctx) -> None:
        self._spatial = ctx

    def _w(self) -> torch.Tensor:
        """The weight as the kernels' axes see it: tap axes exchanged like the volume's (``lead_swap``), a view
        (ATen path; the kernel path passes the parameter itself plus ``_tap_swap`` so that the packing and the
        weight-gradient kernels do the exchange and the flat-buffer fast paths stay on)."""
        k = getattr(self._spatial, "lead_swap", None)
        return self.weight if k is None else self.weight.transpose(2, k)

    def _tap_swap(self) -> int:
        """0, or which tap axis the kernels exchange with kd: 1 = kh (volume split along H), 2 = kw (along W)."""
        k = getattr(self._spatial, "lead_swap", None)
        return 0 if k is None else k - 2

    def _real_in_channels(self, src_c: Sequence[int]) -> List[int]:
        """Real (unpadded) channel count of each source; only a single source may be padded."""
        if len(src_c) == 1:
            return [self.in_channels]
        if sum(src_c) != self.in_channels:
            raise ValueError(f"sources {list(src_c)} do not add up to in_channels={self.in_channels}")
        return list(src_c)

    def _kernel_ok(self) -> bool:
        k = self.kernel_size
        return (k[0] == k[1] == k[2] and k[0] in (1, 3) and self.stride == (1, 1, 1) and self.dilation == (1, 1, 1)
                and self.groups == 1 and self.padding == (k[0] // 2,) * 3 and self.padding_mode == "zeros")

    def forward(self, x: Union[torch.Tensor, Sequence[torch.Tensor]]) -> torch.Tensor:
        xs = [x] if isinstance(x, torch.Tensor) else list(x)
        if use_cuda_kernels(xs[0]):
            if not self._kernel_ok():
                raise NotImplementedError(
                    f"sm_100a conv kernels cover k in (1,3), stride 1, 'same' zero padding; got {self}")
            y = self._cuda_forward(xs)
            out = from_vm(y)
            if y.shape[4] != self.out_channels:
                return out[:, : self.out_channels]
            if self._gn_partials is not None:
                out._sb_gn_partials, self._gn_partials = self._gn_partials, None
            return out
        xin = xs[0] if len(xs) == 1 else torch.cat([t.to(xs[0].dtype) for t in xs], dim=1)
        sp = self._spatial
        if sp is not None and sp.size > 1 and self.kernel_size[0] > 1:
            # sharded volume: neighbours' boundary planes replace the zero padding on the split dims
            xin = sp.halo_pad(xin, self.kernel_size[0] // 2)
            return F.conv3d(xin, self._w(), self.bias, self.stride, sp.conv_padding(self.kernel_size[0]),
                            self.dilation, self.groups)
        return self._conv_forward(xin, self._w(), self.bias)

    def _cuda_forward(self, xs) -> torch.Tensor:
        """Voxel-major output of the kernel path; on a sharded volume the sources first receive their halo."""
        sp = self._spatial
        off = (0, 0, 0)
        if sp is not None and sp.size > 1 and self.kernel_size[0] == 3 and sp.halo_channel is not None:
            vms = [to_vm(t, pad16=True) for t in xs]
            d, h, w = vms[0].shape[1:4]
            real = self._real_in_channels([v.shape[4] for v in vms])
            # out_channels % 32: the weight-gradient kernel that reads the landed slabs tiles gy by 32 channels
            if h >= 8 and w >= 16 and d >= 2 and self.bias is None and real == [v.shape[4] for v in vms] \
                    and self.out_channels % 32 == 0:
                return _ConvHaloFn.apply(self.weight, self.bias, self, sp.halo_channel, *vms)
        if sp is not None and sp.size > 1 and self.kernel_size[0] > 1:
            halo = self.kernel_size[0] // 2
            xs = [sp.halo_pad(t, halo) for t in xs]
            off = tuple(halo if d in sp.dims else 0 for d in (2, 3, 4))
        vms = [to_vm(t, pad16=True) for t in xs]
        fwd_vms = None
        if (len(xs) == 1 and self.kernel_size[0] == 3 and self.in_channels < 16 and not xs[0].requires_grad
                and vms[0].shape[2] >= 8 and vms[0].shape[3] >= 16):
            # few input channels (the stem): the forward pass reads a copy padded to 32 channels so that it runs
            # the kd-fused kernel; the weight gradient keeps the 16-channel copy
            fwd_vms = (to_vm(xs[0], pad16=True, pad_to=32),)
        return _ConvSameFn.apply(self.weight, self.bias, self, off, fwd_vms, *vms)

    def forward_padded(self, x) -> torch.Tensor:
        """CUDA path only: voxel-major output with the channel axis padded to a multiple of 16."""
        xs = [x] if isinstance(x, torch.Tensor) else list(x)
        return self._cuda_forward(xs)


class _ConvTFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, weight, bias, mod, x):
        cout = weight.shape[1]
        wf = mod._cache.get(weight, "fwd", ck.pack_weight_convT_fwd)
        b32 = None
        if bias is not None:
            b32 = mod._cache_b.get(bias, "b", lambda b: b.contiguous())
        y = ck.convT_fwd(x, wf, cout, b32)
        ctx.mod = mod
        ctx.wparam = weight
        ctx.has_bias = bias is not None
        ctx.save_for_backward(weight, x)
        return y

    @staticmethod
    def backward(ctx, gy):
        weight, x = ctx.saved_tensors
        mod = ctx.mod
        gy = gy.contiguous()
        gx = gw = gb = None
        if ctx.needs_input_grad[3]:
            wd = mod._cache.get(weight, "dgrad", ck.pack_weight_convT_dgrad)
            gx = ck.convT_dgrad(gy, wd, x.shape[4])
        if ctx.needs_input_grad[0]:
            direct = direct_grad_target(ctx.wparam)
            if direct is not None:
                ck.conv_wgrad(gy, [x], 2, direct, accumulate=True)
                notify_grad_written(ctx.wparam)
            else:
                gw = torch.empty(weight.shape, dtype=torch.float32, device=weight.device)  # contiguous whatever the parameter layout
                ck.conv_wgrad(gy, [x], 2, gw)
        if ctx.has_bias and ctx.needs_input_grad[1]:
            gb = ck.bias_grad(gy, gy.shape[4])
        return gw, gb, None, gx


class ConvTranspose3d(nn.ConvTranspose3d):
    """k=2, s=2 transposed convolution (the U-Net upsampler); drop-in for ``nn.ConvTranspose3d``."""

    def __init__(self, *args, **kwargs):
        super().__init__(*args, **kwargs)
        self._cache = _PackCache()
        self._cache_b = _PackCache()
        self._spatial = None

    def set_spatial(self, ctx) -> None:
        self._spatial = ctx

    def _w(self) -> torch.Tensor:
        k = getattr(self._spatial, "lead_swap", None)
        return self.weight if k is None else self.weight.transpose(2, k)

    def _kernel_ok(self) -> bool:
        return (self.kernel_size == (2, 2, 2) and self.stride == (2, 2, 2) and self.padding == (0, 0, 0)
                and self.output_padding == (0, 0, 0) and self.groups == 1 and self.dilation == (1, 1, 1)
                and self.in_channels % 16 == 0 and self.out_channels % 8 == 0)

    def forward(self, x: torch.Tensor, output_size=None) -> torch.Tensor:
        if use_cuda_kernels(x):
            if not self._kernel_ok() or output_size is not None:
                raise NotImplementedError(f"sm_100a transposed-conv kernel covers k=2, s=2, no padding; got {self}")
            return from_vm(_ConvTFn.apply(self._w(), self.bias, self, to_vm(x)))
        if getattr(self._spatial, "lead_swap", None) is not None:
            return F.conv_transpose3d(x, self._w(), self.bias, self.stride, self.padding, self.output_padding,
                                      self.groups, self.dilation)
        return super().forward(x, output_size)
