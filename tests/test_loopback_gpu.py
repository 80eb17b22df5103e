"""The fused multi-GPU protocols on ONE GPU (loopback): halo push + convolution, halo-gradient return +
accumulate, cross-shard GroupNorm statistics, and the gradient all-reduce, each against the unsharded result.

Every consumer runs after both ranks' producers were launched (see ``scaffold_b200/parallel/loopback.py``); the all-reduce,
whose ranks wait on one another, runs as one cooperative launch over all ranks' buffers.
"""
import ctypes as C

import pytest
import torch
import torch.nn.functional as F

from scaffold_b200.parallel.loopback import halo_pair, stats_pair

pytestmark = pytest.mark.gpu


def _mods():
    from scaffold_b200.ops import _lib, conv_kernels as ck, gn_kernels as gk
    _lib.lib()
    return _lib, ck, gk


def _ints(shape, lo, hi, g):
    return torch.randint(lo, hi + 1, shape, generator=g, device="cuda").to(torch.bfloat16)


# the last two cases run the two-SM pair kernel: forward with landing slabs (>= 128 output rows), and for 128 -> 256
# also backward-data with slab outputs (128 rows)
@pytest.mark.parametrize("cin,cout,dims", [(64, 64, (8, 16, 32)), (32, 128, (4, 8, 16)), (64, 128, (4, 8, 16)),
                                           (128, 256, (6, 16, 16))])
def test_halo_push_then_conv_forward_dgrad_wgrad_match_the_whole_volume(cin, cout, dims):
    _lib, ck, gk = _mods()
    g = torch.Generator(device="cuda").manual_seed(3)
    n, (d, h, w) = 2, dims
    x = _ints((n, d, h, w, cin), -1, 1, g)
    gy = _ints((n, d, h, w, cout), -1, 1, g)
    wt = torch.randint(-1, 2, (cout, cin, 3, 3, 3), generator=g, device="cuda").float()
    wf, wd = ck.pack_weight_fwd(wt), ck.pack_weight_dgrad(wt)
    (y_ref,) = ck.conv_same([x], wf, 3, [cout])
    (dx_ref,) = ck.conv_same([gy], wd, 3, [cin])
    gw_ref = torch.empty_like(wt)
    ck.conv_wgrad(gy, [x], 3, gw_ref)

    half = d // 2
    xs = [x[:, :half].contiguous(), x[:, half:].contiguous()]
    gys = [gy[:, :half].contiguous(), gy[:, half:].contiguous()]
    chans = halo_pair(2)
    # forward: both pushes first, then both convolutions
    lands = [c.exchange([xs[r][:, 0]], [xs[r][:, -1]]) for r, c in enumerate(chans)]
    ys = [ck.conv_same([xs[r]], wf, 3, [cout], halo=lands[r])[0] for r in range(2)]
    saved = [l.clone() for l in lands]
    torch.cuda.synchronize()
    _lib.check_status()
    assert torch.equal(torch.cat(ys, 1), y_ref)

    # backward-data: halo'd output grid, slabs go home, the owners add them
    outs, slabs = [], []
    for r in range(2):
        sl = [torch.empty((n, 1, h, w, cin), dtype=torch.bfloat16, device="cuda") for _ in range(2)]
        o = ck.conv_same([gys[r]], wd, 3, [cin], out_dims=(half + 2, h, w), in_off=(-1, 0, 0), slabs=sl,
                         out=[torch.empty((n, half, h, w, cin), dtype=torch.bfloat16, device="cuda")])
        outs.append(o)
        slabs.append(sl)
    lands2 = [c.exchange([slabs[r][0][:, 0]], [slabs[r][1][:, 0]]) for r, c in enumerate(chans)]
    for r, c in enumerate(chans):
        c.accumulate(outs[r], lands2[r], cin)
    torch.cuda.synchronize()
    _lib.check_status()
    assert torch.equal(torch.cat([o[0] for o in outs], 1), dx_ref)

    # weight gradient against the halo'd input: the two shards' gradients add up to the whole volume's
    gws = []
    for r in range(2):
        gw = torch.empty_like(wt)
        ck.conv_wgrad(gys[r], [xs[r]], 3, gw, x_halo=saved[r])
        gws.append(gw)
    torch.cuda.synchronize()
    _lib.check_status()
    assert torch.equal(gws[0] + gws[1], gw_ref)


def test_cross_shard_groupnorm_statistics_in_loopback_equal_the_unsharded_normalisation():
    _lib, ck, gk = _mods()
    torch.manual_seed(5)
    n, d, h, w, c, groups = 2, 8, 8, 16, 64, 8
    x = (torch.randn(n, d, h, w, c, device="cuda") * 1.5 + 0.3).to(torch.bfloat16)
    gyv = torch.randn(n, d, h, w, c, device="cuda").to(torch.bfloat16)
    wt, b = torch.randn(c, device="cuda"), torch.randn(c, device="cuda")
    y_ref, mean_ref, rstd_ref = gk.gn_forward(x, wt, b, groups, 1e-5, True)
    dx_ref, dw_ref, db_ref = gk.gn_backward(gyv, x, wt, b, mean_ref, rstd_ref, groups, 1e-5, True)
    half = d // 2
    xs = [x[:, :half].contiguous(), x[:, half:].contiguous()]
    gs = [gyv[:, :half].contiguous(), gyv[:, half:].contiguous()]
    chans = stats_pair(2)
    fins = [gk.gn_stats(xs[r], wt, b, groups, 1e-5, True) for r in range(2)]
    shared = [chans[r].share(fins[r]) for r in range(2)]          # both producers first
    outs = [gk.gn_apply(xs[r], wt, b, groups, 1e-5, True, shared[r][0], shards=2, wait=shared[r][1] + (0.5,))
            for r in range(2)]
    torch.cuda.synchronize()
    _lib.check_status()
    y = torch.cat([o[0] for o in outs], 1)
    assert (y.float() - y_ref.float()).abs().max().item() <= 0.02
    assert torch.allclose(outs[0][1], mean_ref, rtol=1e-4, atol=1e-5) and torch.allclose(outs[1][2], rstd_ref, rtol=1e-4)
    # backward: per-channel sums travel the same way
    bfin = [gk.gn_bwd_partial(gs[r], xs[r], wt, b, outs[r][1], outs[r][2], groups, 1e-5, True) for r in range(2)]
    bshared = [chans[r].share(bfin[r]) for r in range(2)]
    bouts = [gk.gn_bwd_dx(gs[r], xs[r], wt, b, outs[r][1], outs[r][2], groups, 1e-5, True, bshared[r][0], shards=2,
                          wait=bshared[r][1] + (0.5,)) for r in range(2)]
    torch.cuda.synchronize()
    _lib.check_status()
    dx = torch.cat([o[0] for o in bouts], 1)
    assert (dx.float() - dx_ref.float()).abs().max().item() <= 0.03 * max(1.0, dx_ref.float().abs().max().item())


@pytest.mark.parametrize("world", [2, 4, 8])
def test_gradient_allreduce_protocol_in_cooperative_loopback_is_exact(world):
    _lib, ck, gk = _mods()
    from scaffold_b200.parallel.peer import PeerBuffer
    L = _lib.lib()
    _P = C.c_void_p
    fn = L.sb_grad_allreduce_loopback
    fn.argtypes = [C.POINTER(_P), C.POINTER(_P), C.c_int, C.c_longlong, C.c_longlong, C.c_uint, C.c_float, C.c_int,
                   C.c_double, _P, _P]
    fn.restype = C.c_int
    n = (1 << 18) + 12
    bufs = [PeerBuffer(n * 4) for _ in range(world)]
    flags = [PeerBuffer(4096) for _ in range(world)]
    g = torch.Generator(device="cuda").manual_seed(9)
    srcs = [torch.randint(-8, 9, (n,), generator=g, device="cuda").float() for _ in range(world)]
    want = torch.stack(srcs).sum(0) * 0.5   # integers: exact whatever the order
    for epoch in (1, 2):                     # the second round reuses flags and counters
        for r in range(world):
            bufs[r].tensor(torch.float32)[:n].copy_(srcs[r])
        barr = (_P * world)(*[b.local for b in bufs])
        farr = (_P * world)(*[f.local for f in flags])
        rc = fn(barr, farr, world, 0, n, epoch, 0.5, 8, 0.5, _lib.status_tensor("cuda").data_ptr(),
                torch.cuda.current_stream().cuda_stream)
        assert rc == 0
        torch.cuda.synchronize()
        _lib.check_status()
        for r in range(world):
            assert torch.equal(bufs[r].tensor(torch.float32)[:n], want)
    # the production kernel itself with one rank: scale only
    from scaffold_b200.parallel.fused_allreduce import FusedAllReduce
    solo = object.__new__(FusedAllReduce)
    solo.group, solo.world, solo.rank, solo.numel = None, 1, 0, n
    solo.data, solo.flags = bufs[0], flags[0]
    solo.grad = bufs[0].tensor(torch.float32)[:n]
    solo.epoch, solo.ctas, solo.wait_seconds = 2, 16, 0.5
    solo._bufs, solo._flags = bufs[0].ptr_array(), flags[0].ptr_array()
    solo.grad.copy_(srcs[0])
    solo.all_reduce_(scale=0.25)
    torch.cuda.synchronize()
    _lib.check_status()
    assert torch.equal(solo.grad, srcs[0] * 0.25)
    for b in bufs + flags:
        b.close()
