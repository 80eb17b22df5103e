"""Failure detection on the device: every wait in the kernels is bounded.

The failure is made on the host: a flag word that no peer ever raises. The kernel must give up after its
limit, record where it gave up in the status word and return, leaving the context usable; the host turns
the status into ``DeviceWaitTimeout``. Nothing here faults, traps or hangs the GPU.
"""
import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu


def _mods():
    from scaffold_b200.ops import _lib, conv_kernels as ck, gn_kernels as gk
    _lib.lib()
    return _lib, ck, gk


def test_groupnorm_peer_statistics_wait_runs_out_and_context_survives():
    _lib, ck, gk = _mods()
    torch.manual_seed(0)
    x = torch.randn(1, 8, 8, 16, 32, device="cuda").to(torch.bfloat16)
    w, b = torch.ones(32, device="cuda"), torch.zeros(32, device="cuda")
    part = gk.gn_stats(x, w, b, 8, 1e-5, True)
    peer_part = torch.zeros_like(part)
    flags = torch.zeros(2, dtype=torch.int32, device="cuda")  # nobody raises these to epoch 1
    gk.gn_apply(x, w, b, 8, 1e-5, True, [part.data_ptr(), peer_part.data_ptr()], shards=2,
                wait=(flags.data_ptr(), 1, 0.2))
    with pytest.raises(_lib.DeviceWaitTimeout):
        _lib.check_status()
    # the context is intact: the same op without the wait gives the right answer
    y, _, _ = gk.gn_forward(x, w, b, 8)
    torch.cuda.synchronize()
    _lib.check_status()
    ref = F.relu(F.group_norm(x.permute(0, 4, 1, 2, 3).float(), 8, w, b)).permute(0, 2, 3, 4, 1)
    assert (y.float() - ref).abs().max().item() < 0.05


class _DeadNeighbour:
    """Landing slabs whose flags never reach the epoch: a depth neighbour that never pushed its halo."""

    def __init__(self, n, h, w, c):
        self.slabs = [torch.zeros(n, 1, h, w, c, dtype=torch.bfloat16, device="cuda") for _ in range(2)]
        self.flags = torch.zeros(2, dtype=torch.int32, device="cuda")
        self.epoch, self.wait_seconds = 1, 0.2

    def land_ptr(self, source, face):
        return self.slabs[face].data_ptr()

    def flag_ptr(self, face):
        return self.flags[face:].data_ptr()


@pytest.mark.parametrize("kd_fused", [True, False], ids=["kd_fused", "plane"])
def test_conv_halo_wait_runs_out_and_context_survives(kd_fused):
    _lib, ck, gk = _mods()
    torch.manual_seed(1)
    x = torch.randn(1, 4, 16, 16, 64, device="cuda").to(torch.bfloat16)
    wt = torch.randn(64, 64, 3, 3, 3, device="cuda") * 0.05
    wpack = ck.pack_weight_fwd(wt)
    ck.conv_same([x], wpack, 3, [64], halo=_DeadNeighbour(1, 16, 16, 64), kd_fused=kd_fused)
    with pytest.raises(_lib.DeviceWaitTimeout):
        _lib.check_status()
    (y,) = ck.conv_same([x], wpack, 3, [64], kd_fused=kd_fused)
    torch.cuda.synchronize()
    _lib.check_status()
    ref = F.conv3d(x.permute(0, 4, 1, 2, 3).float(), wt.to(torch.bfloat16).float(), padding=1).permute(0, 2, 3, 4, 1)
    assert (y.float() - ref).abs().max().item() < 0.1
