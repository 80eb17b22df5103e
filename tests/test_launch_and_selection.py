"""Launch-shape sniffing and restart templates, the kernel-selection report, the axis exchange of sharded runs,
and the gradient-written notifications: host-side logic, no GPU."""
from pathlib import Path

import pytest
import torch

from scaffold_b200.utils import restart_script as rs


@pytest.mark.parametrize("env,world,want", [
    ({}, None, ("local", 1, 1, 1)),
    ({"WORLD_SIZE": "8", "LOCAL_WORLD_SIZE": "8"}, None, ("torchrun", 1, 8, 8)),
    ({"WORLD_SIZE": "16", "LOCAL_WORLD_SIZE": "8"}, None, ("torchrun", 2, 16, 8)),
    ({"SLURM_JOB_ID": "7", "SLURM_JOB_NUM_NODES": "4", "SLURM_NTASKS": "32"}, None, ("slurm", 4, 32, 8)),
    ({"SLURM_JOBID": "7", "SLURM_NNODES": "2", "SLURM_NPROCS": "8(x2)"}, None, ("slurm", 2, 8, 4)),
    ({"FLUX_JOB_ID": "f1", "FLUX_JOB_NNODES": "2", "FLUX_JOB_SIZE": "16"}, None, ("flux", 2, 16, 8)),
    ({}, 4, ("torchrun", 1, 4, 4)),                       # a known rank count wins over an empty environment
    ({"FLUX_JOB_ID": "f1", "FLUX_JOB_NNODES": "1", "FLUX_JOB_SIZE": "2"}, 8, ("flux", 1, 8, 8)),
])
def test_launch_shape_is_read_from_the_scheduler_then_the_launcher(env, world, want):
    s = rs.launch_shape(env, world)
    assert (s["scheduler"], s["nodes"], s["ranks"], s["per_node"]) == want


def test_restart_script_templates_per_launcher():
    argv = ["benchmark", "-c", "a.yml", "--job-name", "x", "--problem-scale", "7"]
    local = rs.render(Path("/tmp/r"), argv, env={})
    assert "exec python -m scaffold_b200.cli benchmark -c $RUN_DIR/config.yaml --problem-scale 7 --restart" in local
    tr = rs.render(Path("/tmp/r"), argv, env={"WORLD_SIZE": "8", "LOCAL_WORLD_SIZE": "8"})
    assert "torch.distributed.run" in tr and "RANKS_PER_NODE=8" in tr and "--master-addr ${MASTER_ADDR:-127.0.0.1}" in tr
    sl = rs.render(Path("/tmp/r"), argv, env={"SLURM_JOB_ID": "1", "SLURM_NNODES": "2", "SLURM_NTASKS": "16",
                                                "PROFILE_TORCH": "ON", "VIRTUAL_ENV": "/venvs/s"})
    assert "exec srun -N \"$NODES\" -n \"$RANKS\"" in sl and "NODES=2" in sl and "RANKS=16" in sl
    assert "export PROFILE_TORCH=ON" in sl and "/venvs/s/bin/activate" in sl and "scontrol show hostnames" in sl
    fx = rs.render(Path("/tmp/r"), argv, env={"FLUX_JOB_ID": "f", "FLUX_JOB_NNODES": "1", "FLUX_JOB_SIZE": "8"})
    assert "exec flux run -N \"$NODES\" -n \"$RANKS\"" in fx and "--job-name" not in fx


def test_launch_scripts_are_present_and_executable_shell():
    root = Path(__file__).resolve().parents[1] / "scaffold_b200" / "launch"
    text = (root / "b200_8gpu.sh").read_text()
    assert text.startswith("#!/bin/bash") and "generate_fractals" in text and "--dc-num-shards $SHARDS" in text
    assert (root / "b200_8gpu.sh").stat().st_mode & 0o111
    assert "srun" in (root / "slurm_8gpu.job").read_text() and "flux run" in (root / "flux_8gpu.job").read_text()


def test_kernel_selection_walks_shapes_without_memory_or_launches():
    from scaffold_b200.models.unet import UNet
    from scaffold_b200.ops.selection import format_selection, kernel_selection
    model = UNet(3, 9, layers=4, base_width=64)
    rows = kernel_selection(model, 2, (128, 128, 128))
    by = {r["layer"]: r for r in rows}
    assert len(rows) == 45  # 19 convs / transposed convs + 18 GroupNorms + 4 pools + ... in execution order
    assert by["down_list.0.double_conv.3"] == {"layer": "down_list.0.double_conv.3", "op": "conv k3 64->64",
                                               "input": "2x128x128x128", "fwd": "conv_plane3", "dgrad": "conv_plane3",
                                               "wgrad": "wgrad_plane", "halo": "-"}
    # layers with >= 128 output rows run on SM pairs; a 128 -> 64 layer does so only in backward-data (rows = C_in)
    assert by["down_list.2.maxpool_conv.1.double_conv.3"]["fwd"] == "conv_plane2(pair)"
    assert by["down_list.2.maxpool_conv.1.double_conv.3"]["dgrad"] == "conv_plane2(pair)"
    assert by["up_list.3.conv.double_conv.0"]["fwd"] == "conv_plane3"
    assert by["up_list.3.conv.double_conv.0"]["dgrad"] == "conv_plane2(pair)"
    assert by["down_list.1.maxpool_conv.1.double_conv.0"]["dgrad"] == "conv_plane3"   # 64 rows
    assert by["down_list.4.maxpool_conv.1.double_conv.0"]["fwd"] == "conv_small"
    assert by["up_list.0.up"]["op"] == "convT k2 1024->512" and by["up_list.4.conv"]["fwd"] == "igemm"
    assert by["down_list.0.double_conv.0"]["fwd"].startswith("conv_plane3 (32-ch")
    assert by["down_list.1.maxpool_conv.0"]["fwd"] == "maxpool2_fwd"
    # a (channels, groups) pair outside the GroupNorm kernels is reported instead of failing later
    wide = UNet(3, 4, layers=1, base_width=24, group_norm_groups=8)  # 3 channels per group: outside the kernels
    assert any("ATen" in r["fwd"] for r in kernel_selection(wide, 1, (8, 8, 8)))
    text = format_selection(rows, {"grad_allreduce_effective": "fused"})
    assert text.splitlines()[0].startswith("layer") and text.endswith("grad_allreduce_effective: fused")


class _FakeLayout:
    def __init__(self, num_shards):
        self.num_shards, self.shard_dim = tuple(num_shards), (2, 3, 4)
        self.spatial_size = 1
        for n in num_shards:
            self.spatial_size *= n
        self.spatial_group = None

    def sharded_dims(self):
        return [d for d, n in zip(self.shard_dim, self.num_shards) if n > 1]

    def neighbour(self, dim, direction):
        return ("volume-dim", dim, direction)


def test_spatial_context_without_peer_memory_keeps_volume_axes():
    from scaffold_b200.parallel.spatial import SpatialContext
    sp = SpatialContext(_FakeLayout((1, 1, 2)), halo_backend="fused")  # no CUDA / NCCL here: no exchange
    assert sp.lead_swap is None and sp.dims == [4] and sp.halo_channel is None
    t = torch.arange(2 * 3 * 4 * 5 * 6).reshape(2, 3, 4, 5, 6)
    assert sp.to_kernel_space(t) is t and sp.volume_dim(2) == 2
    assert sp.neighbours(4) == (("volume-dim", 4, -1), ("volume-dim", 4, 1))


def test_axis_exchange_maps_kernel_space_to_the_volume_and_back():
    from scaffold_b200.parallel.spatial import SpatialContext
    sp = SpatialContext(_FakeLayout((1, 1, 2)), halo_backend="nccl")
    sp.lead_swap, sp.dims = 4, [2]  # what a CUDA run with the fused halo sets for a W split
    t = torch.arange(2 * 3 * 4 * 5 * 6).reshape(2, 3, 4, 5, 6)
    k = sp.to_kernel_space(t)
    assert k.shape == (2, 3, 6, 5, 4) and torch.equal(sp.from_kernel_space(k), t)
    labels = torch.arange(2 * 4 * 5 * 6).reshape(2, 4, 5, 6)
    assert sp.to_kernel_space(labels, first_spatial=1).shape == (2, 6, 5, 4)
    assert [sp.volume_dim(d) for d in (2, 3, 4)] == [4, 3, 2]
    assert sp.neighbours(2) == (("volume-dim", 4, -1), ("volume-dim", 4, 1))  # kernel depth = the volume's W


def test_halo_channel_accepts_exactly_one_split_axis():
    from scaffold_b200.parallel.halo import HaloChannel
    assert HaloChannel.eligible(_FakeLayout((2, 1, 1))) and HaloChannel.eligible(_FakeLayout((1, 4, 1)))
    assert HaloChannel.eligible(_FakeLayout((1, 1, 8)))
    assert not HaloChannel.eligible(_FakeLayout((2, 2, 1))) and not HaloChannel.eligible(_FakeLayout((1, 1, 1)))


def test_conv_reads_its_weight_through_the_exchanged_taps_on_the_cpu_path():
    """ATen path of a sharded module: convolving the axis-exchanged volume with the tap-exchanged weight equals
    exchanging the axes of the ordinary convolution's output."""
    from scaffold_b200.ops.conv3d import Conv3d, ConvTranspose3d

    class Sp:
        lead_swap, size, dims, halo_channel = 4, 1, [2], None
    torch.manual_seed(0)
    conv = Conv3d(3, 5, kernel_size=3, padding=1, bias=False)
    x = torch.randn(1, 3, 4, 6, 8)
    want = conv(x).transpose(2, 4)
    conv.set_spatial(Sp())
    assert conv._tap_swap() == 2
    assert torch.allclose(conv(x.transpose(2, 4)), want, atol=1e-5)
    up = ConvTranspose3d(4, 2, kernel_size=2, stride=2)
    y = torch.randn(1, 4, 2, 3, 5)
    want = up(y).transpose(2, 4)
    up.set_spatial(Sp())
    assert torch.allclose(up(y.transpose(2, 4)), want, atol=1e-5)


def test_direct_gradient_target_needs_the_flat_buffer_mark():
    from scaffold_b200.ops import layout as L
    p = torch.nn.Parameter(torch.zeros(4, 3))
    assert L.direct_grad_target(p) is None
    p.grad = torch.zeros(4, 3)
    assert L.direct_grad_target(p) is None            # a plain parameter keeps autograd's accumulation
    setattr(p, L.FLAT_GRAD_ATTR, True)
    assert L.direct_grad_target(p) is p.grad
    p.grad = torch.zeros(3, 4).t()
    assert L.direct_grad_target(p) is None            # a non-contiguous gradient view is not written directly


def test_effective_backends_report_what_runs():
    from scaffold_b200.ops.selection import effective_backends

    class R:
        _fused, _buckets = None, None

    class E:
        spatial, layout, reducer = None, None, R()
    out = effective_backends(E())
    assert out == {"grad_allreduce_effective": "none", "grad_overlap_effective": "off",
                   "halo_exchange_effective": "none", "gn_stats_effective": "local"}
