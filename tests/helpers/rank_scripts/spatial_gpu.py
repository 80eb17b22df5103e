"""Rank script (2 GPUs): a U-Net step on a volume split over two spatial shards vs the unsharded step.

usage: spatial_gpu.py <split_dim 2|3|4 | shards "a,b,c"> [nccl|fused]   (world = product of the shard counts)
Both ranks hold the same weights. Each runs forward + fused loss + backward on its half; gradients are summed
over the shards. Rank 0 then repeats the step on the whole volume without sharding and compares loss and grads.
"""
import os
import sys

sys.path.insert(0, os.path.abspath(os.path.join(os.path.dirname(__file__), "..", "..", "..")))  # repo root: runnable directly

import torch
import torch.distributed as dist

rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
dev = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
torch.cuda.set_device(dev)
dist.init_process_group("nccl", device_id=dev)

from scaffold_b200.models.unet import UNet  # noqa: E402
from scaffold_b200.ops import _lib, loss as L  # noqa: E402
from scaffold_b200.parallel.layout import ParallelLayout  # noqa: E402
from scaffold_b200.parallel.spatial import SpatialContext  # noqa: E402
from scaffold_b200.run import attach_spatial  # noqa: E402

spec = sys.argv[1] if len(sys.argv) > 1 else "2"
halo_backend = sys.argv[2] if len(sys.argv) > 2 else "nccl"
if "," in spec:
    shards = [int(v) for v in spec.split(",")]
    split_dim = None
else:
    split_dim = int(spec)
    shards = [1, 1, 1]
    shards[split_dim - 2] = 2
layout = ParallelLayout(shards, (2, 3, 4), world, rank)
spatial = SpatialContext(layout, gn_stats="global", halo_backend=halo_backend)
single_axis = sum(1 for v in shards if v > 1) == 1
if halo_backend == "fused":
    assert spatial.stats_channel is not None
    assert (spatial.halo_channel is not None) == single_axis  # several split axes: slabs travel through NCCL
    if split_dim is not None:
        assert spatial.lead_swap == (None if split_dim == 2 else split_dim)

torch.manual_seed(0)
n_classes = 5
model = UNet(3, n_classes, layers=2, base_width=64).to(dev)
S = 64
g = torch.Generator(device="cuda").manual_seed(5)
x = torch.rand((1, 3, S, S, S), generator=g, device=dev)
y = torch.randint(0, n_classes, (1, S, S, S), generator=g, device=dev, dtype=torch.int16)
sl = [slice(None)] * 5
for k, (dim, nsh) in enumerate(zip((2, 3, 4), shards)):
    ext = S // nsh
    sl[dim] = slice(layout.shard_ind[k] * ext, (layout.shard_ind[k] + 1) * ext)
xl = x[tuple(sl)].contiguous()
yl = y[tuple(sl[:1] + sl[2:])].contiguous()


def step(net, xin, yin, sp):
    net.zero_grad(set_to_none=True)
    with torch.autocast("cuda", dtype=torch.bfloat16):
        logits = net.forward_padded_logits(xin)
    if sp is not None:  # the logits are in kernel space (split axis exchanged with depth); so must the labels be
        yin = sp.to_kernel_space(yin, first_spatial=1).contiguous()
    loss, ce, fg = L.segmentation_loss_fused(logits, yin, n_classes, None, sp)
    loss.backward()
    return loss.detach(), [p.grad.detach().float().clone() for p in net.parameters()]


attach_spatial(model, spatial)
loss_s, grads_s = step(model, xl, yl, spatial)
for gr in grads_s:
    dist.all_reduce(gr)
torch.cuda.synchronize()
_lib.check_status()
if rank == 0:
    attach_spatial(model, None)
    loss_w, grads_w = step(model, x, y, None)
    torch.cuda.synchronize()
    _lib.check_status()
    worst = 0.0
    for a, b in zip(grads_s, grads_w):
        worst = max(worst, (a - b).abs().max().item() / (b.abs().max().item() + 1e-6))
    print(f"RESULT loss {loss_s.item():.6f} {loss_w.item():.6f}")
    print(f"RESULT grad_rel {worst:.5f}")
dist.barrier()
dist.destroy_process_group()
print("DONE")
