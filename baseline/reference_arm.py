"""Reference arm of ``bench.py``: the unmodified reference package from ``baseline/_ref``.

Nothing of this repository's models, kernels or engine is imported here. The
reference's trainer module cannot be imported on this machine (it imports the
external ``distconv`` package, which is a git-URL dependency), so this arm
drives the reference's own public pieces in the order its trainer does
(ScaFFold/utils/trainer.py:563-715, the ``ps is None`` branch):

* ``ScaFFold.unet.unet_model.UNet`` in ``channels_last_3d`` under bf16 autocast
  (its adapters pick cuDNN convolutions on NVIDIA, and its Triton GroupNorm
  when ``SCAFFOLD_GROUPNORM_TRITON=1``, as the reference's NVIDIA job script sets),
* ``compute_sharded_cross_entropy_loss`` + ``compute_sharded_dice`` +
  ``labels_to_onehot`` for the loss,
* ``clip_grad_norm_(1.0)`` + fused ``torch.optim.Adam``,
* ``torch.nn.parallel.DistributedDataParallel`` (the base class of the
  reference's ``DistConvDDP``) for N > 1.
"""
from __future__ import annotations

import os
import sys
from pathlib import Path

REF = Path(__file__).resolve().parent / "_ref"


def run(args):
    if not (REF / "ScaFFold").exists():
        return {"impl": "reference", "unavailable": "baseline/_ref is empty (offline install not done on this box)"}
    os.environ.setdefault("SCAFFOLD_GROUPNORM_TRITON", "1")
    sys.path.insert(0, str(REF))
    import torch
    import torch.distributed as dist
    import torch.nn.functional as F

    from ScaFFold.unet.unet_model import UNet  # noqa: E402
    from baseline.common_config import workload_config  # noqa: E402
    from ScaFFold.utils.dice_score import compute_sharded_dice, labels_to_onehot  # noqa: E402
    from ScaFFold.utils.losses import compute_sharded_cross_entropy_loss  # noqa: E402

    if args.base_width != 64:
        return {"impl": "reference", "unavailable": "the reference U-Net has a fixed base width of 64"}
    if list(args.dc_num_shards) != [1, 1, 1]:
        return {"impl": "reference", "unavailable": "spatial sharding needs the external distconv package (git URL)"}

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=device)
    torch.backends.cudnn.benchmark = True  # ScaFFold/worker.py:171-179

    torch.manual_seed(42)
    n_classes = args.n_categories + 1
    layers = args.scale - args.bottleneck_dim
    model = UNet(3, n_classes, trilinear=False, layers=layers, group_norm_groups=8)
    model = model.to(device=device, memory_format=torch.channels_last_3d)
    net = model
    if world > 1:
        net = torch.nn.parallel.DistributedDataParallel(model, device_ids=[local_rank], output_device=local_rank)
    opt = torch.optim.Adam(model.parameters(), lr=1e-3, fused=True)

    S = 2 ** args.scale
    g = torch.Generator().manual_seed(1234 + rank)
    host = []
    for _ in range(2):
        img = torch.rand((args.batch, 3, S, S, S), generator=g).pin_memory()
        msk = torch.randint(0, n_classes, (args.batch, S, S, S), generator=g, dtype=torch.int16).pin_memory()
        host.append((img, msk))
    dev_batches = [(i.to(device), m.to(device)) for i, m in host]

    def step(images, masks):
        images = images.to(device=device, dtype=torch.float32, memory_format=torch.channels_last_3d, non_blocking=True)
        labels = masks.to(device=device, dtype=torch.long, non_blocking=True).contiguous()
        opt.zero_grad(set_to_none=True)
        with torch.autocast("cuda", dtype=torch.bfloat16):
            preds = net(images)
            with torch.autocast("cuda", enabled=False):
                log_probs = F.log_softmax(preds.float(), dim=1)
                ce = compute_sharded_cross_entropy_loss(preds, labels, None, [1, 1, 1], "cuda", None,
                                                        log_probs=log_probs)
                dice = compute_sharded_dice(log_probs.exp(), labels_to_onehot(labels, n_classes), None)
                loss = ce + (1.0 - dice[:, 1:].mean())
        loss.backward()
        torch.nn.utils.clip_grad_norm_(model.parameters(), max_norm=1.0)
        opt.step()
        return loss.detach()

    def sync():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms):
        if world == 1:
            return ms
        t = torch.tensor([ms], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    for i in range(max(args.warmup, 3)):
        step(*dev_batches[i % 2])
    sync()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        step(*dev_batches[i % 2])
    e1.record()
    sync()
    ms_total = max_over_ranks(e0.elapsed_time(e1))
    for i in range(2):
        float(step(*host[i % 2]).item())
    sync()
    e0.record()
    for i in range(args.steps):
        loss_val = float(step(*host[i % 2]).item())
    e1.record()
    sync()
    ms_e2e = max_over_ranks(e0.elapsed_time(e1))

    vox = args.batch * world * S ** 3
    out = {
        "impl": "reference",
        "metric": "3D U-Net train voxels/sec",
        "value": vox / (ms_total / args.steps / 1e3),
        "unit": "voxels/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_total / args.steps,
        "higher_is_better": True, "scaling": "weak", "dtype": "bf16",
        "data": "synthetic (random volumes and labels of the dataset's shape; random-init weights)",
        "config": workload_config(args.scale, layers + 1, 64, n_classes, sum(p.numel() for p in model.parameters()),
                                  args.batch, world, [1, 1, 1],
                                  {"final_loss": loss_val,
                                   "kernels": "cuDNN conv (cudnn.benchmark), Triton GroupNorm "
                                              "(SCAFFOLD_GROUPNORM_TRITON=1), torch DDP/NCCL, fused Adam"}),
        "e2e": {"value": vox / (ms_e2e / args.steps / 1e3), "unit": "voxels/s",
                "ms_per_step": ms_e2e / args.steps,
                "h2d_bytes_per_step": sum(t.numel() * t.element_size() for t in host[0]), "d2h_bytes_per_step": 4},
    }
    if world > 1:
        dist.destroy_process_group()
    if rank != 0:
        return None
    return out
