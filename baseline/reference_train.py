#!/usr/bin/env python
"""Time-to-Dice run of the reference's own pieces on a dataset this framework generated.

    python baseline/reference_train.py --dataset-dir <dataset> --n-categories 5 --scale 7 --batch 1 \
        --target-dice 0.95 --max-epochs 200 --out <dir>
    (under torch.distributed.run for several data-parallel replicas)

The reference's trainer module cannot be imported on this machine (it imports the external
``distconv`` package), so this script drives, in the order that trainer does
(ScaFFold/utils/trainer.py:257-319,563-715,895-1273):

* the reference's ``FractalDataset`` reading the physical-shard ``.npy`` layout (an interchange check of the
  dataset format at the same time),
* its ``UNet`` in channels_last_3d under bf16 autocast (cuDNN convolutions, Triton GroupNorm),
* ``_compute_ce_class_weights`` + weighted ``compute_sharded_cross_entropy_loss`` + ``compute_sharded_dice``,
* ``clip_grad_norm_(1.0)``, fused Adam, ``CosineAnnealingWarmRestarts(T_0, T_mult, eta_min)`` stepped per epoch,
* validation after every epoch: hard (argmax) Dice averaged over the foreground classes, per sample.

Nothing of this repository's models, kernels or engine is imported. It writes ``train_stats.csv`` with the
reference's columns and prints one JSON line with the seconds of training until the target Dice (epoch
durations summed, the definition behind the figure of merit, ScaFFold/worker.py:342-389).
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time
from pathlib import Path

REF = Path(__file__).resolve().parent / "_ref"


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--dataset-dir", required=True)
    ap.add_argument("--n-categories", type=int, default=5)
    ap.add_argument("--scale", type=int, default=7)
    ap.add_argument("--bottleneck-dim", type=int, default=3)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--target-dice", type=float, default=0.95)
    ap.add_argument("--max-epochs", type=int, default=200)
    ap.add_argument("--lr", type=float, default=1e-3)
    ap.add_argument("--min-lr", type=float, default=1e-4)
    ap.add_argument("--T-0", type=int, default=10)
    ap.add_argument("--T-mult", type=int, default=2)
    ap.add_argument("--seed", type=int, default=42)
    ap.add_argument("--workers", type=int, default=2)
    ap.add_argument("--out", default="reference_run")
    a = ap.parse_args()
    if not (REF / "ScaFFold").exists():
        print(json.dumps({"impl": "reference", "unavailable": "baseline/_ref is empty"}))
        return 0
    os.environ.setdefault("SCAFFOLD_GROUPNORM_TRITON", "1")
    sys.path.insert(0, str(REF))
    import torch
    import torch.distributed as dist
    import torch.nn.functional as F
    from torch.utils.data import DataLoader, DistributedSampler

    from ScaFFold.unet.unet_model import UNet
    from ScaFFold.utils.data_loading import FractalDataset, SpatialShardSpec
    from ScaFFold.utils.dice_score import compute_sharded_dice, labels_to_onehot
    from ScaFFold.utils.losses import _compute_ce_class_weights, compute_sharded_cross_entropy_loss

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=device)
    torch.backends.cudnn.benchmark = True
    torch.manual_seed(a.seed)

    root = Path(a.dataset_dir)
    spec = SpatialShardSpec((2, 3, 4), (1, 1, 1), (0, 0, 0))  # one rank holds the whole volume
    # third argument: the split's pickle of mask values, as the reference trainer passes it (trainer.py:170-181)
    train_set = FractalDataset(str(root / "volumes" / "training"), str(root / "masks" / "training"),
                               str(root / "train_unique_mask_vals"), spec)
    val_set = FractalDataset(str(root / "volumes" / "validation"), str(root / "masks" / "validation"),
                             str(root / "val_unique_mask_vals"), spec)
    n_classes = a.n_categories + 1
    model = UNet(3, n_classes, trilinear=False, layers=a.scale - a.bottleneck_dim, group_norm_groups=8)
    model = model.to(device=device, memory_format=torch.channels_last_3d)
    net = model
    if world > 1:
        net = torch.nn.parallel.DistributedDataParallel(model, device_ids=[local_rank], output_device=local_rank)
    opt = torch.optim.Adam(model.parameters(), lr=a.lr, fused=True)
    sched = torch.optim.lr_scheduler.CosineAnnealingWarmRestarts(opt, T_0=a.T_0, T_mult=a.T_mult, eta_min=a.min_lr)
    weights = _compute_ce_class_weights(train_set, len(train_set), a.n_categories, device, 0.1, world > 1, rank, None)
    sampler = DistributedSampler(train_set, num_replicas=world, rank=rank, shuffle=True, seed=a.seed)
    val_idx = list(range(rank, len(val_set), world))  # every sample on exactly one replica
    common = dict(num_workers=a.workers, pin_memory=True, persistent_workers=a.workers > 0)
    train_loader = DataLoader(train_set, batch_size=a.batch, sampler=sampler, drop_last=False, **common)
    val_loader = DataLoader(torch.utils.data.Subset(val_set, val_idx), batch_size=a.batch, shuffle=False, **common)

    def loss_of(preds, labels):
        with torch.autocast("cuda", enabled=False):
            log_probs = F.log_softmax(preds.float(), dim=1)
            ce = compute_sharded_cross_entropy_loss(preds, labels, None, [1, 1, 1], "cuda", weights, log_probs=log_probs)
            dice = compute_sharded_dice(log_probs.exp(), labels_to_onehot(labels, n_classes), None)
        return ce + (1.0 - dice[:, 1:].mean())

    def reduce_sums(vals):
        t = torch.tensor(vals, device=device, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t)
        return t.tolist()

    out_dir = Path(a.out)
    if rank == 0:
        out_dir.mkdir(parents=True, exist_ok=True)
        (out_dir / "train_stats.csv").write_text(
            "epoch,epoch_loss,overall_loss,val_loss_epoch,val_loss_avg,train_dice,val_dice,epoch_duration,"
            "optimizer_steps,total_optimizer_steps\n")
    # untimed warm-up (cuDNN algorithm search, Triton compilation), state restored afterwards
    snap = {k: v.detach().clone() for k, v in model.state_dict().items()}
    opt_snap = opt.state_dict()
    for i, batch in enumerate(train_loader):
        if i >= 3:
            break
        x = batch["image"].to(device=device, dtype=torch.float32, memory_format=torch.channels_last_3d)
        y = batch["mask"].to(device=device, dtype=torch.long)
        opt.zero_grad(set_to_none=True)
        with torch.autocast("cuda", dtype=torch.bfloat16):
            loss_of(net(x), y).backward()
        opt.step()
    model.load_state_dict(snap)
    opt = torch.optim.Adam(model.parameters(), lr=a.lr, fused=True)
    sched = torch.optim.lr_scheduler.CosineAnnealingWarmRestarts(opt, T_0=a.T_0, T_mult=a.T_mult, eta_min=a.min_lr)
    del opt_snap
    torch.cuda.synchronize()

    total_time, total_steps, reached, val_dice = 0.0, 0, None, 0.0
    epoch = 0
    while val_dice < a.target_dice and epoch < a.max_epochs:
        epoch += 1
        torch.cuda.synchronize()
        t0 = time.time()
        sampler.set_epoch(epoch)
        net.train()
        loss_sum = torch.zeros((), device=device)
        n_seen, steps = 0, 0
        for batch in train_loader:
            x = batch["image"].to(device=device, dtype=torch.float32, memory_format=torch.channels_last_3d,
                                  non_blocking=True)
            y = batch["mask"].to(device=device, dtype=torch.long, non_blocking=True).contiguous()
            opt.zero_grad(set_to_none=True)
            with torch.autocast("cuda", dtype=torch.bfloat16):
                loss = loss_of(net(x), y)
            loss.backward()
            torch.nn.utils.clip_grad_norm_(model.parameters(), max_norm=1.0)
            opt.step()
            loss_sum += loss.detach() * x.shape[0]
            n_seen += x.shape[0]
            steps += 1
        net.eval()
        dice_sum = torch.zeros((), device=device)
        vloss_sum = torch.zeros((), device=device)
        n_val = 0
        with torch.inference_mode():
            for batch in val_loader:
                x = batch["image"].to(device=device, dtype=torch.float32, memory_format=torch.channels_last_3d)
                y = batch["mask"].to(device=device, dtype=torch.long).contiguous()
                with torch.autocast("cuda", dtype=torch.bfloat16):
                    preds = model(x)
                    vloss_sum += loss_of(preds, y) * x.shape[0]
                hard = F.one_hot(preds.argmax(dim=1), n_classes).permute(0, 4, 1, 2, 3).float()
                d = compute_sharded_dice(hard, labels_to_onehot(y, n_classes), None)
                dice_sum += d[:, 1:].mean(dim=1).sum()
                n_val += x.shape[0]
        sched.step()
        tl, ns, ds, vl, nv = reduce_sums([float(loss_sum), n_seen, float(dice_sum), float(vloss_sum), n_val])
        torch.cuda.synchronize()
        duration = time.time() - t0
        total_time += duration
        total_steps += steps
        val_dice = ds / max(nv, 1)
        if reached is None and val_dice >= a.target_dice:
            reached = total_time
        if rank == 0:
            with open(out_dir / "train_stats.csv", "a") as f:
                f.write(f"{epoch},{tl},{tl / max(ns, 1)},{vl},{vl / max(nv, 1)},0,{val_dice},{duration},{steps},"
                        f"{total_steps}\n")
            print(f"epoch {epoch} train_loss {tl / max(ns, 1):.5f} val_loss {vl / max(nv, 1):.5f} val_dice {val_dice:.5f} "
                  f"duration {duration:.2f}s", flush=True)
    if rank == 0:
        print(json.dumps({"impl": "reference", "n_gpus": world, "epochs": epoch, "val_dice": val_dice,
                          "time_to_dice_s": reached, "total_train_time_s": total_time,
                          "target_dice": a.target_dice, "train_volumes": len(train_set), "val_volumes": len(val_set),
                          "batch_per_replica": a.batch}), flush=True)
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
