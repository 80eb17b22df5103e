"""Training loop: datasets, samplers, optimizer/scheduler, warm-up, epochs, CSV, checkpoints.

Public surface kept from ``PyTorchTrainer`` (ScaFFold/utils/trainer.py:366-1273):
``Trainer(model, config, device, log)`` with ``cleanup_or_resume()``, ``warmup()``
and ``train(profiler)``; ``train_stats.csv`` with the columns ``epoch, epoch_loss,
overall_loss, val_loss_epoch, val_loss_avg, train_dice, val_dice, epoch_duration,
optimizer_steps, total_optimizer_steps``; training runs until the validation
Dice reaches ``target_dice`` (or ``epochs``); epoch metrics are sample-weighted
sums reduced over the data-parallel replicas only (the spatial reduction already
happened inside loss and metric); the per-minibatch time is measured with CUDA
events, maximised over ranks and reported as a median, from which the
voxels-per-second figure is derived.
"""
from __future__ import annotations

import math
import os
import statistics
import time
from pathlib import Path
from typing import List, Optional

import torch
import torch.distributed as dist
from torch.utils.data import DataLoader, DistributedSampler, Sampler

from ..data.dataset import FractalDataset, SpatialShardSpec
from ..ops.optim import FusedClipAdam
from ..utils import dist as D
from ..utils.log import gather_and_print_mem
from ..utils.perf import adiak_value, begin_code_region, end_code_region, region
from .prefetch import DevicePrefetcher
from .checkpoint import CheckpointManager
from .engine import TrainEngine
from .evaluate import evaluate

CSV_COLUMNS = ["epoch", "epoch_loss", "overall_loss", "val_loss_epoch", "val_loss_avg", "train_dice", "val_dice",
               "epoch_duration", "optimizer_steps", "total_optimizer_steps"]


class UnpaddedDistributedSampler(Sampler):
    """Contiguous, unpadded split: every sample goes to exactly one replica (ranks may get uneven counts)."""

    def __init__(self, dataset, num_replicas: int, rank: int):
        n = len(dataset)
        base, rem = divmod(n, num_replicas)
        start = rank * base + min(rank, rem)
        self.indices = list(range(start, start + base + (1 if rank < rem else 0)))

    def __iter__(self):
        return iter(self.indices)

    def __len__(self):
        return len(self.indices)

    def set_epoch(self, epoch):  # order is fixed; present for API parity
        return None


def sample_ce_weight_indices(n_train: int, fraction: Optional[float]) -> List[int]:
    """Evenly spaced mask indices, first and last included (the float32 ``linspace`` rule of
    ScaFFold/utils/losses.py:24-39, so both implementations weigh the same masks); all of them when the
    fraction rounds up to the whole split."""
    if n_train <= 0:
        return []
    count = max(1, math.ceil(n_train * float(0.1 if fraction is None else fraction)))
    if count >= n_train:
        return list(range(n_train))
    return torch.linspace(0, n_train - 1, steps=count).long().tolist()


def compute_ce_class_weights(train_set, n_categories: int, device, sample_fraction: float = 0.1, log=None):
    """Cross-entropy class weights ``total / background`` for class 0 and ``total / foreground`` shared by all
    fractal classes, from the voxel histogram of a sample of training masks (local shards, summed over ranks).
    Uniform weights when the sample lacks either kind of voxel. Role of ScaFFold/utils/losses.py:42-114."""
    n_cls = n_categories + 1
    picked = sample_ce_weight_indices(len(train_set), sample_fraction)
    mask_of = getattr(train_set, "load_mask_only", None) or (lambda i: train_set[i]["mask"])
    hist = torch.zeros(n_cls, dtype=torch.long)
    for i in picked:
        hist += torch.bincount(mask_of(i).reshape(-1).long(), minlength=n_cls)[:n_cls]
    hist = hist.to(device)
    if dist.is_initialized() and dist.get_world_size() > 1:
        dist.all_reduce(hist)  # every rank sampled its own shard of the same masks
    bg, fg = (int(v) for v in (hist[0], hist[1:].sum()))
    weights = torch.ones(n_cls, device=device, dtype=torch.float32)
    usable = bg > 0 and fg > 0
    if usable:
        weights[0], weights[1:] = (bg + fg) / bg, (bg + fg) / fg
    if log is not None:
        if not picked:
            log.warning("class weights: the training split is empty; every class weighs 1")
        elif not usable:
            log.warning("class weights: %d sampled masks hold %d background and %d foreground voxels; one kind is "
                        "missing, so every class weighs 1", len(picked), bg, fg)
        else:
            log.info("class weights from masks %s (fraction %s): %d background / %d foreground voxels -> "
                     "background %.4f, foreground %.4f", picked, sample_fraction, bg, fg, float(weights[0]),
                     float(weights[-1]))
    return weights


class PrimedLoader:
    """Iterable over a DataLoader whose next iterator can be created ahead of time.

    ``prime()`` builds the iterator now, so the workers start loading the next epoch's first batches while the
    caller does something else (the validation pass); the following ``iter()`` hands that iterator out. Without it
    every epoch begins with the latency of one sample load (about 80 ms for a 128^3 volume), which is a tenth of an
    epoch once four replicas share the training set."""

    def __init__(self, loader):
        self.loader = loader
        self._it = None

    def __len__(self):
        return len(self.loader)

    def prime(self) -> None:
        self._it = iter(self.loader)

    def __iter__(self):
        it, self._it = self._it, None
        return it if it is not None else iter(self.loader)


def _collate(batch):
    return {"image": torch.stack([b["image"] for b in batch]), "mask": torch.stack([b["mask"] for b in batch])}


class Trainer:
    def __init__(self, model, config, device, log, layout=None, spatial=None):
        self.model, self.config, self.device, self.log = model, config, torch.device(device), log
        self.layout, self.spatial = layout, spatial
        self.world_rank = D.get_world_rank()
        self.n_classes = int(config.n_categories) + 1
        self.run_dir = Path(config.run_dir)
        self.outfile_path = self.run_dir / "train_stats.csv"
        self.start_epoch, self.start_val_dice = 1, 0.0
        self.global_step = 0
        self.total_optimizer_steps = 0
        self._setup_data()
        self._setup_optimization()
        self.checkpoints = CheckpointManager(self.run_dir, config.checkpoint_dir, getattr(config, "async_save", False),
                                             log)

    # -- set-up -------------------------------------------------------------------
    def _setup_data(self) -> None:
        cfg = self.config
        root = Path(cfg.dataset_dir)
        spec = SpatialShardSpec.from_layout(self.layout) if self.layout is not None else SpatialShardSpec()
        self.train_set = FractalDataset(root / "volumes" / "training", root / "masks" / "training", str(root), spec)
        self.val_set = FractalDataset(root / "volumes" / "validation", root / "masks" / "validation", str(root), spec)
        for ds in (self.train_set, self.val_set):
            ds.check_ids_across_ranks()
        replicas = self.layout.ddp_ranks if self.layout is not None else D.get_world_size()
        replica = self.layout.ddp_ind if self.layout is not None else D.get_world_rank()
        self.n_train, self.n_val = len(self.train_set), len(self.val_set)
        bs = int(cfg.local_batch_size)
        if self.n_train < replicas * 1:
            raise ValueError(
                f"The training split has {self.n_train} volume(s) but there are {replicas} data-parallel replicas: "
                "some replica would train on nothing. Use fewer ranks, more spatial shards, or a larger dataset.")
        self.train_sampler = DistributedSampler(self.train_set, num_replicas=replicas, rank=replica, shuffle=True,
                                                seed=int(cfg.training_seed))
        self.val_sampler = UnpaddedDistributedSampler(self.val_set, replicas, replica)
        workers = int(cfg.dataloader_num_workers)
        common = dict(num_workers=workers, pin_memory=self.device.type == "cuda", collate_fn=_collate,
                      persistent_workers=workers > 0)
        if workers > 0:
            common["prefetch_factor"] = 2
        self.train_loader = DataLoader(self.train_set, batch_size=bs, sampler=self.train_sampler, drop_last=False,
                                       **common)
        self.val_loader = DataLoader(self.val_set, batch_size=bs, sampler=self.val_sampler, drop_last=False, **common)
        # the validation set is the same every epoch: after the first pass it is replayed from device memory
        from ..data.device_cache import CachedEvalLoader
        budget = int(float(getattr(cfg, "val_cache_gb", 0.0) or 0.0) * 2 ** 30)
        self.val_batches = CachedEvalLoader(self.val_loader, self.device, budget)
        self.train_batches = PrimedLoader(self.train_loader)
        self.global_batch = bs * replicas
        adiak_value("global_batch_size", self.global_batch)

    def _setup_optimization(self) -> None:
        cfg = self.config
        params = [p for p in self.model.parameters() if p.requires_grad]
        if cfg.optimizer == "ADAM":
            self.optimizer = FusedClipAdam(params, lr=cfg.starting_learning_rate, max_norm=1.0)
        elif cfg.optimizer == "SGD":
            self.optimizer = torch.optim.SGD(params, lr=cfg.starting_learning_rate)
        else:
            self.optimizer = torch.optim.RMSprop(params, lr=cfg.starting_learning_rate, foreach=True)
        self.scheduler = torch.optim.lr_scheduler.CosineAnnealingWarmRestarts(
            self.optimizer, T_0=int(cfg.T_0), T_mult=int(cfg.T_mult), eta_min=float(cfg.min_learning_rate))
        self.grad_scaler = None  # bf16 autocast needs no loss scaling
        self.ce_class_weights = compute_ce_class_weights(self.train_set, int(cfg.n_categories), self.device,
                                                         float(cfg.ce_weight_sample_fraction), self.log)
        self.engine = TrainEngine(self.model, self.optimizer, self.n_classes, self.device, layout=self.layout,
                                  spatial=self.spatial, class_weights=self.ce_class_weights,
                                  amp=bool(cfg.torch_amp), grad_backend=getattr(cfg, "grad_allreduce", "nccl"),
                                  grad_overlap=bool(getattr(cfg, "grad_overlap", False)),
                                  allow_fallback=bool(getattr(cfg, "allow_fallback", False)))
        self._log_kernel_selection()

    def _log_kernel_selection(self) -> None:
        """Once per run, rank 0: the kernel every layer routes to and which peer-memory channels are live
        (role of the start-up report of ScaFFold/utils/trainer.py:808-830)."""
        if self.world_rank != 0:
            return
        from ..ops.selection import effective_backends, format_selection, kernel_selection
        channels = effective_backends(self.engine)
        if self.device.type != "cuda" or not self.engine.amp:
            self.log.info("kernel selection: %s run without bf16 autocast -> every layer runs ATen; channels: %s",
                          self.device.type, channels)
            return
        cfg = self.config
        shards = self.layout.num_shards if self.layout is not None else (1, 1, 1)
        dims = self.layout.shard_dim if self.layout is not None else (2, 3, 4)
        local = [int(cfg.vol_size)] * 3
        for n, d in zip(shards, dims):
            local[d - 2] = -(-local[d - 2] // n)
        k = getattr(self.spatial, "lead_swap", None)
        if k is not None:  # the model works with the split axis exchanged with depth
            local[0], local[k - 2] = local[k - 2], local[0]
        try:
            rows = kernel_selection(self.model, int(cfg.local_batch_size), local, self.spatial)
            self.log.info("kernel selection (local volume %s, batch %s):\n%s", "x".join(map(str, local)),
                          cfg.local_batch_size, format_selection(rows, channels))
        except Exception as exc:  # the report must never stop a run
            self.log.warning("kernel selection report failed: %s", exc)

    # -- reductions -----------------------------------------------------------------
    def _all_reduce_data_parallel(self, t: torch.Tensor) -> None:
        if not dist.is_initialized() or dist.get_world_size() == 1:
            return
        if self.layout is not None:
            if self.layout.ddp_ranks > 1:
                dist.all_reduce(t, group=self.layout.ddp_group)
        else:
            dist.all_reduce(t)

    def _median_minibatch_time(self, events) -> Optional[float]:
        """Per-batch CUDA-event times, max over ranks per batch, then the median (seconds)."""
        if not events:
            return None
        torch.cuda.synchronize()
        t = torch.tensor([a.elapsed_time(b) / 1e3 for a, b in events], device=self.device)
        if dist.is_initialized() and dist.get_world_size() > 1:
            sizes = [None] * dist.get_world_size()
            dist.all_gather_object(sizes, int(t.numel()), group=D.control_group())
            n = min(sizes)
            t = t[:n].contiguous()
            if n == 0:
                return None
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(statistics.median(t.cpu().tolist()))

    # -- resume ------------------------------------------------------------------------
    def cleanup_or_resume(self) -> None:
        cfg = self.config
        resumed = None
        if cfg.train_from_scratch and not getattr(cfg, "restart", False):
            self.checkpoints.wipe()
        else:
            resumed = self.checkpoints.load(self.model, self.optimizer, self.scheduler)
        if resumed is not None:
            self.start_epoch = int(resumed["epoch"]) + 1
            self.start_val_dice = float(resumed.get("val_dice", 0.0) or 0.0)
            self.global_step = int(resumed.get("global_step", 0))
            self.total_optimizer_steps = int(resumed.get("total_optimizer_steps", 0))
            self.log.info("resumed from %s: next epoch %d, val dice %.6f", resumed.get("_loaded_from"),
                          self.start_epoch, self.start_val_dice)
        if self.world_rank == 0:
            self._prepare_csv(resumed is not None)
        D.barrier()

    def _prepare_csv(self, resumed: bool) -> None:
        """Fresh run: header only. Resume: keep the rows of epochs before ``start_epoch``."""
        rows = []
        if resumed and self.outfile_path.exists():
            with open(self.outfile_path) as f:
                for line in f.read().splitlines()[1:]:
                    try:
                        if int(line.split(",")[0]) < self.start_epoch:
                            rows.append(line)
                    except ValueError:
                        continue
        tmp = self.outfile_path.with_suffix(".csv.tmp")
        with open(tmp, "w", newline="") as f:
            f.write(",".join(CSV_COLUMNS) + "\n")
            for line in rows:
                f.write(line + "\n")
        os.replace(tmp, self.outfile_path)

    # -- warm-up -------------------------------------------------------------------------
    def warmup(self) -> None:
        """Run ``warmup_batches`` real steps (also a ragged final batch shape), then restore every state."""
        n = int(self.config.warmup_batches or 0)
        if n <= 0:
            return
        snap = CheckpointManager.snapshot(self.model, self.optimizer, self.scheduler)
        self.model.train()
        done = 0
        ragged = self.n_train_local() % int(self.config.local_batch_size)
        with region("warmup"):
            while done < n:
                for batch in self.train_loader:
                    self.engine.step(batch["image"], batch["mask"])
                    done += 1
                    if done >= n:
                        break
            if ragged:
                batch = next(iter(self.train_loader))
                self.engine.step(batch["image"][:ragged], batch["mask"][:ragged])
            if self.device.type == "cuda":
                torch.cuda.synchronize()
        CheckpointManager.restore(snap, self.model, self.optimizer, self.scheduler)
        D.barrier()

    def n_train_local(self) -> int:
        return len(self.train_sampler)

    # -- the loop ---------------------------------------------------------------------------
    def train(self, profiler=None) -> dict:
        cfg = self.config
        epoch, val_score = self.start_epoch, self.start_val_dice
        epoch_times, minibatch_times = [], []
        last_ckpt_epoch, trained_any = None, False
        val_loss_avg = float("inf")
        vox_per_batch = self.global_batch * int(cfg.vol_size) ** 3
        start = time.time()
        csv = open(self.outfile_path, "a", newline="") if self.world_rank == 0 else None
        try:
            while val_score < cfg.target_dice:
                if cfg.epochs != -1 and epoch > cfg.epochs:
                    self.log.warning("stopping after the configured %s epochs with validation Dice %.4f below the "
                                     "target %s", cfg.epochs, val_score, cfg.target_dice)
                    break
                t0 = time.time()
                self.train_sampler.set_epoch(epoch)
                self.val_sampler.set_epoch(epoch)
                self.model.train()
                loss_sum = torch.zeros((), device=self.device)
                dice_sum = torch.zeros((), device=self.device)
                n_samples, steps, events = 0, 0, []
                full_batches = self.n_train_local() // int(cfg.local_batch_size)
                begin_code_region("batch_loop")
                prefetch = DevicePrefetcher(self.train_batches, self.device)
                for bi, batch in enumerate(prefetch):
                    timed = self.device.type == "cuda" and bi < full_batches
                    if timed:
                        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                        e0.record()
                    with region("run_training_batch"):
                        bs = batch["image"].shape[0]
                        loss = self.engine.step(batch["image"], batch["mask"])
                    if timed:
                        e1.record()
                        events.append((e0, e1))
                    if epoch == self.start_epoch and bi == 0:
                        gather_and_print_mem(self.log, "first_batch", self.device)
                    loss_sum += loss * bs
                    dice_sum += self.engine.last_dice * bs
                    n_samples += bs
                    steps += 1
                    self.global_step += 1
                    self.total_optimizer_steps += 1
                    if profiler is not None:
                        profiler.step()
                end_code_region("batch_loop")
                info = torch.stack([loss_sum, dice_sum, torch.tensor(float(n_samples), device=self.device)]).float()
                self._all_reduce_data_parallel(info)
                g_samples = max(info[2].item(), 1.0)
                epoch_loss_total = info[0].item()
                overall_loss = epoch_loss_total / g_samples
                train_dice = info[1].item() / g_samples
                t_train = time.time() - t0  # the .item() above waited for the last step
                # the next epoch's first batches load while validation runs
                self.train_sampler.set_epoch(epoch + 1)
                self.train_batches.prime()

                d_sum, v_loss_epoch, _, _, n_val = evaluate(self.engine, self.val_batches, progress=self.world_rank == 0)
                vinfo = torch.tensor([d_sum, v_loss_epoch, float(n_val)], device=self.device, dtype=torch.float32)
                self._all_reduce_data_parallel(vinfo)
                g_val = max(vinfo[2].item(), 1.0)
                val_score = vinfo[0].item() / g_val
                v_loss_epoch = vinfo[1].item()
                val_loss_avg = v_loss_epoch / g_val
                if not (math.isfinite(overall_loss) and math.isfinite(val_loss_avg)):
                    raise ValueError(f"Non-finite loss at epoch {epoch} (train_loss={overall_loss}, "
                                     f"val_loss={val_loss_avg}): training diverged, aborting before checkpointing.")
                if not cfg.disable_scheduler:
                    self.scheduler.step()
                duration = time.time() - t0
                epoch_times.append(duration)
                mb = self._median_minibatch_time(events)
                if mb is not None:
                    minibatch_times.append(mb)
                lr = self.optimizer.param_groups[0]["lr"]
                self.log.info(" epoch %d | train_loss=%.6f | val_loss=%.6f | train_dice_score %.6f | val_dice_score "
                              "%.6f | lr %.8f | optimizer_steps %d | total_optimizer_steps %d", epoch, overall_loss,
                              val_loss_avg, train_dice, val_score, lr, steps, self.total_optimizer_steps)
                if csv is not None:
                    csv.write(",".join(str(v) for v in (epoch, epoch_loss_total, overall_loss, v_loss_epoch,
                                                         val_loss_avg, train_dice, val_score, duration, steps,
                                                         self.total_optimizer_steps)) + "\n")
                    csv.flush()
                    extra = (f" Median of minibatch times: {mb:.6f} seconds ({vox_per_batch / mb / 1e6:.2f} "
                             f"Mvoxel/s)." if mb else "")
                    self.log.info("Epoch %s completed in %.6f seconds. Total train time so far: %.6f seconds.%s",
                                  epoch, duration, time.time() - start, extra)
                    self.log.info("Epoch %s phases: training %.3f s (of which the host waited %.3f s for the data "
                                  "loader), validation %.3f s.", epoch, t_train, prefetch.wait_s,
                                  duration - t_train)
                with region("checkpoint"):
                    if cfg.checkpoint_interval > 0 and epoch % cfg.checkpoint_interval == 0:
                        self._save(epoch, val_loss_avg, val_score)
                        last_ckpt_epoch = epoch
                epoch += 1
                trained_any = True
                if math.isnan(val_score):
                    raise ValueError("Invalid value (NaN) encountered in dice score computation")
        finally:
            if csv is not None:
                csv.close()
        completed = epoch - 1
        if not trained_any:
            self.log.warning("No new epoch was trained (start epoch %s, 'epochs' %s, starting val dice %s vs "
                             "target_dice %s): this run had no epoch left to run, and no checkpoint was written.",
                             self.start_epoch, cfg.epochs, self.start_val_dice, cfg.target_dice)
        elif cfg.checkpoint_interval > 0 and completed >= 1 and last_ckpt_epoch != completed:
            self._save(completed, val_loss_avg, val_score)
        self.checkpoints.finalize_saves()
        out = {"final_epochs": completed, "total_optimizer_steps": self.total_optimizer_steps, "val_dice": val_score}
        if epoch_times:
            out["epoch_time_s"] = statistics.median(epoch_times)
            adiak_value("epoch_time_s", out["epoch_time_s"])
            self.log.info("Median of epoch times: %.6f seconds.", out["epoch_time_s"])
        if minibatch_times:
            out["minibatch_time_s"] = statistics.median(minibatch_times)
            out["voxels_per_second"] = vox_per_batch / out["minibatch_time_s"]
            adiak_value("minibatch_time_s", out["minibatch_time_s"])
            adiak_value("voxels_per_second", out["voxels_per_second"])
            self.log.info("Median of epoch minibatch time medians: %.6f seconds (%.2f Mvoxel/s).",
                          out["minibatch_time_s"], out["voxels_per_second"] / 1e6)
        adiak_value("final_epochs", completed)
        adiak_value("total_optimizer_steps", self.total_optimizer_steps)
        return out

    def _save(self, epoch: int, val_loss_avg: float, val_dice: float) -> None:
        extras = {"train_mask_values": self.train_set.mask_values, "global_step": self.global_step,
                  "total_optimizer_steps": self.total_optimizer_steps, "val_dice": val_dice}
        self.checkpoints.save(epoch, val_loss_avg, self.model, self.optimizer, self.scheduler, self.grad_scaler,
                              extras)
