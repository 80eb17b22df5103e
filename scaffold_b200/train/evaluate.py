"""Validation pass (ScaFFold/utils/evaluate.py:27-254).

Runs under ``no_grad`` with the same forward + loss as training; the metric is
the hard (argmax) Dice averaged over the foreground classes, per sample. Sums are
sample-weighted and kept on the device; the host reads them once at the end.
Returns ``(dice_sum, val_loss_sum, val_loss_avg, n_batches, n_samples)`` for
this rank; the caller reduces over the data-parallel replicas.
"""
from __future__ import annotations

import torch


@torch.no_grad()
def evaluate(engine, dataloader, progress: bool = False):
    model = engine.model
    was_training = model.training
    model.eval()
    device = engine.device
    dice_sum = torch.zeros((), device=device)
    loss_sum = torch.zeros((), device=device)
    n_batches = n_samples = 0
    it = dataloader
    if progress:
        try:
            from tqdm import tqdm
            it = tqdm(dataloader, desc="Validation round", unit="batch", leave=False, disable=True)
        except Exception:
            it = dataloader
    for batch in it:
        bs = batch["image"].shape[0]
        loss, dice = engine.eval_step(batch["image"], batch["mask"])
        dice_sum += dice[:, 1:].mean(dim=1).sum()
        loss_sum += loss * bs
        n_batches += 1
        n_samples += bs
    if was_training:
        model.train()
    d, l = float(dice_sum.item()), float(loss_sum.item())  # the one host sync
    return d, l, (l / n_samples if n_samples else 0.0), n_batches, n_samples
