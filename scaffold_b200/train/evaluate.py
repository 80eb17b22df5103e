"""Validation pass (ScaFFold/utils/evaluate.py:27-254).

Runs under ``no_grad`` with the same forward + loss as training; the metric is
the hard (argmax) Dice averaged over the foreground classes, per sample. Sums are
sample-weighted and kept on the device; the host reads them once at the end.
Returns ``(dice_sum, val_loss_sum, val_loss_avg, n_batches, n_samples)`` for
this rank; the caller reduces over the data-parallel replicas.
"""
from __future__ import annotations

import sys

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
    if progress and sys.stderr.isatty():  # a progress bar only where someone watches; logs stay clean
        from tqdm import tqdm
        it = tqdm(dataloader, desc="validation", unit="batch", leave=False)
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
    if device.type == "cuda":
        from ..ops import _lib
        _lib.check_status(device)  # a bounded device wait that ran out, or a label the loss kernel refused
    return d, l, (l / n_samples if n_samples else 0.0), n_batches, n_samples
