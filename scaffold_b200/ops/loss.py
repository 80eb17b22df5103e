"""Segmentation loss and Dice metric.

``segmentation_loss`` = class-weighted cross entropy + (1 - mean foreground soft
Dice), evaluated in fp32 over the full (possibly spatially sharded) volume:

* CE: sum of per-voxel weighted NLL divided by the sum of the target weights
  (what ``reduction="mean"`` means with class weights), numerator and
  denominator reduced over the spatial shards together
  (ScaFFold/utils/losses.py:117-205);
* soft Dice per (sample, class): ``(2*sum(p*q) + eps) / (sum(p) + sum(q) + eps)``
  with an empty/empty pair scoring 1, averaged over the foreground classes
  (ScaFFold/utils/dice_score.py:101-136, ScaFFold/utils/trainer.py:331-333,660-663).

On CUDA the sums come from one fused pass over the bf16 logits and the
gradient from one more (``csrc/loss.cu``); the only cross-shard traffic is one
all-reduce of ``N*(3C+2)`` floats. The pure-PyTorch formulas below are the CPU
path and the oracle of the GPU tests.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional, Tuple

import torch
import torch.nn.functional as F

from . import _lib

_P = C.c_void_p
_lib.register("sb_loss_blocks", [C.c_longlong], C.c_int)
_lib.register("sb_loss_sums", [_P, _P, C.c_int, _P, _P, _P, C.c_int, C.c_longlong, C.c_int, C.c_int, C.c_int, _P, _P])
_lib.register("sb_loss_grad", [_P, _P, C.c_int, _P, _P, _P, _P, C.c_int, C.c_longlong, C.c_int, C.c_int, _P, _P])

FUSED_MAX_CLASSES = 32  # widest head of csrc/loss.cu (LOSS_MAXC); wider heads take the PyTorch formula


def fused_supported(n_classes: int) -> bool:
    return 1 <= n_classes <= FUSED_MAX_CLASSES

EPS = 1e-6


def labels_to_onehot(labels: torch.Tensor, num_classes: int) -> torch.Tensor:
    """int labels [B, D, H, W] -> float32 one-hot [B, C, D, H, W] (scatter, no int64 intermediate)."""
    b, *spatial = labels.shape
    out = torch.zeros((b, num_classes, *spatial), dtype=torch.float32, device=labels.device)
    out.scatter_(1, labels.long().unsqueeze(1), 1.0)
    return out


def spatial_all_reduce(t: torch.Tensor, spatial) -> torch.Tensor:
    """Sum over the spatial shards; identity gradient (every shard adds its own term)."""
    if spatial is None or spatial.size == 1:
        return t
    return _SpatialAllReduce.apply(t, spatial)


class _SpatialAllReduce(torch.autograd.Function):
    @staticmethod
    def forward(ctx, t, spatial):
        out = t.clone()
        spatial.all_reduce_sum(out)
        return out

    @staticmethod
    def backward(ctx, g):
        return g, None


def dice_from_sums(inter2: torch.Tensor, sets: torch.Tensor, eps: float = EPS) -> torch.Tensor:
    sets = torch.where(sets == 0, inter2, sets)
    return (inter2 + eps) / (sets + eps)


def sharded_dice(preds: torch.Tensor, targets: torch.Tensor, spatial=None, eps: float = EPS) -> torch.Tensor:
    """Dice per (sample, class) of [B, C, D, H, W] tensors, summed over the spatial shards."""
    dims = (-1, -2, -3)
    packed = torch.stack([2.0 * (preds * targets).sum(dims), preds.sum(dims) + targets.sum(dims)])
    packed = spatial_all_reduce(packed, spatial)
    return dice_from_sums(packed[0], packed[1], eps)


def sharded_cross_entropy(log_probs: torch.Tensor, labels: torch.Tensor, class_weights=None, spatial=None):
    ce = F.nll_loss(log_probs, labels.long(), weight=class_weights, reduction="none").sum()
    if class_weights is None:
        den = ce.new_full((), float(labels.numel()))
    else:
        den = class_weights.to(ce.dtype)[labels.long()].sum()
    packed = spatial_all_reduce(torch.stack([ce, den]), spatial)
    return packed[0] / packed[1].clamp_min(torch.finfo(ce.dtype).eps)


def segmentation_loss_reference(logits: torch.Tensor, labels: torch.Tensor, n_classes: int,
                                class_weights: Optional[torch.Tensor] = None, spatial=None):
    """PyTorch formula. logits [B, C, D, H, W] (any float dtype), labels [B, D, H, W]."""
    log_probs = F.log_softmax(logits.float(), dim=1)
    ce = sharded_cross_entropy(log_probs, labels, class_weights, spatial)
    dice = sharded_dice(log_probs.exp(), labels_to_onehot(labels, n_classes), spatial)
    fg = dice[:, 1:].mean()
    return ce + (1.0 - fg), ce.detach(), fg.detach()


# ---------------------------------------------------------------------------
# fused CUDA path
# ---------------------------------------------------------------------------
_LABEL_KIND = {torch.int16: 2, torch.int32: 4, torch.int64: 8}


def _sums(logits_vm: torch.Tensor, labels: torch.Tensor, n_classes: int, cw, argmax: bool) -> torch.Tensor:
    n, d, h, w, cp = logits_vm.shape
    s = d * h * w
    L = _lib.lib()
    blocks = L.sb_loss_blocks(s)
    k = 3 * n_classes + 2
    ws = torch.empty((n, blocks, k), dtype=torch.float32, device=logits_vm.device)
    sums = torch.empty((n, k), dtype=torch.float32, device=logits_vm.device)
    if labels.dtype not in _LABEL_KIND:
        labels = labels.long()
    labels = labels.contiguous()
    _lib.check(L.sb_loss_sums(logits_vm.data_ptr(), labels.data_ptr(), _LABEL_KIND[labels.dtype], _lib.ptr(cw),
                              ws.data_ptr(), sums.data_ptr(), n, s, n_classes, cp, 1 if argmax else 0,
                              _lib.status_tensor(logits_vm.device).data_ptr(), _lib.stream_ptr()), "sb_loss_sums")
    return sums


class _FusedLossFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits_vm, labels, n_classes, cw, spatial):
        c = n_classes
        sums = _sums(logits_vm, labels, c, cw, False)
        if spatial is not None and spatial.size > 1:
            spatial.all_reduce_sum(sums)
        n = sums.shape[0]
        P, Q, I = sums[:, :c], sums[:, c:2 * c], sums[:, 2 * c:3 * c]
        num, den = sums[:, 3 * c].sum(), sums[:, 3 * c + 1].sum()
        den = den.clamp_min(torch.finfo(torch.float32).eps)
        inter2, sets = 2.0 * I, P + Q
        empty = sets == 0
        U = torch.where(empty, inter2, sets)
        dice = (inter2 + EPS) / (U + EPS)
        fg = dice[:, 1:].mean()
        ce = num / den
        # d loss / d p_c(v) = alpha * [y = c] + beta  (foreground classes only)
        m = float(n * (c - 1))
        alpha = -2.0 / (m * (U + EPS))
        beta = (inter2 + EPS) / (m * (U + EPS) ** 2)
        alpha = torch.where(empty, torch.zeros_like(alpha), alpha)
        beta = torch.where(empty, torch.zeros_like(beta), beta)
        alpha[:, 0] = 0
        beta[:, 0] = 0
        ctx.save_for_backward(logits_vm, labels, torch.stack([alpha, beta], 1).contiguous(), den.reshape(1))
        ctx.cw, ctx.c = cw, c
        ctx.mark_non_differentiable(labels)
        return ce + (1.0 - fg), ce, fg

    @staticmethod
    def backward(ctx, g, _gce, _gfg):
        logits_vm, labels, coef, den = ctx.saved_tensors
        n, d, h, w, cp = logits_vm.shape
        coef = (coef * g).contiguous()
        kce = (g / den).reshape(1).float().contiguous()
        dl = torch.empty_like(logits_vm)
        lab = labels if labels.dtype in _LABEL_KIND else labels.long()
        lab = lab.contiguous()
        _lib.check(_lib.lib().sb_loss_grad(logits_vm.data_ptr(), lab.data_ptr(), _LABEL_KIND[lab.dtype],
                                           _lib.ptr(ctx.cw), coef.data_ptr(), kce.data_ptr(), dl.data_ptr(), n,
                                           d * h * w, ctx.c, cp, _lib.status_tensor(logits_vm.device).data_ptr(),
                                           _lib.stream_ptr()), "sb_loss_grad")
        return dl, None, None, None, None


def segmentation_loss_fused(logits_vm: torch.Tensor, labels: torch.Tensor, n_classes: int,
                            class_weights: Optional[torch.Tensor] = None, spatial=None):
    """CUDA: voxel-major bf16 logits ``[N, D, H, W, pad(n_classes)]`` -> (loss, ce, fg_dice)."""
    if class_weights is not None:
        class_weights = class_weights.float().contiguous()
    return _FusedLossFn.apply(logits_vm.contiguous(), labels, n_classes, class_weights, spatial)


def hard_dice_fused(logits_vm: torch.Tensor, labels: torch.Tensor, n_classes: int, spatial=None) -> torch.Tensor:
    """Validation metric: Dice per (sample, class) of the argmax prediction, from fused counts."""
    c = n_classes
    sums = _sums(logits_vm.contiguous(), labels, c, None, True)
    if spatial is not None and spatial.size > 1:
        spatial.all_reduce_sum(sums)
    P, Q, I = sums[:, :c], sums[:, c:2 * c], sums[:, 2 * c:3 * c]
    return dice_from_sums(2.0 * I, P + Q)


def hard_dice_reference(logits: torch.Tensor, labels: torch.Tensor, n_classes: int, spatial=None) -> torch.Tensor:
    pred = F.one_hot(logits.argmax(dim=1), n_classes).permute(0, 4, 1, 2, 3).float()
    return sharded_dice(pred, labels_to_onehot(labels, n_classes), spatial)
