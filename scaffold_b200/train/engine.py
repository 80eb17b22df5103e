"""One training / evaluation step, shared by the trainer and ``bench.py``.

``TrainEngine.step(images, masks)`` is the public per-step call: it moves the
batch to the device (from pinned host memory when it lives there), runs
forward -> fused loss -> backward -> gradient reduction -> clip + Adam, and
returns the loss as a device scalar (reading it is the caller's one host
sync). Mirrors ``PyTorchTrainer._run_training_batch``
(ScaFFold/utils/trainer.py:563-715) with the B200 kernel path underneath.
"""
from __future__ import annotations

from contextlib import nullcontext
from typing import Optional, Tuple

import torch

from ..ops import loss as L
from ..ops.layout import AMP_DTYPE
from ..ops.optim import FusedClipAdam
from ..parallel.ddp import GradReducer
from ..utils.perf import region


class TrainEngine:
    def __init__(self, model, optimizer, n_classes: int, device, layout=None, spatial=None,
                 class_weights: Optional[torch.Tensor] = None, amp: bool = True, grad_backend: str = "nccl",
                 max_norm: float = 1.0, grad_overlap: bool = False, allow_fallback: bool = False):
        self.model, self.optimizer = model, optimizer
        self.n_classes = n_classes
        self.device = torch.device(device)
        self.layout, self.spatial = layout, spatial
        self.class_weights = class_weights
        self.amp = amp
        self.max_norm = max_norm
        self.cuda = self.device.type == "cuda"
        # the fused loss kernels keep one voxel's classes in registers (at most 32); wider heads use the PyTorch formula
        self.fused_loss = self.cuda and self.amp and L.fused_supported(n_classes)
        self.flat = optimizer.attach() if isinstance(optimizer, FusedClipAdam) else None
        params = [p for p in model.parameters() if p.requires_grad]
        self.reducer = GradReducer(layout, flat=self.flat, params=params, backend=grad_backend, overlap=grad_overlap,
                                   allow_fallback=allow_fallback)
        if isinstance(optimizer, FusedClipAdam):
            optimizer.reduce_scale = self.reducer.scale
        self.last_ce = self.last_dice = None
        self._loss_event = None
        self._loss_host = None

    # -- data movement --------------------------------------------------------
    def to_device(self, images: torch.Tensor, masks: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        with region("image_to_device"):
            if self.cuda:
                images = images.to(self.device, non_blocking=True)
                masks = masks.to(self.device, non_blocking=True)
            else:
                images = images.to(self.device, dtype=torch.float32)
                masks = masks.to(self.device)
        return images, masks

    def _autocast(self):
        if not self.amp:
            return nullcontext()
        return torch.autocast(self.device.type, dtype=AMP_DTYPE)

    # -- forward + loss ---------------------------------------------------------
    def forward_loss(self, images: torch.Tensor, masks: torch.Tensor):
        """Returns (loss, ce, foreground soft dice, logits-or-None)."""
        with region("predict"):
            fused = self.fused_loss
            with self._autocast():
                if fused:
                    logits_vm = self.model.forward_padded_logits(images)
                else:
                    logits = self.model(images)
        with region("calculate_loss"):
            if fused:
                if self.spatial is not None and self.spatial.lead_swap is not None:
                    masks = self.spatial.to_kernel_space(masks, first_spatial=1).contiguous()  # as the logits are
                loss, ce, fg = L.segmentation_loss_fused(logits_vm, masks, self.n_classes, self.class_weights,
                                                         self.spatial)
                return loss, ce, fg, (logits_vm, masks)
            with torch.autocast(self.device.type, enabled=False):
                loss, ce, fg = L.segmentation_loss_reference(logits, masks, self.n_classes, self.class_weights,
                                                             self.spatial)
            return loss, ce, fg, logits

    # -- the step ------------------------------------------------------------------
    def step(self, images: torch.Tensor, masks: torch.Tensor, loss_host: Optional[torch.Tensor] = None) -> torch.Tensor:
        """One optimizer step; returns the loss as a device scalar.

        ``loss_host`` (a pinned one-element fp32 tensor) receives the loss by an asynchronous copy enqueued right
        after the forward pass; ``read_loss()`` then returns it without waiting for backward and the update, so a
        loop that looks at every step's loss does not drain the GPU between steps.
        """
        images, masks = self.to_device(images, masks)
        self.optimizer.zero_grad(set_to_none=self.flat is None)
        loss, ce, fg, _ = self.forward_loss(images, masks)
        if loss_host is not None and self.cuda:
            loss_host.copy_(loss.detach().reshape(loss_host.shape), non_blocking=True)
            if self._loss_event is None:
                self._loss_event = torch.cuda.Event()
            self._loss_event.record()
            self._loss_host = loss_host
        elif loss_host is not None:
            loss_host.copy_(loss.detach().reshape(loss_host.shape))
            self._loss_host = loss_host
        with region("backward"):
            loss.backward()
        with region("step_and_update"):
            self.reducer.reduce()
            if not isinstance(self.optimizer, FusedClipAdam):
                params = [p for p in self.model.parameters() if p.grad is not None]
                if self.reducer.scale != 1.0:
                    torch._foreach_mul_([p.grad for p in params], self.reducer.scale)
                torch.nn.utils.clip_grad_norm_(params, self.max_norm)
            self.optimizer.step()
        self.last_ce, self.last_dice = ce.detach(), fg.detach()
        return loss.detach()

    def read_loss(self) -> float:
        """Host value of the loss that the last ``step(..., loss_host=...)`` copied out."""
        if self._loss_host is None:
            raise RuntimeError("read_loss() needs a step(..., loss_host=pinned_tensor) before it")
        if self._loss_event is not None and self.cuda:
            self._loss_event.synchronize()
        return float(self._loss_host.reshape(-1)[0])

    @torch.no_grad()
    def eval_step(self, images: torch.Tensor, masks: torch.Tensor):
        """Returns (loss, hard-dice per (sample, class)) for one validation batch."""
        images, masks = self.to_device(images, masks)
        loss, ce, fg, logits = self.forward_loss(images, masks)
        if self.fused_loss:
            logits, masks = logits  # kernel-space pair of the fused path
            dice = L.hard_dice_fused(logits, masks, self.n_classes, self.spatial)
        else:
            dice = L.hard_dice_reference(logits.float(), masks, self.n_classes, self.spatial)
        return loss, dice
