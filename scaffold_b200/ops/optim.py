"""Fused global-norm clip + Adam over flat parameter and gradient buffers.

``FusedClipAdam`` subclasses ``torch.optim.Adam`` so its ``state_dict`` has the
stock layout (per-parameter ``step`` / ``exp_avg`` / ``exp_avg_sq``), which keeps
checkpoints interchangeable with the reference's ``torch.optim.Adam``
(ScaFFold/utils/trainer.py:257-319). On CUDA all parameters, gradients and
moments are views into four flat fp32 buffers: the clip needs one reduction
kernel, the update one streaming kernel (``csrc/optim.cu``), and the flat
gradient buffer is what the data-parallel reducer communicates.
"""
from __future__ import annotations

import ctypes as C
from typing import Iterable, Optional

import torch

from . import _lib
from .layout import FLAT_GRAD_ATTR, bump_weights_epoch

_P = C.c_void_p
_lib.register("sb_opt_blocks", [C.c_longlong], C.c_int)
_lib.register("sb_grad_norm", [_P, C.c_longlong, _P, _P, _P])
_lib.register("sb_adam_step", [_P, _P, _P, _P, C.c_longlong, C.c_float, C.c_float, C.c_float, C.c_float, C.c_int,
                               C.c_float, _P, C.c_float, _P])


def _align(n: int, a: int = 64) -> int:
    return (n + a - 1) // a * a


class FlatBuffers:
    """Re-homes a module's parameters (and their gradients) into two flat fp32 buffers."""

    def __init__(self, params: Iterable[torch.nn.Parameter]):
        self.params = [p for p in params if p.requires_grad]
        dev = self.params[0].device
        self.offsets, off = [], 0
        for p in self.params:
            self.offsets.append(off)
            off += _align(p.numel())
        self.numel = off
        self.data = torch.zeros(off, dtype=torch.float32, device=dev)
        self.grad = torch.zeros(off, dtype=torch.float32, device=dev)
        for p, o in zip(self.params, self.offsets):
            view = self.data[o:o + p.numel()].view_as(p)
            view.copy_(p.data)
            p.data = view
            p.grad = self.grad[o:o + p.numel()].view_as(p)
            setattr(p, FLAT_GRAD_ATTR, True)

    def rehome_grad(self, new_grad: torch.Tensor) -> None:
        """Move the gradient buffer into ``new_grad`` (e.g. peer-visible memory) and re-point every ``.grad``."""
        if new_grad.numel() != self.numel or new_grad.dtype != torch.float32:
            raise ValueError("replacement gradient buffer must be fp32 with the same number of elements")
        new_grad.copy_(self.grad)
        self.grad = new_grad
        for p, o in zip(self.params, self.offsets):
            p.grad = self.grad[o:o + p.numel()].view_as(p)

    def rebind_grads(self) -> None:
        """Point every ``.grad`` back at the flat buffer (after ``zero_grad(set_to_none=True)``)."""
        for p, o in zip(self.params, self.offsets):
            if p.grad is None or p.grad.data_ptr() != self.grad.data_ptr() + 4 * o:
                p.grad = self.grad[o:o + p.numel()].view_as(p)

    def zero_grad(self) -> None:
        self.grad.zero_()
        self.rebind_grads()


class FusedClipAdam(torch.optim.Adam):
    """Adam whose ``step`` clips the global gradient norm to ``max_norm`` and updates in one pass."""

    def __init__(self, params, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, max_norm: Optional[float] = 1.0):
        params = list(params)
        super().__init__(params, lr=lr, betas=betas, eps=eps, weight_decay=0.0)
        self.max_norm = max_norm
        self.flat: Optional[FlatBuffers] = None
        self._m = self._v = None
        self._norm = None
        self._partials = None
        self._steps = 0
        self.reduce_scale = 1.0  # factor applied to every gradient before clipping (reducer averaging)

    # -- flat state -------------------------------------------------------
    def _ensure_flat(self) -> bool:
        if self.flat is not None:
            return True
        ps = [p for g in self.param_groups for p in g["params"] if p.requires_grad]
        if not ps or not all(p.is_cuda and p.dtype == torch.float32 for p in ps) or len(self.param_groups) != 1:
            return False
        self.flat = FlatBuffers(ps)
        dev = self.flat.data.device
        self._m = torch.zeros_like(self.flat.data)
        self._v = torch.zeros_like(self.flat.data)
        self._norm = torch.zeros(1, dtype=torch.float32, device=dev)
        self._partials = torch.zeros(_lib.lib().sb_opt_blocks(self.flat.numel), dtype=torch.float32, device=dev)
        self._step_t = torch.tensor(0.0)  # one host tensor shared by every parameter's state
        for p, o in zip(self.flat.params, self.flat.offsets):
            st = self.state[p]
            old_m, old_v = st.get("exp_avg"), st.get("exp_avg_sq")
            st["exp_avg"] = self._m[o:o + p.numel()].view_as(p)
            st["exp_avg_sq"] = self._v[o:o + p.numel()].view_as(p)
            if old_m is not None:
                st["exp_avg"].copy_(old_m)
                st["exp_avg_sq"].copy_(old_v)
            step = st.get("step")
            if step is not None:
                self._steps = int(step.item() if torch.is_tensor(step) else step)
            st["step"] = self._step_t
        self._step_t.fill_(float(self._steps))
        return True

    def attach(self) -> Optional[FlatBuffers]:
        """Flatten now (CUDA only) and return the buffers; ``None`` on CPU."""
        return self.flat if self._ensure_flat() else None

    def load_state_dict(self, state_dict):
        super().load_state_dict(state_dict)
        if self.flat is not None:
            # re-home the loaded moments into the flat buffers
            for p, o in zip(self.flat.params, self.flat.offsets):
                st = self.state[p]
                self._m[o:o + p.numel()].view_as(p).copy_(st["exp_avg"])
                self._v[o:o + p.numel()].view_as(p).copy_(st["exp_avg_sq"])
                st["exp_avg"] = self._m[o:o + p.numel()].view_as(p)
                st["exp_avg_sq"] = self._v[o:o + p.numel()].view_as(p)
                step = st.get("step", 0)
                self._steps = int(step.item() if torch.is_tensor(step) else step)
                st["step"] = self._step_t
            self._step_t.fill_(float(self._steps))

    def zero_grad(self, set_to_none: bool = True):
        if self.flat is not None:
            self.flat.zero_grad()
        else:
            super().zero_grad(set_to_none=set_to_none)

    @property
    def grad_norm(self) -> Optional[torch.Tensor]:
        """Device scalar: the pre-clip global gradient norm of the last step (CUDA path)."""
        return self._norm

    @torch.no_grad()
    def step(self, closure=None):
        if not self._ensure_flat():
            # CPU / mixed placement: clip with torch, step with the stock implementation
            if self.max_norm is not None:
                ps = [p for g in self.param_groups for p in g["params"] if p.grad is not None]
                if self.reduce_scale != 1.0:
                    for p in ps:
                        p.grad.mul_(self.reduce_scale)
                torch.nn.utils.clip_grad_norm_(ps, self.max_norm)
            return super().step(closure)
        f = self.flat
        f.rebind_grads()
        g = self.param_groups[0]
        L = _lib.lib()
        s = _lib.stream_ptr()
        max_norm = float(self.max_norm) if self.max_norm is not None else -1.0
        if max_norm > 0:
            _lib.check(L.sb_grad_norm(f.grad.data_ptr(), f.numel, self._partials.data_ptr(), self._norm.data_ptr(), s),
                       "sb_grad_norm")
        self._steps += 1
        b1, b2 = g["betas"]
        _lib.check(L.sb_adam_step(f.data.data_ptr(), f.grad.data_ptr(), self._m.data_ptr(), self._v.data_ptr(),
                                  f.numel, float(g["lr"]), float(b1), float(b2), float(g["eps"]), self._steps,
                                  max_norm, self._norm.data_ptr(), float(self.reduce_scale), s), "sb_adam_step")
        self._step_t.fill_(float(self._steps))
        bump_weights_epoch()
        from .conv3d import repack_all
        repack_all()  # one launch refreshes the bf16 operand copies of every convolution for the next step
        return None
