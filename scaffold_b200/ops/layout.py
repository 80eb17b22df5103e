"""Activation layout helpers.

Modules exchange ordinary NCDHW-shaped tensors whose memory is channels-last
(``torch.channels_last_3d``); the kernels see the same memory as a contiguous
voxel-major ``[N, D, H, W, C]`` tensor. Both conversions are views when the
memory format already matches.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

AMP_DTYPE = torch.bfloat16


_aten_only = [False]


class aten_only:
    """Context manager: route every module through ATen (the oracle of the parity tests)."""

    def __enter__(self):
        self._old = _aten_only[0]
        _aten_only[0] = True
        return self

    def __exit__(self, *exc):
        _aten_only[0] = self._old


def use_cuda_kernels(x: torch.Tensor) -> bool:
    """True when the sm_100a kernel path applies: CUDA tensor, bf16 or autocast-to-bf16."""
    if not x.is_cuda or _aten_only[0]:
        return False
    if x.dtype == torch.bfloat16:
        return True
    return torch.is_autocast_enabled("cuda") and torch.get_autocast_dtype("cuda") == torch.bfloat16


def to_vm(x: torch.Tensor, pad16: bool = False, pad_to: int = 16) -> torch.Tensor:
    """NCDHW-shaped tensor -> contiguous voxel-major bf16 ``[N, D, H, W, C]``."""
    if (pad16 and x.is_cuda and x.dim() == 5 and x.shape[1] < 16 and x.is_contiguous()
            and x.dtype in (torch.float32, torch.bfloat16) and not x.requires_grad):
        # input staging kernel: layout change + down-cast + channel padding in one pass
        from . import _lib
        n, c, d, h, w = x.shape
        y = torch.empty((n, d, h, w, pad_to), dtype=torch.bfloat16, device=x.device)
        _lib.check(_lib.lib().sb_stage_input(x.data_ptr(), int(x.dtype == torch.bfloat16), n, c, d * h * w,
                                             y.data_ptr(), pad_to, _lib.stream_ptr()), "sb_stage_input")
        return y
    v = x.permute(0, 2, 3, 4, 1)
    if v.dtype != torch.bfloat16:
        v = v.to(torch.bfloat16)
    c = v.shape[4]
    if pad16 and c % pad_to != 0:
        v = F.pad(v, (0, pad_to - c % pad_to))
    return v.contiguous()


def from_vm(y: torch.Tensor) -> torch.Tensor:
    """Voxel-major ``[N, D, H, W, C]`` -> NCDHW-shaped view (channels-last memory)."""
    return y.permute(0, 4, 1, 2, 3)


# Parameters updated through raw pointers (the fused optimizer) do not bump the
# tensors' version counters; packed operand caches also key on this epoch.
_weights_epoch = [0]


def bump_weights_epoch() -> None:
    _weights_epoch[0] += 1


def weights_epoch() -> int:
    return _weights_epoch[0]


# Parameters whose ``.grad`` is a view into a flat gradient buffer (set up by the fused optimizer) are marked
# with this attribute; the convolution backward passes then add their weight gradient straight into that view
# (no temporary tensor, no autograd accumulation kernel) and tell the listeners below that it is there.
FLAT_GRAD_ATTR = "_sb_flat_grad"
_grad_written_listeners = []


def direct_grad_target(param):
    """The flat-buffer gradient view of ``param`` when the kernels may accumulate into it directly, else None."""
    if not getattr(param, FLAT_GRAD_ATTR, False):
        return None
    g = param.grad
    if g is None or g.dtype != torch.float32 or not g.is_contiguous() or g.shape != param.shape:
        return None
    return g


def add_grad_written_listener(fn) -> None:
    """Register a bound method (held weakly: a reducer that is dropped stops listening by itself)."""
    import weakref
    _grad_written_listeners.append(weakref.WeakMethod(fn) if hasattr(fn, "__self__") else (lambda f=fn: f))


def remove_grad_written_listener(fn) -> None:
    _grad_written_listeners[:] = [r for r in _grad_written_listeners if r() is not None and r() != fn]


def notify_grad_written(param) -> None:
    """Called by a backward pass that wrote ``param.grad`` itself (autograd's accumulate hooks do not fire then)."""
    dead = False
    for ref in list(_grad_written_listeners):
        fn = ref()
        if fn is None:
            dead = True
        else:
            fn(param)
    if dead:
        _grad_written_listeners[:] = [r for r in _grad_written_listeners if r() is not None]
