"""ctypes binding of ``libscaffold_b200.so`` (see ``csrc/host_api.h``).

The library is looked up in-tree (``scaffold_b200/_native``). On a machine
with a GPU a missing library is an error, never a silent fallback: the CUDA
code paths of :mod:`scaffold_b200.ops` call :func:`lib` and raise.
"""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

import torch

_NATIVE = Path(__file__).resolve().parent.parent / "_native" / "libscaffold_b200.so"
_lib = None

ERRORS = {
    1: "driver entry point unavailable",
    2: "TMA alignment rule violated (16-byte base / stride)",
    3: "cuTensorMapEncodeTiled refused the tensor description",
    4: "shape not supported by the kernel",
    5: "kernel launch failed",
    6: "request exceeds a fixed capacity",
}


class NativeError(RuntimeError):
    pass


class SbConvArgs(C.Structure):
    _fields_ = [
        ("src", C.c_void_p * 2),
        ("src_c", C.c_int * 2),
        ("src_ld", C.c_int * 2),
        ("N", C.c_int), ("D", C.c_int), ("H", C.c_int), ("W", C.c_int),
        ("ksize", C.c_int),
        ("wpack", C.c_void_p),
        ("cout_pad", C.c_int),
        ("dst", C.c_void_p * 2),
        ("dst_c", C.c_int * 2),
        ("dst_ld", C.c_int * 2),
        ("bias", C.c_void_p),
        ("status", C.c_void_p),
        ("force_plain", C.c_int),
        ("in_d", C.c_int), ("in_h", C.c_int), ("in_w", C.c_int),
        ("off_d", C.c_int), ("off_h", C.c_int), ("off_w", C.c_int),
        ("halo_land", (C.c_void_p * 2) * 2),
        ("halo_flag", C.c_void_p * 2),
        ("halo_epoch", C.c_uint),
        ("halo_wait_s", C.c_double),
        ("slab_out", C.c_void_p * 2),
        ("slab_ld", C.c_int),
        ("wpack_kd", C.c_void_p),
        ("workspace", C.c_void_p),
        ("workspace_elems", C.c_longlong),
        ("gn_part", C.c_void_p),
        ("gn_groups", C.c_int),
    ]


class SbPackArgs(C.Structure):
    _fields_ = [
        ("w", C.c_void_p),
        ("cout", C.c_int), ("cin", C.c_int), ("real0", C.c_int), ("pad0", C.c_int),
        ("cin_pad", C.c_int), ("cout_pad", C.c_int),
        ("fwd", C.c_void_p), ("fwd_kd", C.c_void_p), ("dgrad", C.c_void_p), ("dgrad_kd", C.c_void_p),
        ("tap_swap", C.c_int),
    ]


class SbPackJob(C.Structure):
    _fields_ = [("a", SbPackArgs), ("tile0", C.c_int), ("tiles_x", C.c_int)]


class SbConvTArgs(C.Structure):
    _fields_ = [
        ("src", C.c_void_p),
        ("src_ld", C.c_int),
        ("N", C.c_int), ("D", C.c_int), ("H", C.c_int), ("W", C.c_int),
        ("cin", C.c_int), ("cout", C.c_int),
        ("wpack", C.c_void_p),
        ("wrows", C.c_int),
        ("dst", C.c_void_p),
        ("dst_ld", C.c_int),
        ("bias", C.c_void_p),
        ("status", C.c_void_p),
    ]


class SbWgradArgs(C.Structure):
    _fields_ = [
        ("gy", C.c_void_p),
        ("gy_c", C.c_int), ("gy_ld", C.c_int),
        ("x", C.c_void_p * 2),
        ("x_c", C.c_int * 2), ("x_ld", C.c_int * 2),
        ("N", C.c_int), ("D", C.c_int), ("H", C.c_int), ("W", C.c_int),
        ("ksize", C.c_int),
        ("workspace", C.c_void_p),
        ("workspace_elems", C.c_longlong),
        ("dw", C.c_void_p),
        ("dw_cout", C.c_int), ("dw_cin", C.c_int),
        ("accumulate", C.c_int),
        ("status", C.c_void_p),
        ("splits", C.c_int),
        ("xin_d", C.c_int), ("xin_h", C.c_int), ("xin_w", C.c_int),
        ("xoff_d", C.c_int), ("xoff_h", C.c_int), ("xoff_w", C.c_int),
        ("xhalo", (C.c_void_p * 2) * 2),
        ("tap_swap", C.c_int),
    ]


def available() -> bool:
    return _NATIVE.exists()


def lib() -> C.CDLL:
    """The loaded native library; builds it first if nvcc is present and it is missing."""
    global _lib
    if _lib is not None:
        return _lib
    if not _NATIVE.exists():
        if os.environ.get("SCAFFOLD_B200_NO_AUTOBUILD", "0") != "1":
            from ..build import build_native

            build_native()
        if not _NATIVE.exists():
            raise NativeError(
                f"{_NATIVE} is missing; run `python -m scaffold_b200.build` (needs nvcc). "
                "The CUDA paths have no framework fallback."
            )
    handle = C.CDLL(str(_NATIVE))
    for name, argt in _SIGNATURES.items():
        fn = getattr(handle, name, None)
        if fn is None:
            continue
        fn.argtypes = argt[0]
        fn.restype = argt[1]
    _lib = handle
    return handle


_P = C.c_void_p
_SIGNATURES = {
    "sb_conv_fwd": ([C.POINTER(SbConvArgs), _P], C.c_int),
    "sb_conv_fwd_workspace": ([C.POINTER(SbConvArgs)], C.c_longlong),
    "sb_conv_gn_splits": ([C.POINTER(SbConvArgs)], C.c_int),
    "sb_conv_pair_plan": ([C.POINTER(SbConvArgs), C.c_int, C.POINTER(C.c_int), C.POINTER(C.c_int)], C.c_int),
    "sb_pack_conv3": ([C.POINTER(SbPackArgs), _P], C.c_int),
    "sb_pack_conv3_plan": ([C.POINTER(SbPackJob), C.c_int], C.c_longlong),
    "sb_pack_conv3_batch": ([_P, C.c_int, C.c_longlong, _P], C.c_int),
    "sb_stage_input": ([_P, C.c_int, C.c_int, C.c_int, C.c_longlong, _P, C.c_int, _P], C.c_int),
    "sb_colsum_blocks": ([], C.c_int),
    "sb_colsum": ([_P, C.c_longlong, C.c_int, _P, C.c_int, _P, _P], C.c_int),
    "sb_convT_fwd": ([C.POINTER(SbConvTArgs), _P], C.c_int),
    "sb_convT_dgrad": ([C.POINTER(SbConvTArgs), _P], C.c_int),
    "sb_conv_wgrad": ([C.POINTER(SbWgradArgs), _P], C.c_int),
    "sb_conv_wgrad_workspace": ([C.POINTER(SbWgradArgs)], C.c_longlong),
    "sb_launch_count": ([], C.c_longlong),
}


def register(name: str, argtypes, restype=C.c_int) -> None:
    """Declare the signature of one more entry point (used by the op modules)."""
    _SIGNATURES[name] = (argtypes, restype)
    if _lib is not None:
        fn = getattr(_lib, name)
        fn.argtypes = argtypes
        fn.restype = restype


def launch_count() -> int:
    """Kernels launched by the native library so far in this process."""
    return int(lib().sb_launch_count())


def check(rc: int, what: str) -> None:
    if rc != 0:
        raise NativeError(f"{what}: {ERRORS.get(rc, 'error')} (code {rc})")


def stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


def ptr(t) -> int:
    return 0 if t is None else t.data_ptr()


# ---------------------------------------------------------------------------
# Status words: device-side bounded waits report here instead of hanging.
# ---------------------------------------------------------------------------
_status = {}

SITES = {
    1: "conv producer waiting for a free stage",
    2: "conv MMA waiting for a free accumulator",
    3: "conv MMA waiting for operands",
    4: "conv epilogue waiting for the accumulator",
    11: "wgrad producer waiting for a free stage",
    12: "wgrad MMA waiting for operands",
    13: "wgrad epilogue waiting for the accumulator",
    21: "plane conv: activation producer waiting for a free slot",
    22: "plane conv: weight producer waiting for a free slot",
    23: "plane conv: MMA waiting for a weight tap",
    24: "plane conv: MMA waiting for an activation plane",
    25: "plane conv: MMA waiting for a free accumulator",
    26: "plane conv: epilogue waiting for the accumulators",
    27: "plane conv: waiting for a neighbour's halo plane",
    51: "halo accumulate: waiting for a neighbour's gradient slab",
    31: "plane wgrad: producer waiting for a free stage",
    32: "plane wgrad: MMA waiting for operands",
    33: "plane wgrad: epilogue waiting for the accumulators",
    41: "gradient all-reduce: waiting for the peers' gradients",
    42: "gradient all-reduce: waiting for the peers' completion",
    61: "fused loss: a label outside [0, n_classes) (detail = label value, sample); the voxel was skipped",
    62: "fused loss gradient: a label outside [0, n_classes) (detail = label value, sample); the voxel was skipped",
}

CODES = {1: "mbarrier wait ran out", 2: "flag wait ran out", 3: "bad argument seen on the device"}


class DeviceArgumentError(RuntimeError):
    """A kernel met data it refuses to use (e.g. a label outside the class range) and skipped it."""


class DeviceWaitTimeout(RuntimeError):
    """A bounded device-side wait ran out (the kernel returned instead of hanging)."""


def status_tensor(device) -> torch.Tensor:
    key = torch.device(device).index or 0
    t = _status.get(key)
    if t is None:
        t = torch.zeros(4, dtype=torch.int32, device=device)
        _status[key] = t
    return t


def check_status(device=None) -> None:
    """Host read of the status word (synchronises); raises if a wait timed out."""
    for key, t in list(_status.items()):
        if device is not None and (torch.device(device).index or 0) != key:
            continue
        v = t.cpu().tolist()
        if v[0] == 3:
            t.zero_()
            raise DeviceArgumentError(
                f"{SITES.get(v[1], 'site %d' % v[1])}: detail {v[2] if v[2] < 2 ** 31 else v[2] - 2 ** 32}, {v[3]}")
        if v[0] != 0:
            t.zero_()
            raise DeviceWaitTimeout(
                f"device status code {v[0]} at site {v[1]} ({SITES.get(v[1], '?')}), detail {v[2]}, {v[3]}"
            )
