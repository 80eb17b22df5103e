"""Process-group bring-up and the Python-object control plane.

Replaces the reference's two transports (torch.distributed for tensors, mpi4py
for Python objects; ScaFFold/utils/distributed.py:28-306, ScaFFold/cli.py:584-662)
with one: ``torch.distributed``. Rank and world size come from whichever
launcher started the job (torchrun, Open MPI, MVAPICH, PMI/PALS, Slurm, Flux);
the device is bound *before* the first collective; the backend is ``nccl`` when
CUDA is visible, else ``gloo``. The control-plane helpers implement the
decide-on-rank-0-and-broadcast protocol: every rank-0-only action publishes its
outcome, so a failure on one rank is raised on every rank instead of hanging
the others.
"""
from __future__ import annotations

import datetime
import os
import pickle
from typing import Any, Callable, List, Optional, Sequence

import torch
import torch.distributed as dist

# launcher -> environment variable, in priority order
_RANK_VARS = ("RANK", "OMPI_COMM_WORLD_RANK", "MV2_COMM_WORLD_RANK", "PMI_RANK", "PMIX_RANK", "PALS_RANKID",
              "SLURM_PROCID", "FLUX_TASK_RANK")
_SIZE_VARS = ("WORLD_SIZE", "OMPI_COMM_WORLD_SIZE", "MV2_COMM_WORLD_SIZE", "PMI_SIZE", "PALS_NRANKS",
              "SLURM_NTASKS", "FLUX_JOB_SIZE")
_LOCAL_RANK_VARS = ("LOCAL_RANK", "OMPI_COMM_WORLD_LOCAL_RANK", "MV2_COMM_WORLD_LOCAL_RANK", "MPI_LOCALRANKID",
                    "PALS_LOCAL_RANKID", "SLURM_LOCALID", "FLUX_TASK_LOCAL_ID")
_LOCAL_SIZE_VARS = ("LOCAL_WORLD_SIZE", "OMPI_COMM_WORLD_LOCAL_SIZE", "MV2_COMM_WORLD_LOCAL_SIZE",
                    "MPI_LOCALNRANKS", "PALS_LOCAL_SIZE", "SLURM_NTASKS_PER_NODE", "SLURM_TASKS_PER_NODE")


def _to_int(text: Optional[str]) -> Optional[int]:
    """Tolerant integer parse: '4', ' 4 ', '4(x2)' (Slurm task lists) -> 4; anything else -> None."""
    if text is None:
        return None
    text = text.strip()
    digits = ""
    for ch in text:
        if ch.isdigit():
            digits += ch
        else:
            break
    return int(digits) if digits else None


def _first_env(names: Sequence[str]) -> Optional[int]:
    for n in names:
        v = _to_int(os.environ.get(n))
        if v is not None:
            return v
    return None


def get_world_rank() -> int:
    if dist.is_available() and dist.is_initialized():
        return dist.get_rank()
    return _first_env(_RANK_VARS) or 0


def get_world_size() -> int:
    if dist.is_available() and dist.is_initialized():
        return dist.get_world_size()
    return _first_env(_SIZE_VARS) or 1


def get_local_rank() -> int:
    v = _first_env(_LOCAL_RANK_VARS)
    if v is not None:
        return v
    n = torch.cuda.device_count() if torch.cuda.is_available() else 0
    return get_world_rank() % n if n else 0


def get_local_size() -> int:
    v = _first_env(_LOCAL_SIZE_VARS)
    if v is not None:
        return v
    return min(get_world_size(), torch.cuda.device_count() or 1) if torch.cuda.is_available() else get_world_size()


def get_device() -> torch.device:
    """The device of this rank. A launcher that masks GPUs per rank leaves exactly one visible: use it."""
    if not torch.cuda.is_available():
        return torch.device("cpu")
    n = torch.cuda.device_count()
    return torch.device("cuda", 0 if n == 1 else get_local_rank() % n)


def initialize_dist(rendezvous: str = "env", timeout_s: int = 1800, init_file: Optional[str] = None) -> torch.device:
    """Create the default process group (idempotent) and return this rank's device."""
    device = get_device()
    if device.type == "cuda":
        torch.cuda.set_device(device)  # before the first collective, so NCCL binds the right GPU
    if dist.is_initialized():
        return device
    rank, world = get_world_rank(), get_world_size()
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29500")
    backend = "nccl" if device.type == "cuda" else "gloo"
    kwargs = dict(backend=backend, rank=rank, world_size=world, timeout=datetime.timedelta(seconds=timeout_s))
    if rendezvous == "env":
        os.environ.setdefault("RANK", str(rank))
        os.environ.setdefault("WORLD_SIZE", str(world))
        kwargs["init_method"] = "env://"
    elif rendezvous == "tcp":
        kwargs["init_method"] = f"tcp://{os.environ['MASTER_ADDR']}:{os.environ['MASTER_PORT']}"
    elif rendezvous == "file":
        if not init_file:
            raise ValueError("file rendezvous needs init_file")
        kwargs["init_method"] = f"file://{init_file}"
    else:
        raise ValueError(f"unknown rendezvous {rendezvous!r}")
    if backend == "nccl":
        kwargs["device_id"] = device
    dist.init_process_group(**kwargs)
    dist.barrier()
    return device


def check_launcher_world_size() -> None:
    """The launcher's idea of the world (env) and the process group's must agree."""
    env = _first_env(_SIZE_VARS)
    if env is not None and dist.is_initialized() and env != dist.get_world_size():
        raise RuntimeError(
            f"launcher reports {env} ranks but the process group has {dist.get_world_size()}; "
            "the job was started with mismatched launch parameters")


# ---------------------------------------------------------------------------
# control plane (Python objects)
# ---------------------------------------------------------------------------
_control_group = None


def control_group():
    """A gloo group over all ranks for object collectives (NCCL groups pickle through the GPU)."""
    global _control_group
    if not dist.is_initialized() or dist.get_world_size() == 1:
        return None
    if dist.get_backend() == "gloo":
        return None  # the default group already is gloo
    if _control_group is None:
        _control_group = dist.new_group(backend="gloo")
    return _control_group


def barrier() -> None:
    if dist.is_initialized() and dist.get_world_size() > 1:
        dist.barrier()


def bcast_obj(obj: Any, src: int = 0) -> Any:
    if not dist.is_initialized() or dist.get_world_size() == 1:
        return obj
    box = [obj if dist.get_rank() == src else None]
    dist.broadcast_object_list(box, src=src, group=control_group())
    return box[0]


def allgather_obj(obj: Any) -> List[Any]:
    if not dist.is_initialized() or dist.get_world_size() == 1:
        return [obj]
    out: List[Any] = [None] * dist.get_world_size()
    dist.all_gather_object(out, obj, group=control_group())
    return out


def allreduce_min_int(value: int) -> int:
    if not dist.is_initialized() or dist.get_world_size() == 1:
        return int(value)
    return min(allgather_obj(int(value)))


def allreduce_sum_int(value: int) -> int:
    if not dist.is_initialized() or dist.get_world_size() == 1:
        return int(value)
    return sum(allgather_obj(int(value)))


class RemoteError(RuntimeError):
    """An exception raised on another rank, re-raised here so that every rank fails together."""


def _describe(exc: BaseException) -> dict:
    return {"type": type(exc).__name__, "module": type(exc).__module__, "message": str(exc),
            "rank": get_world_rank()}


def rebuild_error(info: dict) -> BaseException:
    """Same exception class when it is a builtin, else ``RemoteError``, with the origin rank in the text."""
    import builtins
    cls = getattr(builtins, info["type"], None)
    text = f"[rank {info['rank']}] {info['message']}"
    if isinstance(cls, type) and issubclass(cls, Exception):
        try:
            return cls(text)
        except Exception:
            pass
    return RemoteError(f"{info['type']}: {text}")


def run_on_root(fn: Callable[[], Any], root: int = 0) -> Any:
    """Run ``fn`` on ``root`` only, broadcast ``(error, result)``: all ranks return or raise alike.

    ``KeyboardInterrupt`` on the root is re-raised there verbatim after the
    others have been told.
    """
    rank = get_world_rank()
    err, result, interrupt = None, None, None
    if rank == root:
        try:
            result = fn()
        except KeyboardInterrupt as exc:  # tell the others, then re-raise here
            interrupt = exc
            err = _describe(exc)
        except Exception as exc:
            err = _describe(exc)
    err, result = bcast_obj((err, result), src=root)
    if interrupt is not None:
        raise interrupt
    if err is not None:
        raise rebuild_error(err)
    return result


def consensus(ok: bool, message: str = "") -> None:
    """Every rank reports success/failure; if any failed, all raise with the collected messages."""
    reports = allgather_obj((bool(ok), message, get_world_rank()))
    failed = [(r, m) for good, m, r in reports if not good]
    if failed:
        raise RemoteError("; ".join(f"rank {r}: {m}" for r, m in failed))
