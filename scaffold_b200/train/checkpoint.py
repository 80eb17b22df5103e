"""Checkpoint / resume.

File format and protocol kept from ScaFFold/utils/checkpointing.py:29-796: one
``torch.save`` dict with ``epoch``, ``val_loss_avg``, ``model_state_dict`` (of the
unwrapped module), ``optimizer_state_dict``, ``grad_scaler_state_dict``,
``scheduler_state_dict``, ``rng_state_pytorch``, ``rng_state_pytorch_cuda``,
``rng_state_numpy``, ``rng_state_python`` plus caller extras, stored as
``<run_dir>/<checkpoint_dir>/checkpoint_last.pth`` and ``checkpoint_best.pth``
(best = lowest ``val_loss_avg``, written as a byte copy of last).

* only rank 0 writes: temp file + fsync + ``os.replace`` (atomic); orphaned temp
  files of a killed run are swept at start-up;
* every save outcome is broadcast, so all ranks raise ``CheckpointSaveError``
  together; with ``async_save`` a single writer thread does the I/O and the
  outcome of save N is collected at save N+1 or ``finalize_saves``;
* on resume rank 0 reads the file and the state is broadcast; a corrupt
  ``last`` is quarantined as ``.corrupt`` and ``best`` is tried instead;
* host-side ``snapshot`` / ``restore`` let the warm-up run real steps and then
  put model, optimizer, scheduler and RNG streams back.
"""
from __future__ import annotations

import copy
import os
import random
import shutil
import threading
from concurrent.futures import Future, ThreadPoolExecutor
from pathlib import Path
from typing import Any, Dict, Optional

import numpy as np
import torch

from ..utils import dist as D

LAST_NAME = "checkpoint_last.pth"
BEST_NAME = "checkpoint_best.pth"
TMP_MARK = ".tmp-ckpt-"


class CheckpointSaveError(RuntimeError):
    pass


def capture_rng() -> Dict[str, Any]:
    return {
        "rng_state_pytorch": torch.get_rng_state(),
        "rng_state_pytorch_cuda": torch.cuda.get_rng_state_all() if torch.cuda.is_available() else [],
        "rng_state_numpy": np.random.get_state(),
        "rng_state_python": random.getstate(),
    }


def restore_rng(state: Dict[str, Any]) -> None:
    if state.get("rng_state_pytorch") is not None:
        torch.set_rng_state(state["rng_state_pytorch"].cpu() if torch.is_tensor(state["rng_state_pytorch"])
                            else state["rng_state_pytorch"])
    cuda = state.get("rng_state_pytorch_cuda")
    if cuda and torch.cuda.is_available() and len(cuda) == torch.cuda.device_count():
        torch.cuda.set_rng_state_all([s.cpu() for s in cuda])
    if state.get("rng_state_numpy") is not None:
        np.random.set_state(state["rng_state_numpy"])
    if state.get("rng_state_python") is not None:
        random.setstate(state["rng_state_python"])


def _to_host(obj):
    if torch.is_tensor(obj):
        return obj.detach().to("cpu", copy=True)
    if isinstance(obj, dict):
        return {k: _to_host(v) for k, v in obj.items()}
    if isinstance(obj, (list, tuple)):
        return type(obj)(_to_host(v) for v in obj)
    return copy.deepcopy(obj)


class CheckpointManager:
    def __init__(self, run_dir, checkpoint_dir: str = "checkpoints", async_save: bool = False, log=None):
        self.dir = Path(run_dir) / checkpoint_dir
        self.last_path, self.best_path = self.dir / LAST_NAME, self.dir / BEST_NAME
        self.log = log
        self.rank = D.get_world_rank()
        self.best_val_loss = float("inf")
        self._best_before_pending = float("inf")  # value to return to when an asynchronous write fails
        self.async_save = bool(async_save)
        self._pool: Optional[ThreadPoolExecutor] = ThreadPoolExecutor(max_workers=1) if self.async_save else None
        self._pending: Optional[Future] = None
        self._lock = threading.Lock()
        if self.rank == 0:
            self.dir.mkdir(parents=True, exist_ok=True)
            self.sweep_orphans()

    # -- housekeeping -----------------------------------------------------------
    def sweep_orphans(self) -> int:
        n = 0
        for f in self.dir.glob(f"*{TMP_MARK}*"):
            try:
                f.unlink()
                n += 1
            except OSError:
                pass
        return n

    def wipe(self) -> None:
        """train_from_scratch: remove every checkpoint of this run (rank 0)."""
        if self.rank == 0 and self.dir.exists():
            for f in self.dir.iterdir():
                if f.is_file():
                    f.unlink()
        self.best_val_loss = float("inf")

    # -- saving -------------------------------------------------------------------
    def _write(self, payload: Dict[str, Any], is_best: bool) -> None:
        tmp = self.dir / f"{LAST_NAME}{TMP_MARK}{os.getpid()}"
        try:
            with open(tmp, "wb") as f:
                torch.save(payload, f)
                f.flush()
                os.fsync(f.fileno())
            os.replace(tmp, self.last_path)
            if is_best:
                tmpb = self.dir / f"{BEST_NAME}{TMP_MARK}{os.getpid()}"
                shutil.copyfile(self.last_path, tmpb)  # byte copy: cheaper than serialising twice
                with open(tmpb, "rb+") as f:
                    os.fsync(f.fileno())
                os.replace(tmpb, self.best_path)
        finally:
            for t in (tmp, self.dir / f"{BEST_NAME}{TMP_MARK}{os.getpid()}"):
                if t.exists():
                    try:
                        t.unlink()
                    except OSError:
                        pass

    def _collect_pending(self) -> Optional[str]:
        """Rank 0: outcome of the in-flight asynchronous save, if any."""
        err = None
        if self._pending is not None:
            try:
                self._pending.result()
            except Exception as exc:
                err = f"{type(exc).__name__}: {exc}"
            self._pending = None
        return err

    def _agree(self, err: Optional[str]) -> None:
        err = D.bcast_obj(err, src=0)
        if err is not None:
            raise CheckpointSaveError(f"checkpoint save failed on rank 0: {err}")

    def save(self, epoch: int, val_loss_avg: float, model, optimizer, scheduler=None, grad_scaler=None,
             extras: Optional[Dict[str, Any]] = None) -> bool:
        """Collective. Returns True when this checkpoint is the new best."""
        is_best = bool(val_loss_avg < self.best_val_loss)
        err = None
        if self.rank == 0:
            err = self._collect_pending()
            if err is None:
                try:
                    module = getattr(model, "module", model)
                    payload = {
                        "epoch": int(epoch),
                        "val_loss_avg": float(val_loss_avg),
                        "model_state_dict": _to_host(module.state_dict()),
                        "optimizer_state_dict": _to_host(optimizer.state_dict()),
                        "grad_scaler_state_dict": grad_scaler.state_dict() if grad_scaler is not None else {},
                        "scheduler_state_dict": scheduler.state_dict() if scheduler is not None else {},
                        **capture_rng(),
                    }
                    payload.update(extras or {})
                    if self._pool is not None:
                        self._pending = self._pool.submit(self._write, payload, is_best)
                    else:
                        self._write(payload, is_best)
                except Exception as exc:
                    err = f"{type(exc).__name__}: {exc}"
        self._agree_or_roll_back(err)
        # only a save that every rank knows succeeded (or, asynchronous, was handed to the writer) moves the mark;
        # the previous value is kept until the writer's outcome is collected
        confirmed = self.best_val_loss
        if is_best:
            self.best_val_loss = float(val_loss_avg)
        self._best_before_pending = confirmed if self._pool is not None else self.best_val_loss
        return is_best

    def _agree_or_roll_back(self, err: Optional[str]) -> None:
        """Agree on ``err``; a failure also takes back a 'best' mark set for a write that never landed."""
        try:
            self._agree(err)
        except CheckpointSaveError:
            self.best_val_loss = self._best_before_pending
            raise

    def finalize_saves(self) -> None:
        """Collective: wait for the asynchronous writer and agree on its outcome."""
        err = self._collect_pending() if self.rank == 0 else None
        self._agree_or_roll_back(err)
        self._best_before_pending = self.best_val_loss

    def close(self) -> None:
        if self._pool is not None:
            self._pool.shutdown(wait=True)
            self._pool = None

    # -- loading ----------------------------------------------------------------------
    def _read(self, path: Path):
        return torch.load(path, map_location="cpu", weights_only=False)

    def _load_on_root(self) -> Optional[Dict[str, Any]]:
        for path in (self.last_path, self.best_path):
            if not path.exists():
                continue
            try:
                state = self._read(path)
                if not isinstance(state, dict) or "model_state_dict" not in state:
                    raise ValueError("not a checkpoint dict")
                state["_loaded_from"] = path.name
                return state
            except Exception as exc:
                quarantine = path.with_suffix(path.suffix + ".corrupt")
                try:
                    os.replace(path, quarantine)
                except OSError:
                    pass
                if self.log is not None:
                    self.log.warning("checkpoint %s is unreadable (%s); moved to %s", path, exc, quarantine.name)
        return None

    def load(self, model, optimizer=None, scheduler=None, grad_scaler=None, restore_rng_state: bool = True
             ) -> Optional[Dict[str, Any]]:
        """Collective. Returns the loaded dict (minus the big state dicts) or None when there is nothing to load."""
        state = D.run_on_root(self._load_on_root)
        if state is None:
            return None
        module = getattr(model, "module", model)
        module.load_state_dict(state["model_state_dict"])
        if optimizer is not None and state.get("optimizer_state_dict"):
            optimizer.load_state_dict(state["optimizer_state_dict"])
        if scheduler is not None and state.get("scheduler_state_dict"):
            scheduler.load_state_dict(state["scheduler_state_dict"])
        if grad_scaler is not None and state.get("grad_scaler_state_dict"):
            grad_scaler.load_state_dict(state["grad_scaler_state_dict"])
        if restore_rng_state:
            restore_rng(state)
        self.best_val_loss = min(self.best_val_loss, float(state.get("val_loss_avg", float("inf"))))
        try:
            from ..ops.layout import bump_weights_epoch
            bump_weights_epoch()
        except Exception:
            pass
        return {k: v for k, v in state.items() if k not in ("model_state_dict", "optimizer_state_dict")}

    # -- warm-up snapshot -----------------------------------------------------------
    @staticmethod
    def snapshot(model, optimizer, scheduler=None) -> Dict[str, Any]:
        module = getattr(model, "module", model)
        return {"model": _to_host(module.state_dict()), "optimizer": _to_host(optimizer.state_dict()),
                "scheduler": copy.deepcopy(scheduler.state_dict()) if scheduler is not None else None,
                "rng": capture_rng()}

    @staticmethod
    def restore(snap: Dict[str, Any], model, optimizer, scheduler=None) -> None:
        module = getattr(model, "module", model)
        module.load_state_dict(snap["model"])
        optimizer.load_state_dict(snap["optimizer"])
        if scheduler is not None and snap["scheduler"] is not None:
            scheduler.load_state_dict(snap["scheduler"])
        restore_rng(snap["rng"])
        try:
            from ..ops.layout import bump_weights_epoch
            bump_weights_epoch()
        except Exception:
            pass
