"""Dataset cache: find a reusable dataset or generate one, once, for all ranks.

Key and layout follow ScaFFold/datagen/get_dataset.py:34-556. The cache id is
``sha256(canonical JSON of the dataset-defining keys)[:12]`` (format version 5,
``n_categories``, ``n_instances_used_per_fractal``, ``problem_scale``,
``dataset_seed``, ``variance_threshold``, ``n_fracts_per_vol``, ``val_split`` and
the shard layout with its dims sorted, so equivalent layouts share an id). A
dataset lives at ``<dataset_dir>/<id>/<timestamp>__<commit>/`` next to a
``meta.yaml``; generation happens in ``.tmp_*`` staging and is published with one
atomic rename. Rank 0 decides (reuse / generate) and broadcasts; stale staging
directories (no heartbeat for 24 h) are swept; every failure is agreed on by all
ranks before anyone raises.
"""
from __future__ import annotations

import copy
import datetime
import hashlib
import json
import os
import shutil
import subprocess
import time
from pathlib import Path
from typing import Any, Dict, Optional

import yaml

from ..utils import dist as D
from . import volumes
from .volumes import HEARTBEAT_FILE

META_FILENAME = "meta.yaml"
TMP_PREFIX = ".tmp_"
STALE_STAGING_AGE_SECONDS = 24 * 60 * 60
DATASET_FORMAT_VERSION = 5
INCLUDE_KEYS = ["dataset_format_version", "n_categories", "n_instances_used_per_fractal", "problem_scale",
                "dataset_seed", "variance_threshold", "n_fracts_per_vol", "val_split", "dc_num_shards",
                "dc_shard_dims"]


def _as_dict(config) -> Dict[str, Any]:
    return dict(config) if isinstance(config, dict) else dict(vars(config))


def volume_config(config) -> Dict[str, Any]:
    d = _as_dict(config)
    d["dataset_format_version"] = DATASET_FORMAT_VERSION
    d.setdefault("dc_num_shards", [1, 1, 1])
    d.setdefault("dc_shard_dims", [2, 3, 4])
    missing = [k for k in INCLUDE_KEYS if k not in d]
    if missing:
        raise KeyError(f"Missing expected top-level keys in run YAML: {missing}. Required INCLUDE_KEYS={INCLUDE_KEYS}")
    out = {k: d[k] for k in INCLUDE_KEYS}
    if len(out["dc_num_shards"]) != len(out["dc_shard_dims"]):
        raise ValueError(f"dc_num_shards {out['dc_num_shards']} must have same length as dc_shard_dims "
                         f"{out['dc_shard_dims']}")
    pairs = sorted((int(dim), int(n)) for n, dim in zip(out["dc_num_shards"], out["dc_shard_dims"]))
    out["dc_shard_dims"] = [dim for dim, _ in pairs]
    out["dc_num_shards"] = [n for _, n in pairs]
    return out


def config_id(config) -> str:
    s = json.dumps(volume_config(config), separators=(",", ":"), sort_keys=True).encode()
    return hashlib.sha256(s).hexdigest()[:12]


def git_commit_short(source_dir: Optional[Path] = None) -> str:
    try:
        src = source_dir or Path(__file__).resolve().parent
        out = subprocess.run(["git", "-C", str(src), "rev-parse", "--short", "HEAD"], capture_output=True, text=True,
                             timeout=10)
        if out.returncode == 0 and out.stdout.strip():
            return out.stdout.strip()
    except Exception:
        pass
    return "no-commit-id"


def _newest_mtime(path: Path, max_dirs: int = 10000, max_depth: int = 3) -> float:
    newest, seen = path.stat().st_mtime, 0
    hb = path / HEARTBEAT_FILE
    if hb.exists():
        newest = max(newest, hb.stat().st_mtime)
    stack = [(path, 0)]
    while stack and seen < max_dirs:
        d, depth = stack.pop()
        seen += 1
        try:
            for e in os.scandir(d):
                try:
                    newest = max(newest, e.stat(follow_symlinks=False).st_mtime)
                    if e.is_dir(follow_symlinks=False) and depth < max_depth:
                        stack.append((Path(e.path), depth + 1))
                except OSError:
                    continue
        except OSError:
            continue
    return newest


def sweep_stale_staging(id_dir: Path, log=None, now: Optional[float] = None) -> int:
    """Remove ``.tmp_*`` directories nothing has touched for 24 h; returns how many were removed."""
    removed = 0
    if not id_dir.exists():
        return 0
    now = time.time() if now is None else now
    for d in id_dir.iterdir():
        if not (d.is_dir() and d.name.startswith(TMP_PREFIX)):
            continue
        try:
            if now - _newest_mtime(d) > STALE_STAGING_AGE_SECONDS:
                shutil.rmtree(d, ignore_errors=True)
                removed += 1
                if log is not None:
                    log.info("removed stale staging directory %s", d)
        except OSError:
            continue
    return removed


def find_reusable(id_dir: Path, require_commit: Optional[str] = None) -> Optional[Path]:
    """Newest published dataset below ``id_dir`` whose meta.yaml parses (and matches the commit if asked)."""
    if not id_dir.exists():
        return None
    best = None
    for d in sorted(id_dir.iterdir()):
        if not d.is_dir() or d.name.startswith(TMP_PREFIX):
            continue
        meta = d / META_FILENAME
        try:
            info = yaml.safe_load(meta.read_text()) or {}
        except Exception:
            continue
        if info.get("dataset_format_version") != DATASET_FORMAT_VERSION:
            continue
        if require_commit and info.get("code_commit", info.get("commit")) != require_commit:
            continue
        best = d
    return best


def get_dataset(config, require_commit: bool = False, log=None) -> Path:
    """Collective. Returns the path of a dataset matching ``config`` (generated if none exists)."""
    cid = config_id(config)
    id_dir = Path(config.dataset_dir) / cid
    commit = git_commit_short()

    def decide():
        id_dir.mkdir(parents=True, exist_ok=True)
        sweep_stale_staging(id_dir, log)
        found = find_reusable(id_dir, commit if require_commit else None)
        if found is not None:
            return {"reuse": str(found)}
        ts = datetime.datetime.now().strftime("%Y%m%d-%H%M%S")
        return {"staging": str(id_dir / f"{TMP_PREFIX}{ts}__{commit}"), "final": str(id_dir / f"{ts}__{commit}")}

    plan = D.run_on_root(decide)
    if "reuse" in plan:
        if log is not None:
            log.info("reusing dataset %s", plan["reuse"])
        return Path(plan["reuse"])

    staging, final = Path(plan["staging"]), Path(plan["final"])
    gen_config = copy.copy(config)
    gen_config.dataset_dir = str(staging)
    err, interrupt = None, None
    try:
        volumes.main(gen_config, log)
    except KeyboardInterrupt as exc:
        interrupt, err = exc, "KeyboardInterrupt"
    except Exception as exc:
        err = f"{type(exc).__name__}: {exc}"
    try:
        D.consensus(err is None, err or "")
    finally:
        if interrupt is not None:
            raise interrupt

    def publish():
        # the reference's schema (ScaFFold/datagen/get_dataset.py:527-535): the keys that define the dataset live
        # under `config_subset`, so either implementation's loader reads the other's datasets
        meta = {"config_id": cid, "dataset_format_version": DATASET_FORMAT_VERSION,
                "config_subset": dict(volume_config(config)), "include_keys": list(INCLUDE_KEYS),
                "code_commit": commit, "created_at": time.strftime("%Y-%m-%dT%H:%M:%SZ", time.gmtime()),
                "vol_size": int(config.vol_size), "point_num": int(config.point_num)}
        with open(staging / META_FILENAME, "w") as f:
            yaml.safe_dump(meta, f, sort_keys=True)
            f.flush()
            os.fsync(f.fileno())
        hb = staging / HEARTBEAT_FILE
        if hb.exists():
            hb.unlink()
        os.replace(staging, final)
        return str(final)

    out = D.run_on_root(publish)
    D.barrier()
    return Path(out)
