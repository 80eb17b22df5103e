"""Run configuration: one declarative schema drives loading, validation and dumping.

Public surface kept from the reference (ScaFFold/utils/config_utils.py:88-349,
ScaFFold/configs/benchmark_default.yml): the same YAML keys and defaults,
strict rejection of unknown keys, scalar-only keys ("no sweeps"), ``dist: 0``
rejected, base + override file merge, and a dumped ``config.yaml`` that loads
back (derived keys are accepted on input). Superset keys for the measured
configurations (``unet_base_width``, ``n_channels``, ``gn_stats``,
``grad_allreduce``, ``halo_exchange``, ``point_num_override``) are optional and
default to the reference behaviour.
"""
from __future__ import annotations

import math
import os
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Callable, Dict, Iterable, List, Optional

import yaml

MAX_SEED = 2**32 - 1
_REQUIRED = object()


def require_nonneg_number(name: str, value: Any) -> float:
    if isinstance(value, bool) or not isinstance(value, (int, float)) or not (value >= 0):
        raise ValueError(f"{name} must be a non-negative number; got {value!r}")
    return float(value)


def require_positive_int(name: str, value: Any) -> int:
    if isinstance(value, bool) or not isinstance(value, int) or value < 1:
        raise ValueError(f"{name} must be a positive integer; got {value!r}")
    return value


def require_flag(name: str, value: Any) -> bool:
    """0/1 or a YAML boolean; anything else (2, -1, "no") is a typo, not a truth value."""
    if isinstance(value, bool):
        return value
    if isinstance(value, int) and value in (0, 1):
        return bool(value)
    raise ValueError(f"{name} must be 0, 1, or a boolean; got {value!r}")


def require_seed(name: str, value: Any) -> int:
    if isinstance(value, bool) or not isinstance(value, int):
        raise ValueError(f"{name} must be an integer; got {value!r}")
    if not 0 <= value <= MAX_SEED:
        raise ValueError(f"{name} must be in [0, {MAX_SEED}]; got {value}")
    return value


def validate_unet_dims(problem_scale: int, unet_bottleneck_dim: Any) -> int:
    """``0 <= unet_bottleneck_dim <= problem_scale - 1`` so the U-Net has >= 1 level."""
    if isinstance(unet_bottleneck_dim, bool) or not isinstance(unet_bottleneck_dim, int):
        raise ValueError(f"unet_bottleneck_dim must be an integer; got {unet_bottleneck_dim!r}")
    layers = problem_scale - unet_bottleneck_dim
    if unet_bottleneck_dim < 0 or layers < 1:
        raise ValueError(
            f"unet_bottleneck_dim={unet_bottleneck_dim} is out of range for problem_scale={problem_scale}: "
            f"need 0 <= unet_bottleneck_dim <= {problem_scale - 1} (unet_layers = problem_scale - "
            f"unet_bottleneck_dim = {layers}). Raise problem_scale or lower unet_bottleneck_dim."
        )
    return unet_bottleneck_dim


@dataclass(frozen=True)
class Key:
    """One configuration key: default (or required), scalar-only flag, optional converter."""
    name: str
    default: Any = _REQUIRED
    scalar: bool = False
    conv: Optional[Callable[[str, Any], Any]] = None


def _path(name: str, v: Any) -> str:
    return str(Path(v).resolve())


def _flag(name: str, v: Any) -> bool:
    return bool(v)


def _choice(*allowed: str) -> Callable[[str, Any], str]:
    def conv(name: str, v: Any) -> str:
        if v not in allowed:
            raise ValueError(f"{name} must be one of {allowed}; got {v!r}")
        return v
    return conv


SCHEMA: List[Key] = [
    Key("base_run_dir", _REQUIRED, conv=_path),
    Key("dataset_dir", "datasets/", conv=_path),
    Key("fract_base_dir", "fractals/", conv=_path),
    Key("job_name", "benchmark"),
    Key("n_categories", _REQUIRED, scalar=True, conv=require_positive_int),
    Key("problem_scale", _REQUIRED, scalar=True),
    Key("unet_bottleneck_dim", _REQUIRED, scalar=True),
    Key("n_fracts_per_vol", _REQUIRED, scalar=True),
    Key("n_instances_used_per_fractal", _REQUIRED, scalar=True),
    Key("local_batch_size", _REQUIRED, scalar=True),
    Key("dataloader_num_workers", _REQUIRED, scalar=True),
    Key("epochs", _REQUIRED, scalar=True),
    Key("optimizer", _REQUIRED, scalar=True),
    Key("disable_scheduler", _REQUIRED, conv=_flag),
    Key("more_determinism", _REQUIRED, conv=_flag),
    Key("datagen_from_scratch", _REQUIRED, conv=_flag),
    Key("train_from_scratch", _REQUIRED, conv=_flag),
    Key("val_split", _REQUIRED, scalar=True),
    Key("dataset_seed", _REQUIRED, scalar=True, conv=require_seed),
    Key("training_seed", _REQUIRED, scalar=True, conv=require_seed),
    Key("framework", _REQUIRED),
    Key("starting_learning_rate", _REQUIRED, scalar=True),
    Key("min_learning_rate", _REQUIRED, scalar=True),
    Key("T_0", _REQUIRED, scalar=True),
    Key("T_mult", _REQUIRED, scalar=True),
    Key("variance_threshold", _REQUIRED, scalar=True),
    Key("torch_amp", _REQUIRED, conv=_flag),
    Key("loss_freq", _REQUIRED, scalar=True),
    Key("checkpoint_dir", _REQUIRED),
    Key("normalize", _REQUIRED),
    Key("group_norm_groups", 8, scalar=True),
    Key("warmup_batches", None, scalar=True),
    Key("activation_checkpointing", 0, scalar=True, conv=require_flag),
    Key("ce_weight_sample_fraction", 0.1, scalar=True),
    Key("dataset_reuse_enforce_commit_id", _REQUIRED),
    Key("target_dice", _REQUIRED, scalar=True),
    Key("checkpoint_interval", _REQUIRED, scalar=True),
    Key("async_save", False, conv=_flag),
    Key("dc_num_shards", _REQUIRED),
    Key("dc_shard_dims", _REQUIRED),
    Key("restart", False, conv=_flag),
    # --- superset keys (not in the reference schema) ---
    Key("unet_base_width", 64, scalar=True, conv=require_positive_int),
    Key("n_channels", 3, scalar=True, conv=require_positive_int),
    Key("gn_stats", "global", conv=_choice("global", "per_shard")),
    Key("grad_allreduce", "fused", conv=_choice("fused", "nccl")),
    Key("grad_overlap", True, conv=_flag),
    Key("halo_exchange", "fused", conv=_choice("fused", "nccl")),
    Key("allow_fallback", False, conv=_flag),
    Key("val_cache_gb", 16.0, scalar=True, conv=require_nonneg_number),  # GiB of device memory for the validation set
    Key("point_num_override", None, scalar=True),
    Key("datagen_device", "auto", conv=_choice("auto", "cpu", "cuda")),
]

_BY_NAME: Dict[str, Key] = {k.name: k for k in SCHEMA}

# accepted on input but never required: derived / run-time bookkeeping
DERIVED_KEYS = frozenset({"scale", "dc_total_shards", "dist"})
AUX_KEYS = frozenset({
    "command", "config", "verbose", "run_dir", "run_iter", "benchmark_run_dir", "unet_layers",
    "vol_size", "point_num", "scheduler_metadata", "machine_name", "datagen_batch_size",
})
KNOWN_KEYS = frozenset(_BY_NAME) | DERIVED_KEYS


def allowed_keys() -> frozenset:
    return KNOWN_KEYS | AUX_KEYS


class Config:
    """Validated settings of one benchmark configuration."""

    KNOWN_KEYS = KNOWN_KEYS
    AUX_KEYS = AUX_KEYS

    def __init__(self, config_dict: Dict[str, Any], strict: bool = True):
        self._check_keys(config_dict, strict)
        if "dist" in config_dict and not bool(config_dict["dist"]):
            raise ValueError(
                "The 'dist: 0' mode is not supported: training always runs with distributed execution; "
                "use a one-rank launch for singleton runs."
            )
        for key in SCHEMA:
            if key.name in config_dict:
                value = config_dict[key.name]
            elif key.default is _REQUIRED:
                raise KeyError(key.name)
            else:
                value = key.default
            if key.conv is not None and value is not None:
                value = key.conv(key.name, value)
            setattr(self, key.name, value)
        if not isinstance(self.problem_scale, int) or isinstance(self.problem_scale, bool):
            print("WARNING: problem_scale found to be non-integer. Truncating to nearest int.")
            self.problem_scale = math.floor(self.problem_scale)
        self.unet_bottleneck_dim = validate_unet_dims(self.problem_scale, self.unet_bottleneck_dim)
        self.unet_layers = self.problem_scale - self.unet_bottleneck_dim
        self.scale = 1
        self.dc_num_shards = list(self.dc_num_shards)
        self.dc_shard_dims = list(self.dc_shard_dims)
        if len(self.dc_num_shards) != len(self.dc_shard_dims):
            raise ValueError(
                f"Configuration Mismatch: num_shards {self.dc_num_shards} must have same length as "
                f"shard_dim {self.dc_shard_dims}"
            )
        self.dc_total_shards = math.prod(self.dc_num_shards)
        # derived problem geometry (ScaFFold/cli.py:307-335)
        self.vol_size = 2 ** self.problem_scale
        self.point_num = int(config_dict.get("point_num") or self.point_num_override
                             or max(1, self.vol_size ** 3 // 256))
        for aux in ("verbose", "machine_name", "scheduler_metadata", "datagen_batch_size", "command"):
            if aux in config_dict:
                setattr(self, aux, config_dict[aux])

    @staticmethod
    def _check_keys(config_dict: Dict[str, Any], strict: bool) -> None:
        unknown = sorted(set(config_dict) - allowed_keys())
        if unknown:
            message = f"Unknown config key(s): {', '.join(unknown)}"
            if strict:
                raise ValueError(message)
            print(f"WARNING: {message}")
        lists = sorted(k.name for k in SCHEMA if k.scalar and isinstance(config_dict.get(k.name), list))
        if lists:
            details = "; ".join(
                f"{k}: parameter sweeps are no longer supported; got list {config_dict[k]}" for k in lists)
            raise ValueError(
                f"{details}. Each of these keys must hold a single value; launch one benchmark run per "
                "parameter setting.")

    def to_dict(self) -> Dict[str, Any]:
        return {k: v for k, v in vars(self).items() if not k.startswith("_")}

    def __repr__(self) -> str:
        return f"{type(self).__name__}({self.to_dict()})"


class RunConfig(Config):
    """A configuration bound to one run directory."""

    def __init__(self, config_dict: Dict[str, Any], strict: bool = True):
        super().__init__(config_dict, strict=strict)
        self.run_dir = config_dict["run_dir"]
        self.run_iter = config_dict["run_iter"]


def load_config_files(file_paths: Iterable[str]) -> Dict[str, Any]:
    """First file: complete config. Later files: partial overrides (unknown key => error)."""
    file_paths = list(file_paths)
    if not file_paths:
        raise ValueError("At least one config file is required")
    merged: Optional[Dict[str, Any]] = None
    for i, fp in enumerate(file_paths):
        if not os.path.exists(fp):
            raise FileNotFoundError(f"Config file '{fp}' not found")
        with open(fp, "r") as f:
            d = yaml.safe_load(f) or {}
        if i == 0:
            merged = dict(d)
            continue
        unknown = sorted(set(d) - allowed_keys())
        if unknown:
            raise ValueError(f"Unknown config key(s) in override file '{fp}': {', '.join(unknown)}")
        merged.update(d)
    return merged


def load_config(file_path: str, config_type: str) -> Config:
    if not os.path.exists(file_path):
        raise FileNotFoundError(f"Config file '{file_path}' not found")
    with open(file_path, "r") as f:
        d = yaml.safe_load(f)
    if config_type == "benchmark":
        return Config(d)
    if config_type == "run":
        return RunConfig(d)
    raise ValueError(f"Invalid config type specified: {config_type}. Must be either 'benchmark' or 'run'")


def default_config_path() -> Path:
    return Path(__file__).resolve().parent / "configs" / "benchmark_default.yml"
