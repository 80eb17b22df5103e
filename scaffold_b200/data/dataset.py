"""Dataset loader for the physical-shard ``.npy`` layout.

Behaviour kept from ScaFFold/utils/data_loading.py:40-594:

* format versions: v5 = one file per (volume, shard) named
  ``<id>_shardNNNNNN[_mask].npy``; v2 = one whole-volume file per id, sliced on
  load; a directory without ``meta.yaml`` is legacy v1 (channels-last volumes,
  arbitrary label values remapped through the ``*_unique_mask_vals`` pickle);
  a ``meta.yaml`` that cannot be read or carries no version is an error, never
  a silent legacy fallback;
* the shard layout on disk must equal the layout the run asks for;
* ids are sorted; an id matching two files is an error; every rank hashes its
  id list (SHA-256) and the hashes are compared across ranks;
* ``__getitem__`` returns ``{"image": float32 (3,d,h,w), "mask": int16 (d,h,w)}``
  (a narrow mask carrier: the consumer widens it on the device).
"""
from __future__ import annotations

import hashlib
import pickle
import re
from dataclasses import dataclass
from pathlib import Path
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch
import yaml
from torch.utils.data import Dataset

from ..utils import dist as D
from ..utils.sharding import (canonical_sharding, normalize_sharding, shard_file_suffix, shard_indices_to_id,
                              spatial_slices, total_shards)

META_FILENAME = "meta.yaml"
LEGACY_VERSION = 1
WHOLE_VOLUME_VERSION = 2
PHYSICAL_SHARD_VERSION = 5
MAX_VERSION = 5
_SHARD_RE = re.compile(r"^(?P<id>.+)_shard(?P<shard>\d{6})(?P<mask>_mask)?$")


@dataclass(frozen=True)
class SpatialShardSpec:
    """Which spatial shard of every volume this rank reads."""
    num_shards: Tuple[int, ...] = (1, 1, 1)
    shard_dims: Tuple[int, ...] = (2, 3, 4)
    shard_indices: Tuple[int, ...] = (0, 0, 0)

    def __post_init__(self):
        n, d = normalize_sharding(self.num_shards, self.shard_dims)
        object.__setattr__(self, "num_shards", n)
        object.__setattr__(self, "shard_dims", d)
        object.__setattr__(self, "shard_indices", tuple(int(i) for i in self.shard_indices))

    @property
    def shard_id(self) -> int:
        return shard_indices_to_id(self.shard_indices, self.num_shards)

    @property
    def total(self) -> int:
        return total_shards(self.num_shards)

    @classmethod
    def from_layout(cls, layout) -> "SpatialShardSpec":
        return cls(tuple(layout.num_shards), tuple(layout.shard_dim), tuple(layout.shard_ind))


def load_dataset_metadata(root: Path) -> dict:
    meta_path = Path(root) / META_FILENAME
    if not meta_path.exists():
        return {"dataset_format_version": LEGACY_VERSION}
    try:
        meta = yaml.safe_load(meta_path.read_text())
    except Exception as exc:
        raise ValueError(
            f"Dataset metadata {meta_path} exists but could not be read ({type(exc).__name__}: {exc}). A dataset "
            f"carrying a {META_FILENAME} is not a legacy dataset; refusing to guess its layout. Repair the file or "
            "regenerate the dataset.") from exc
    version = meta.get("dataset_format_version") if isinstance(meta, dict) else None
    try:
        int(version)
    except (TypeError, ValueError):
        raise ValueError(
            f"Dataset metadata {meta_path} is missing a usable 'dataset_format_version' (got {version!r}). A dataset "
            f"carrying a {META_FILENAME} is not a legacy dataset; refusing to guess its layout. Repair the file or "
            "regenerate the dataset.") from None
    return meta


class FractalDataset(Dataset):
    def __init__(self, images_dir, mask_dir, data_dir: str = "", spatial_shard_spec: Optional[SpatialShardSpec] = None,
                 mask_suffix: str = "_mask"):
        self.images_dir, self.mask_dir = Path(images_dir), Path(mask_dir)
        self.mask_suffix = mask_suffix
        self.spec = spatial_shard_spec or SpatialShardSpec()
        self.root = self.images_dir.parents[1]
        self.meta = load_dataset_metadata(self.root)
        self.version = int(self.meta["dataset_format_version"])
        if self.version > MAX_VERSION:
            raise RuntimeError(f"Unsupported dataset format version {self.version}; expected <= {MAX_VERSION}")
        self.physical = self.version >= PHYSICAL_SHARD_VERSION
        if self.physical:
            self._check_physical_layout()
        self.shard_suffix = shard_file_suffix(self.spec.shard_id) if self.physical else ""
        self.ids, self._paths = self._index()
        if not self.ids:
            raise RuntimeError(f"No input file found in {self.images_dir}, make sure you put your images there")
        self.mask_values = self._load_mask_values() if self.version == LEGACY_VERSION else None

    # -- index ----------------------------------------------------------------
    def _check_physical_layout(self) -> None:
        layout = self.meta.get("config_subset") or self.meta  # reference schema first, flat keys of older datasets
        if layout.get("dc_num_shards") is None or layout.get("dc_shard_dims") is None:
            raise RuntimeError("Physical dataset is missing shard metadata. Expected config_subset.dc_num_shards / "
                               "config_subset.dc_shard_dims in meta.yaml.")
        disk = canonical_sharding(layout["dc_num_shards"], layout["dc_shard_dims"])
        want = canonical_sharding(self.spec.num_shards, self.spec.shard_dims)
        if disk != want:
            raise ValueError(
                f"Dataset at {self.root} was written with shard layout num_shards={list(disk[0])} on dims "
                f"{list(disk[1])}, but the run asks for num_shards={list(want[0])} on dims {list(want[1])}. "
                "Physical shards cannot be re-cut on load; generate a dataset for this layout.")
        # shard ids on disk are row-major in the canonical (sorted-dim) order
        pairs = sorted(zip(self.spec.shard_dims, self.spec.num_shards, self.spec.shard_indices))
        idx = tuple(i for _, _, i in pairs)
        self._disk_shard = shard_indices_to_id(idx, disk[0])

    def _shard_id_on_disk(self) -> int:
        return getattr(self, "_disk_shard", self.spec.shard_id)

    def _index(self) -> Tuple[List[str], Dict[str, Path]]:
        paths: Dict[str, Path] = {}
        if self.physical:
            self.shard_suffix = shard_file_suffix(self._shard_id_on_disk())
        for f in sorted(self.images_dir.iterdir()):
            if f.name.startswith(".") or f.suffix != ".npy":
                continue
            stem = f.stem
            if self.physical:
                m = _SHARD_RE.match(stem)
                if not m or m.group("mask") or int(m.group("shard")) != self._shard_id_on_disk():
                    continue
                ident = m.group("id")
            else:
                ident = stem
            if ident in paths:
                raise RuntimeError(f"Either no image or multiple images found for the ID {ident}: "
                                   f"{[str(paths[ident]), str(f)]}")
            paths[ident] = f
        ids = sorted(paths, key=lambda s: (len(s), s))
        return ids, paths

    def ids_digest(self) -> bytes:
        return hashlib.sha256("\n".join(self.ids).encode()).digest()

    def check_ids_across_ranks(self) -> None:
        """All ranks of a replica group must iterate the same ids in the same order."""
        digests = D.allgather_obj(self.ids_digest())
        if len(set(digests)) != 1:
            bad = [r for r, d in enumerate(digests) if d != digests[0]]
            raise RuntimeError(f"Dataset id lists differ across ranks (ranks {bad} disagree with rank 0) in "
                               f"{self.images_dir}; the ranks see different directory contents")

    def _load_mask_values(self):
        name = "train_unique_mask_vals" if "training" in str(self.images_dir) else "val_unique_mask_vals"
        with open(self.root / name, "rb") as f:
            return pickle.load(f)["mask_values"]

    # -- access -----------------------------------------------------------------
    def __len__(self) -> int:
        return len(self.ids)

    def _mask_path(self, ident: str) -> Path:
        return self.mask_dir / f"{ident}{self.shard_suffix}{self.mask_suffix}.npy"

    def _slices(self, shape_dhw: Sequence[int]):
        return spatial_slices(shape_dhw, self.spec.num_shards, self.spec.shard_dims, self.spec.shard_id)

    def _load_mask(self, ident: str) -> np.ndarray:
        path = self._mask_path(ident)
        if not path.exists():
            raise RuntimeError(f"Either no mask or multiple masks found for the ID {ident}: {path}")
        mask = np.load(path, mmap_mode=None if self.physical else "r")
        if not self.physical and self.spec.total > 1:
            sl = self._slices(mask.shape[-3:])
            mask = mask[sl]
        mask = np.asarray(mask)
        if self.version == LEGACY_VERSION:
            lut = {v: i for i, v in enumerate(self.mask_values)}
            out = np.zeros(mask.shape, dtype=np.int16)
            for v, i in lut.items():
                out[mask == v] = i
            mask = out
        return mask

    @staticmethod
    def _to_mask_carrier(mask: np.ndarray) -> torch.Tensor:
        mask = np.ascontiguousarray(mask.astype(np.int16, copy=False))
        if not mask.flags.writeable:  # a memory-mapped int16 mask read whole: detach it from the file
            mask = mask.copy()
        return torch.from_numpy(mask)

    def load_mask_only(self, idx: int) -> torch.Tensor:
        return self._to_mask_carrier(self._load_mask(self.ids[idx]))

    def __getitem__(self, idx: int):
        ident = self.ids[idx]
        img = np.load(self._paths[ident], mmap_mode=None if self.physical else "r")
        if self.version == LEGACY_VERSION:
            img = np.moveaxis(np.asarray(img), -1, 0)  # legacy volumes are channels-last
        if not self.physical and self.spec.total > 1:
            sl = self._slices(img.shape[-3:])
            img = img[(slice(None), *sl)]
        img = np.ascontiguousarray(img, dtype=np.float32)
        if not img.flags.writeable:  # still the read-only memory map (whole-volume file, nothing cut off): detach it
            img = img.copy()
        return {"image": torch.from_numpy(img), "mask": self._to_mask_carrier(self._load_mask(ident))}
