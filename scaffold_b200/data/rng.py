"""Seed derivation for data generation.

``derive_seed(*keys)`` hashes little-endian u64 keys with BLAKE2b-64 and keeps
the low 32 bits, so every (seed, category, instance) gets an independent,
order-free stream (ScaFFold/datagen/rng.py:37-61). Streams themselves are
counter-based here (``numpy`` Philox / SplitMix64 in the native kernels), not
numba's Mersenne Twister, so datasets are deterministic in this framework's own
seeds but not bit-identical to the reference's.
"""
from __future__ import annotations

import hashlib
import struct

import numpy as np


def derive_seed(*keys: int) -> int:
    h = hashlib.blake2b(digest_size=8)
    for k in keys:
        h.update(struct.pack("<Q", int(k) & 0xFFFFFFFFFFFFFFFF))
    return int.from_bytes(h.digest(), "little") & 0xFFFFFFFF


def generator(*keys: int) -> np.random.Generator:
    """A Philox generator keyed by ``keys`` (a ``SeedSequence`` of the tuple)."""
    return np.random.Generator(np.random.Philox(np.random.SeedSequence([int(k) for k in keys])))
