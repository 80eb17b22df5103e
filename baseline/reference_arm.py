"""Reference arm of ``bench.py``: the unmodified reference package from ``baseline/_ref``.

Nothing of this repository's models, kernels or engine is imported here.
"""
from __future__ import annotations


def run(args):
    return {"impl": "reference", "unavailable": "reference arm not wired yet"}
