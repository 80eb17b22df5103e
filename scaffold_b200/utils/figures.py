"""Standard figures from ``train_stats.csv``: ``figures/{train_loss,val_dice,val_loss}.png``.

Headless (``savefig`` only, Agg backend); when matplotlib is not installed the
curves are written as ``.csv`` series instead, so the artefact names stay
discoverable (ScaFFold/viz/standard_viz.py:26-111).
"""
from __future__ import annotations

import csv
from pathlib import Path
from typing import Dict, List


def read_stats(run_dir) -> Dict[str, List[float]]:
    cols: Dict[str, List[float]] = {}
    with open(Path(run_dir) / "train_stats.csv") as f:
        for row in csv.DictReader(f):
            for k, v in row.items():
                cols.setdefault(k, []).append(float(v))
    return cols


def standard_figures(run_dir) -> List[Path]:
    cols = read_stats(run_dir)
    out_dir = Path(run_dir) / "figures"
    out_dir.mkdir(exist_ok=True)
    series = {"train_loss": "overall_loss", "val_dice": "val_dice", "val_loss": "val_loss_avg"}
    written: List[Path] = []
    try:
        import matplotlib
        matplotlib.use("Agg")
        import matplotlib.pyplot as plt
    except Exception:
        plt = None
    for name, col in series.items():
        xs, ys = cols.get("epoch", []), cols.get(col, [])
        if plt is None:
            path = out_dir / f"{name}.csv"
            with open(path, "w") as f:
                f.write("epoch," + col + "\n")
                for x, y in zip(xs, ys):
                    f.write(f"{int(x)},{y}\n")
        else:
            path = out_dir / f"{name}.png"
            fig, ax = plt.subplots(figsize=(6, 4))
            ax.plot(xs, ys, marker="o")
            ax.set_xlabel("epoch")
            ax.set_ylabel(col)
            ax.set_title(name)
            fig.tight_layout()
            fig.savefig(path)
            plt.close(fig)
        written.append(path)
    return written
