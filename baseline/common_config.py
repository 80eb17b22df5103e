"""The ``config`` block both arms of ``bench.py`` print: same keys, same strings for the same work.

Everything that describes the workload (model, scale, width, classes, batch, volume, parallelism)
is here and is identical for the two arms; what differs between the implementations (kernels,
backends, the loss value reached) goes under the separate ``arm`` key.
"""
from __future__ import annotations


def workload_config(scale: int, levels: int, base_width: int, n_classes: int, n_params: int, batch_per_replica: int,
                    replicas: int, num_shards, arm: dict) -> dict:
    S = 2 ** scale
    sp = 1
    for n in num_shards:
        sp *= int(n)
    return {
        "model": f"3D U-Net scale {scale}: {levels} levels, base width {base_width}, GroupNorm(8), "
                 f"{n_classes} classes, {n_params} params",
        "scale": scale,
        "base_width": base_width,
        "n_classes": n_classes,
        "global_batch": batch_per_replica * replicas,
        "batch_per_replica": batch_per_replica,
        "seq_len": S ** 3,
        "volume": [S, S, S],
        "parallelism": f"dp{replicas}" + (f"xsp{sp}{[int(n) for n in num_shards]}" if sp > 1 else ""),
        "optimizer": "Adam lr 1e-3, global-norm clip 1.0",
        "loss": "cross entropy + (1 - mean foreground soft Dice)",
        "l2_policy": "inputs larger than L2 (activations of one step are several GB; two batches rotate)",
        "arm": arm,
    }
