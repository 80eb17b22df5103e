"""Rank script: a tiny scale-4 benchmark run through the public driver on CPU/gloo.

usage: benchmark_tiny.py <work_dir> <shards_w> [epochs] [extra yaml]
Prints RESULT lines with the per-epoch losses read back from train_stats.csv.
"""
import csv
import faulthandler
import os
import sys

sys.path.insert(0, os.path.abspath(os.path.join(os.path.dirname(__file__), "..", "..", "..")))  # repo root: runnable directly
from pathlib import Path

import yaml

faulthandler.dump_traceback_later(int(os.environ.get("SCAFFOLD_TEST_FAULT_TIMEOUT", "200")), exit=True)

from scaffold_b200 import config as C  # noqa: E402
from scaffold_b200.run import benchmark, generate_fractals  # noqa: E402
from scaffold_b200.utils import dist as D  # noqa: E402

work = Path(sys.argv[1])
shards_w = int(sys.argv[2])
epochs = int(sys.argv[3]) if len(sys.argv) > 3 else 2
extra = yaml.safe_load(sys.argv[4]) if len(sys.argv) > 4 else {}

d = yaml.safe_load(C.default_config_path().read_text())
d.update(base_run_dir=str(work / "runs"), dataset_dir=str(work / "ds"), fract_base_dir=str(work / "fr"),
         problem_scale=4, unet_bottleneck_dim=3, n_categories=2, n_instances_used_per_fractal=6, n_fracts_per_vol=3,
         datagen_device="cpu", point_num_override=600, dataloader_num_workers=0, warmup_batches=1, epochs=epochs,
         target_dice=2.0, local_batch_size=2, dc_num_shards=[1, 1, shards_w], checkpoint_interval=1,
         unet_base_width=16, val_split=50)
d.update(extra)
D.initialize_dist()
world = D.get_world_size()
run_dir = work / f"run_w{world}_s{shards_w}_{d.get('job_name', 'x')}"
d["run_dir"] = d.get("run_dir") or str(run_dir)
d["run_iter"] = 0
generate_fractals(dict(d))
out = benchmark(dict(d))
if D.get_world_rank() == 0:
    with open(Path(d["run_dir"]) / "train_stats.csv") as f:
        for row in csv.DictReader(f):
            print(f"RESULT epoch{row['epoch']} {row['overall_loss']} {row['val_loss_avg']} {row['val_dice']}")
    print(f"RESULT final_epochs {out['final_epochs']}")
    print(f"RESULT files {sorted(p.name for p in Path(d['run_dir']).iterdir())}")
print("DONE")
