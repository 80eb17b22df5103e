"""Rank script (gloo, CPU): validation metrics reduced over data-parallel replicas equal the one-process values.

Five validation samples over two replicas (3 + 2, no padding): each rank evaluates its own samples, the
sample-weighted sums are all-reduced as the trainer does, and rank 0 compares with evaluating all five alone.
"""
import os
import sys

sys.path.insert(0, os.path.abspath(os.path.join(os.path.dirname(__file__), "..", "..", "..")))  # repo root: runnable directly

import faulthandler

import torch
import torch.distributed as dist

faulthandler.dump_traceback_later(int(os.environ.get("SCAFFOLD_TEST_FAULT_TIMEOUT", "200")), exit=True)
dist.init_process_group("gloo")
rank, world = dist.get_rank(), dist.get_world_size()

from scaffold_b200.models.unet import UNet  # noqa: E402
from scaffold_b200.parallel.layout import ParallelLayout  # noqa: E402
from scaffold_b200.train.engine import TrainEngine  # noqa: E402
from scaffold_b200.train.evaluate import evaluate  # noqa: E402
from scaffold_b200.train.trainer import UnpaddedDistributedSampler  # noqa: E402

torch.manual_seed(3)
n_classes = 4
model = UNet(3, n_classes, layers=1, base_width=8)
layout = ParallelLayout((1, 1, 1), (2, 3, 4), world, rank)
engine = TrainEngine(model, torch.optim.Adam(model.parameters(), lr=1e-3), n_classes, "cpu", layout=layout, amp=False)
g = torch.Generator().manual_seed(17)
images = torch.randn(5, 3, 8, 8, 8, generator=g)
masks = torch.randint(0, n_classes, (5, 8, 8, 8), generator=g, dtype=torch.int16)


def batches(indices, bs=2):
    idx = list(indices)
    return [{"image": images[idx[i:i + bs]], "mask": masks[idx[i:i + bs]]} for i in range(0, len(idx), bs)]


mine = UnpaddedDistributedSampler(range(5), layout.ddp_ranks, layout.ddp_ind)
d_sum, l_sum, _, _, n = evaluate(engine, batches(mine))
t = torch.tensor([d_sum, l_sum, float(n)], dtype=torch.float64)
dist.all_reduce(t, group=layout.ddp_group)
if rank == 0:
    d_all, l_all, _, _, n_all = evaluate(engine, batches(range(5)))
    print(f"RESULT counts {int(t[2])} {n_all}")
    print(f"RESULT dice {t[0].item() / t[2].item():.7f} {d_all / n_all:.7f}")
    print(f"RESULT loss {t[1].item() / t[2].item():.7f} {l_all / n_all:.7f}")
dist.barrier()
dist.destroy_process_group()
print("DONE")
