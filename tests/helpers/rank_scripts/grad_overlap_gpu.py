"""Rank script (one GPU per rank): bucketed gradient reduction under backward gives the same weights as one
reduction after backward (fused peer-memory backend and NCCL backend)."""
import copy
import os
import sys

sys.path.insert(0, os.path.abspath(os.path.join(os.path.dirname(__file__), "..", "..", "..")))  # repo root: runnable directly

import torch
import torch.distributed as dist

rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
dev = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
dist.init_process_group("nccl", device_id=dev)
from scaffold_b200.models.unet import UNet  # noqa: E402
from scaffold_b200.ops import _lib  # noqa: E402
from scaffold_b200.ops.optim import FusedClipAdam  # noqa: E402
from scaffold_b200.parallel.layout import ParallelLayout  # noqa: E402
from scaffold_b200.train.engine import TrainEngine  # noqa: E402

backend = sys.argv[1] if len(sys.argv) > 1 else "fused"
torch.manual_seed(0)
base = UNet(3, 4, layers=2, base_width=16).to(dev)
layout = ParallelLayout([1, 1, 1], [2, 3, 4], world, rank)
g = torch.Generator().manual_seed(10 + rank)
batches = [(torch.randn(1, 3, 32, 32, 32, generator=g), torch.randint(0, 4, (1, 32, 32, 32), generator=g).to(torch.int16))
           for _ in range(3)]


def run(overlap):
    model = copy.deepcopy(base)
    opt = FusedClipAdam(model.parameters(), lr=1e-3)
    eng = TrainEngine(model, opt, 4, dev, layout=layout, grad_backend=backend, grad_overlap=overlap)
    # a small bucket size so that several buckets are in flight
    if overlap:
        assert eng.reducer._buckets is not None and len(eng.reducer._buckets) >= 1
    losses = [float(eng.step(*b)) for b in batches]
    torch.cuda.synchronize()
    _lib.check_status()
    return losses, torch.cat([p.detach().flatten() for p in model.parameters()]).clone()


l0, w0 = run(False)
l1, w1 = run(True)
same = bool(torch.equal(w0, w1))
close = float((w0 - w1).abs().max())
# every rank holds the same weights after the steps
ref = w1.clone()
dist.broadcast(ref, 0)
agree = bool(torch.equal(ref, w1))
if rank == 0:
    print(f"RESULT same {same} {close}")
    print(f"RESULT agree {agree}")
    print(f"RESULT losses {l0} {l1}")
dist.barrier()
dist.destroy_process_group()
print("DONE")
