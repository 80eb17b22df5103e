"""Rank script (one GPU per rank): fused peer-memory all-reduce vs NCCL, plus a timing line."""
import os
import sys

sys.path.insert(0, os.path.abspath(os.path.join(os.path.dirname(__file__), "..", "..", "..")))  # repo root: runnable directly

import torch
import torch.distributed as dist

rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
dist.init_process_group("nccl", device_id=torch.device("cuda", int(os.environ["LOCAL_RANK"])))
from scaffold_b200.ops import _lib  # noqa: E402
from scaffold_b200.parallel.fused_allreduce import FusedAllReduce  # noqa: E402

n = int(sys.argv[1]) if len(sys.argv) > 1 else (1 << 22) + 12
ar = FusedAllReduce(n)
g = torch.Generator(device="cuda").manual_seed(100 + rank)
ok = True
for trial in range(3):
    src = torch.randint(-8, 9, (n,), generator=g, device="cuda").float()  # integers: the sum is exact in any order
    ar.grad.copy_(src)
    ref = src.clone()
    dist.all_reduce(ref)
    torch.cuda.synchronize()
    dist.barrier()
    ar.all_reduce_(scale=0.5)
    torch.cuda.synchronize()
    _lib.check_status()
    ok &= bool(torch.equal(ar.grad, ref * 0.5))
# partial range
ar.grad.fill_(float(rank + 1))
torch.cuda.synchronize(); dist.barrier()
ar.all_reduce_(offset=1024, count=5000)
torch.cuda.synchronize(); _lib.check_status()
tot = float(sum(range(1, world + 1)))
ok &= bool((ar.grad[1024:6024] == tot).all()) and bool((ar.grad[:1024] == rank + 1).all()) and bool((ar.grad[6024:] == rank + 1).all())
# timing at a gradient-sized buffer
big = 90_302_537
ar2 = FusedAllReduce(big)
nc = torch.zeros(big, device="cuda")
def timeit(fn):
    for _ in range(3): fn()
    torch.cuda.synchronize(); dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(10): fn()
    e1.record(); torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / 10], device="cuda"); dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.item()
t_f = timeit(lambda: ar2.all_reduce_())
t_n = timeit(lambda: dist.all_reduce(nc))
_lib.check_status()
if rank == 0:
    print(f"RESULT equal {ok}")
    print(f"RESULT time_ms fused {t_f:.3f} nccl {t_n:.3f} bytes {big * 4}")
dist.barrier()
ar.close(); ar2.close()
dist.destroy_process_group()
print("DONE")
