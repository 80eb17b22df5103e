"""Host-side logic of the gradient reducer: once-per-step counting of a bucket's gradients (a parameter may be
announced twice: by the kernel that wrote its gradient into the flat buffer and by autograd's accumulate hook),
the effective-backend report and the scaling factor (role of the DDP reducer behind ScaFFold/worker.py:81-97)."""
import torch

from scaffold_b200.parallel.ddp import GradReducer


def _reducer_with_two_buckets():
    r = GradReducer(None)
    params = [torch.nn.Parameter(torch.zeros(1)) for _ in range(3)]
    b_last = {"lo": 10, "hi": 20, "n": 2, "pending": 2, "launched": False, "seen": set()}
    b_first = {"lo": 0, "hi": 10, "n": 1, "pending": 1, "launched": False, "seen": set()}
    r._buckets = [b_last, b_first]
    r._bucket_of = {id(params[2]): b_last, id(params[1]): b_last, id(params[0]): b_first}
    launched = []

    def fake_launch(b):
        b["launched"] = True
        launched.append((b["lo"], b["hi"]))
    r._launch = fake_launch
    return r, params, launched


def test_a_bucket_launches_once_all_of_its_gradients_were_announced_once():
    r, p, launched = _reducer_with_two_buckets()
    r._on_grad(p[2])
    r._on_grad(p[2])                       # the accumulate hook after a direct write: not counted twice
    assert launched == []
    r._on_grad(p[1])
    assert launched == [(10, 20)]
    r._on_grad(p[1])                       # a late duplicate for a launched bucket is ignored
    r._on_grad(torch.nn.Parameter(torch.zeros(1)))   # a parameter outside the flat buffer is ignored
    assert launched == [(10, 20)]
    r._on_grad(p[0])
    assert launched == [(10, 20), (0, 10)]


def test_single_rank_reducer_is_a_no_op_with_unit_scale():
    r = GradReducer(None)
    assert r.effective_backend == "none" and r.scale == 1.0
    r.reduce()                             # nothing to do, no process group needed

    class Layout:                          # 2 replicas x 2 shards: sum over shards, mean over replicas
        world_size = 4

        @staticmethod
        def grad_scale():
            return 0.5
    assert GradReducer(Layout()).scale == 0.5 and GradReducer(Layout()).world == 4
