"""Multi-GPU tests (skipped with fewer than two visible GPUs): child processes, one rank per GPU."""
import os
import subprocess
import sys

import pytest
import torch

from helpers.launch import ROOT, free_port, results

pytestmark = pytest.mark.gpu


def _torchrun(script, nproc, args=(), timeout=300):
    env = dict(os.environ)
    env["PYTHONPATH"] = f"{ROOT}:{env.get('PYTHONPATH', '')}"
    env["NCCL_NVLS_ENABLE"] = "0"
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", str(free_port()), str(script), *args]
    return subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, env=env, cwd=str(ROOT))


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_fused_allreduce_matches_nccl_on_two_gpus():
    proc = _torchrun(ROOT / "tests" / "helpers" / "rank_scripts" / "fused_allreduce_gpu.py", 2)
    assert proc.returncode == 0, proc.stdout[-2000:] + proc.stderr[-2000:]
    assert results(proc.stdout)["equal"] == ["True"]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("split_dim,halo", [(2, "nccl"), (4, "nccl"), (2, "fused"), (3, "fused"), (4, "fused")])
def test_two_spatial_shards_match_the_whole_volume_on_gpu(split_dim, halo):
    proc = _torchrun(ROOT / "tests" / "helpers" / "rank_scripts" / "spatial_gpu.py", 2, [str(split_dim), halo])
    assert proc.returncode == 0, proc.stdout[-2000:] + proc.stderr[-3000:]
    res = results(proc.stdout)
    a, b = (float(v) for v in res["loss"][0].split())
    assert abs(a - b) <= 2e-3 * max(1.0, abs(b)), res
    assert float(res["grad_rel"][0]) < 0.08, res


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("backend", ["fused", "nccl"])
def test_bucketed_gradient_reduction_under_backward_matches_the_single_call(backend):
    proc = _torchrun(ROOT / "tests" / "helpers" / "rank_scripts" / "grad_overlap_gpu.py", 2, [backend])
    assert proc.returncode == 0, proc.stdout[-2000:] + proc.stderr[-3000:]
    res = results(proc.stdout)
    assert res["agree"] == ["True"], res
    if backend == "fused":  # rank-ordered sums: bitwise the same whatever the bucketing
        assert res["same"][0].split()[0] == "True", res
    else:
        assert float(res["same"][0].split()[1]) < 1e-4, res


@pytest.mark.skipif(torch.cuda.device_count() < 8, reason="needs eight GPUs")
def test_eight_shards_on_three_axes_match_the_whole_volume_on_gpu():
    proc = _torchrun(ROOT / "tests" / "helpers" / "rank_scripts" / "spatial_gpu.py", 8, ["2,2,2", "fused"], timeout=600)
    assert proc.returncode == 0, proc.stdout[-2000:] + proc.stderr[-3000:]
    res = results(proc.stdout)
    a, b = (float(v) for v in res["loss"][0].split())
    assert abs(a - b) <= 2e-3 * max(1.0, abs(b)), res
    assert float(res["grad_rel"][0]) < 0.08, res


@pytest.mark.skipif(torch.cuda.device_count() < 8, reason="needs eight GPUs")
def test_fused_allreduce_matches_nccl_on_eight_gpus():
    proc = _torchrun(ROOT / "tests" / "helpers" / "rank_scripts" / "fused_allreduce_gpu.py", 8, timeout=600)
    assert proc.returncode == 0, proc.stdout[-2000:] + proc.stderr[-2000:]
    assert results(proc.stdout)["equal"] == ["True"]
