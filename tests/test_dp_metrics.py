"""Data-parallel metric reductions on 2 gloo ranks with an odd, unpadded validation split
(role of tests/helpers/rank_scripts/metrics_train_2rank.py in the reference)."""
from helpers.launch import ROOT, results, torchrun_gloo


def test_validation_sums_over_two_replicas_equal_the_single_process_values():
    proc = torchrun_gloo(ROOT / "tests" / "helpers" / "rank_scripts" / "metrics_2rank.py", 2)
    assert proc.returncode == 0, proc.stdout[-2000:] + proc.stderr[-3000:]
    res = results(proc.stdout)
    assert res["counts"] == ["5 5"]
    for key in ("dice", "loss"):
        a, b = (float(v) for v in res[key][0].split())
        assert abs(a - b) <= 1e-5 * max(1.0, abs(b)), (key, a, b)
