"""Shape calculator, cost model, tolerance policy and census (CPU only)."""
import io
import json

import pytest
import torch

from scaffold_b200.analysis import reference as R
from scaffold_b200.analysis import shapes as S
from scaffold_b200.analysis import unet_shapes as U


def test_traced_parameter_count_matches_the_module():
    from scaffold_b200.models.unet import UNet
    for scale, bott, classes, width in ((5, 3, 6, 16), (6, 3, 9, 8)):
        tr = U.trace_unet(scale, bott, 1, classes - 1, 3, 8, base_width=width)
        with torch.device("meta"):
            m = UNet(3, classes, layers=scale - bott, group_norm_groups=8, base_width=width)
        assert tr.params == sum(p.numel() for p in m.parameters())
        per_block = tr.params_per_block()
        for name, child in list(m.down_list.named_children()):
            assert per_block[f"down_list.{name}"] == sum(p.numel() for p in child.parameters())


def test_scale7_numbers():
    tr = U.trace_unet(7, 3, 2, 8)
    assert tr.params == 90_302_537
    assert tr.ops[0].global_out == (2, 64, 128, 128, 128)
    assert tr.halo_exchanges_fwd == 0
    sharded = U.trace_unet(7, 3, 2, 8, dc_num_shards=(2, 1, 1))
    assert sharded.halo_exchanges_fwd == 18  # one per 3x3x3 convolution
    first = sharded.ops[0]
    assert first.local_out == (2, 64, 64, 128, 128) and first.halo_in == (2, 3, 66, 128, 128)
    assert first.halo_bytes == 2 * 3 * 2 * 128 * 128 * 2


def test_shard_spec_validation_and_report():
    with pytest.raises(ValueError):
        U.trace_unet(5, 3, 1, dc_num_shards=(16, 1, 1))  # the bottleneck is 8 voxels deep
    with pytest.raises(ValueError):
        U.ShardSpec.from_config([2], [1])
    buf = io.StringIO()
    U.print_report(U.trace_unet(5, 3, 1, dc_num_shards=(2, 2, 1)), out=buf)
    assert "halo exchanges per step" in buf.getvalue()
    assert U.main(["--problem-scale", "5", "--json"]) == 0


def test_conv_problem_cost_model():
    p = S.ConvProblem(2, 64, 64, (128, 128, 128))
    assert p.flops() == 2 * 2 * 128 ** 3 * 64 * 64 * 27
    assert p.gemm_shape("fwd") == (2 * 128 ** 3, 64, 64 * 27)
    assert p.gemm_shape("wgrad") == (64, 64 * 27, 2 * 128 ** 3)
    assert p.route("fwd") == "conv_plane3" and p.route("wgrad") == "wgrad_plane"
    assert S.ConvProblem(2, 3, 64, (128, 128, 128)).route("fwd") == "conv_plane"   # 16 padded channels
    wide = S.ConvProblem(2, 128, 256, (32, 32, 32))
    assert wide.route("fwd") == "conv_plane2(pair)" and wide.route("fwd", pair=False) == "conv_plane3"
    assert wide.route("dgrad") == "conv_plane2(pair)"           # backward-data rows = C_in = 128
    assert S.ConvProblem(2, 128, 64, (128, 128, 128)).route("fwd") == "conv_plane3"     # 64 output rows
    assert S.ConvProblem(2, 128, 64, (128, 128, 128)).route("dgrad") == "conv_plane2(pair)"
    assert S.ConvProblem(2, 96, 128, (32, 32, 32)).route("fwd") == "conv_plane3"        # sources not in 64s
    assert S.ConvProblem(2, 512, 1024, (8, 8, 8)).route("fwd") == "conv_small"
    assert S.ConvProblem(2, 64, 128, (4, 4, 4)).route("fwd") == "igemm"
    t = S.ConvProblem(1, 128, 64, (4, 8, 16), 2, True)
    assert t.output_shape == (1, 64, 8, 16, 32) and t.gemm_shape("fwd") == (4 * 8 * 16, 8 * 64, 128)
    h = S.ConvProblem(1, 64, 64, (6, 16, 16), halo=(1, 0, 0))
    assert h.out_spatial == (4, 16, 16)
    assert p.efficiency(p.roofline_seconds() * 1e3) == pytest.approx(1.0)
    assert p.arithmetic_intensity() > 500
    assert S.edge_cases(True)[-1].index_exceeds_int32 and not p.index_exceeds_int32


def test_corpora():
    c = S.scaffold_corpus()
    assert len(c) == 23 and sum(1 for p in c if p.transposed) == 4
    dec = [p for p in c if p.split_cin]
    assert len(dec) == 4 and all(p.split_cin[0] + p.split_cin[1] == p.cin for p in dec)
    sharded = S.scaffold_corpus(shards=(2, 1, 1))
    assert sharded[1].spatial == (66, 128, 128) and sharded[1].out_spatial == (64, 128, 128)
    tot = S.summarize(c)
    assert tot["all"] == pytest.approx(tot["fwd"] + tot["dgrad"] + tot["wgrad"])
    assert len(list(S.all_problems())) == 23 * 3 + len(S.edge_cases())


def test_tolerance_policy():
    g = torch.Generator().manual_seed(0)
    x = R.exact_operand((1, 8, 4, 6, 6), g, density=0.5)
    w = R.exact_operand((4, 8, 3, 3, 3), g, density=0.5)
    assert set(x.unique().tolist()) <= {-1.0, 0.0, 1.0}
    ref = R.conv3d_reference(x, w)
    assert torch.equal(ref, ref.round())
    R.assert_exact(ref.to(torch.bfloat16), ref)
    with pytest.raises(AssertionError):
        R.assert_exact((ref + 1).to(torch.bfloat16), ref)
    xr, wr = torch.randn(1, 8, 4, 6, 6), torch.randn(4, 8, 3, 3, 3)
    refr = R.conv3d_reference(xr.bfloat16(), wr.bfloat16())
    got = torch.nn.functional.conv3d(xr.bfloat16().float(), wr.bfloat16().float(), padding=1).bfloat16()
    R.assert_close(got, refr, k_terms=8 * 27)
    with pytest.raises(AssertionError):
        R.assert_close(got * 1.05, refr, k_terms=8 * 27)


def test_census_counts_launcher_calls(monkeypatch):
    from scaffold_b200.analysis.census import ConvCensus, make_corpus, problem_of
    from scaffold_b200.ops import conv_kernels as ck
    calls = []
    monkeypatch.setattr(ck, "conv_same", lambda *a, **k: calls.append("same") or ["y"])
    monkeypatch.setattr(ck, "conv_wgrad", lambda *a, **k: calls.append("wgrad"))
    x = torch.zeros(2, 4, 8, 16, 64)
    with ConvCensus() as c:
        ck.conv_same([x], None, 3, [64])
        ck.conv_same([x], None, 3, [64])
        ck.conv_wgrad(x, [x], 3, None)
    assert calls == ["same", "same", "wgrad"]
    recs = c.records()
    assert recs[0]["count"] == 2 and recs[0]["op"] == "conv_same" and recs[0]["dims"] == [4, 8, 16]
    assert problem_of(recs[0]).flops() == 2 * 2 * 4 * 8 * 16 * 64 * 64 * 27
    corpus = make_corpus(recs, [{"op": "conv_fwd", "cin": 64, "cout": 64, "size": 16, "batch": 2, "ms": 0.5}])
    assert corpus[0]["measured_ms"] == 0.5 and corpus[0]["route"] == "conv_plane3"
    json.dumps(corpus)
    assert ck.conv_same([x], None, 3, [64]) == ["y"]  # launchers restored


def test_committed_corpus_fixture_matches_the_analytic_corpus():
    from scaffold_b200.analysis import corpus
    from scaffold_b200.analysis.shapes import scaffold_corpus
    doc = corpus.load()
    probs = scaffold_corpus(7, 3, 2)
    assert sum(layer["count"] for layer in doc["layers"]) == len(probs)
    labels = {p.label for p in probs}
    assert {layer["label"] for layer in doc["layers"]} == labels
    for layer in doc["layers"]:
        for d in ("fwd", "dgrad", "wgrad"):
            e = layer["directions"][d]
            assert e["flops"] > 0 and e["roofline_ms"] > 0 and e["route"]
            if "ms" in e:  # measured rows carry the paired ratio and its interval
                assert e["ms"] > 0 and e["library_ms"] > 0 and e["ci"][0] <= e["ratio"] <= e["ci"][1]
    # the fixture answers "which layers matter": the 128^3 layers hold most of the forward time
    big = sum(layer["count"] * layer["directions"]["fwd"].get("ms", 0) for layer in doc["layers"]
              if layer["spatial"][0] == 128)
    assert big > 0.4 * doc["totals"]["fwd"]["ms_per_step"]
    rebuilt = corpus.build([], 7, 2)
    assert [layer["label"] for layer in rebuilt["layers"]] == [layer["label"] for layer in doc["layers"]]


def test_paired_ratio_statistics():
    from scaffold_b200.bench.harness import ratio_ci, t95
    import math
    g, lo, hi = ratio_ci([math.log(2.0)] * 6)
    assert abs(g - 2.0) < 1e-12 and abs(lo - 2.0) < 1e-9 and abs(hi - 2.0) < 1e-9
    g, lo, hi = ratio_ci([math.log(v) for v in (1.9, 2.0, 2.1, 2.0, 1.95, 2.05)])
    assert lo < g < hi and 1.9 < lo and hi < 2.1
    assert t95(2) > t95(10) > t95(100) == 1.96 and math.isinf(t95(1))
