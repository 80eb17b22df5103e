"""Config schema, CLI merge precedence, run-directory rules and the restart script (CPU only)."""
import os
from pathlib import Path

import pytest
import yaml

from scaffold_b200 import cli
from scaffold_b200 import config as C
from scaffold_b200.utils import restart_script


def base_dict(tmp_path, **kw):
    d = yaml.safe_load(C.default_config_path().read_text())
    d.update(base_run_dir=str(tmp_path / "runs"), dataset_dir=str(tmp_path / "ds"), fract_base_dir=str(tmp_path / "fr"))
    d.update(kw)
    return d


def test_defaults_load_and_derive(tmp_path):
    cfg = C.Config(base_dict(tmp_path))
    assert cfg.unet_layers == 4 and cfg.vol_size == 128 and cfg.point_num == 128 ** 3 // 256
    assert cfg.dc_total_shards == 1 and cfg.gn_stats == "global" and cfg.unet_base_width == 64


def test_unknown_key_rejected_and_sweeps_rejected(tmp_path):
    with pytest.raises(ValueError, match="Unknown config key"):
        C.Config(base_dict(tmp_path, not_a_key=1))
    with pytest.raises(ValueError, match="sweeps are no longer supported"):
        C.Config(base_dict(tmp_path, problem_scale=[6, 7]))


@pytest.mark.parametrize("bad", [dict(dist=0), dict(unet_bottleneck_dim=7), dict(unet_bottleneck_dim=-1),
                                 dict(n_categories=0), dict(dataset_seed=-1), dict(activation_checkpointing=2),
                                 dict(dc_num_shards=[1, 2]), dict(gn_stats="nope")])
def test_bad_values_rejected(tmp_path, bad):
    with pytest.raises((ValueError, KeyError)):
        C.Config(base_dict(tmp_path, **bad))


def test_dumped_config_reloads(tmp_path):
    cfg = C.Config(base_dict(tmp_path))
    dumped = {k: v for k, v in cfg.to_dict().items()}
    C.Config(dumped)  # derived keys (unet_layers, vol_size, ...) are accepted on input


def test_override_files_merge_and_reject_unknown(tmp_path):
    base, ov, bad = tmp_path / "b.yml", tmp_path / "o.yml", tmp_path / "x.yml"
    base.write_text(yaml.safe_dump(base_dict(tmp_path)))
    ov.write_text(yaml.safe_dump({"problem_scale": 5}))
    bad.write_text(yaml.safe_dump({"problem_scael": 5}))
    assert C.load_config_files([str(base), str(ov)])["problem_scale"] == 5
    with pytest.raises(ValueError, match="override file"):
        C.load_config_files([str(base), str(bad)])


def _args(tmp_path, *extra):
    base = tmp_path / "b.yml"
    base.write_text(yaml.safe_dump(base_dict(tmp_path, problem_scale=5)))
    argv = ["benchmark", "-c", str(base), *extra]
    return cli.build_parser().parse_args(argv), argv


def test_cli_flag_beats_file_and_artefacts_are_written(tmp_path):
    args, argv = _args(tmp_path, "--problem-scale", "4", "--dc-num-shards", "1", "1", "2")
    merged = cli.build_run_config(args, argv)
    assert merged["problem_scale"] == 4 and merged["vol_size"] == 16 and merged["unet_layers"] == 1
    assert merged["dc_num_shards"] == [1, 1, 2]
    run_dir = Path(merged["run_dir"])
    assert run_dir.parent == tmp_path / "runs" and not merged["restart"]
    for name in ("config.yaml", "overrides.yaml", "restart.sh"):
        assert (run_dir / name).exists()
    assert yaml.safe_load((run_dir / "overrides.yaml").read_text()) == {"problem_scale": 4, "dc_num_shards": [1, 1, 2]}
    dumped = yaml.safe_load((run_dir / "config.yaml").read_text())
    assert dumped["run_dir"] is None  # a fresh run's config does not turn into a resume when replayed
    C.Config(dumped)
    assert os.access(run_dir / "restart.sh", os.X_OK)


def test_restart_without_run_dir_is_rejected_before_any_directory(tmp_path):
    args, argv = _args(tmp_path, "--restart")
    with pytest.raises(ValueError, match="no run directory"):
        cli.build_run_config(args, argv)
    assert not (tmp_path / "runs").exists()


def test_run_dir_resumes_and_needs_a_checkpoint(tmp_path):
    rd = tmp_path / "old_run"
    args, argv = _args(tmp_path, "--run-dir", str(rd))
    merged = cli.build_run_config(args, argv)
    assert merged["restart"] is True and merged["train_from_scratch"] is False and merged["run_dir"] == str(rd)
    assert "no checkpoint" in cli.missing_checkpoint_error(merged)
    (rd / "checkpoints").mkdir()
    (rd / "checkpoints" / "checkpoint_best.pth").write_bytes(b"x")
    assert cli.missing_checkpoint_error(merged) is None


def test_bad_config_creates_no_run_dir(tmp_path):
    args, argv = _args(tmp_path, "--unet-bottleneck-dim", "9")
    with pytest.raises(ValueError):
        cli.build_run_config(args, argv)
    assert not (tmp_path / "runs").exists()


def test_restart_script_rewrites_argv():
    out = restart_script.rewrite_argv(["benchmark", "-c", "a.yml", "-c", "b.yml", "--base-run-dir", "x",
                                       "--job-name=foo", "--problem-scale", "6", "--restart", "--run-dir", "old"])
    assert out == ["benchmark", "-c", "$RUN_DIR/config.yaml", "--problem-scale", "6", "--restart", "--run-dir",
                   "$RUN_DIR"]
    text = restart_script.render(Path("/tmp/r"), ["benchmark", "-c", "a.yml"])
    assert 'RUN_DIR="$(cd' in text and "--restart --run-dir $RUN_DIR" in text


def test_grad_overlap_key_and_flag(tmp_path):
    merged = C.load_config_files([str(C.default_config_path())])
    assert C.Config(dict(merged, base_run_dir=str(tmp_path))).grad_overlap is True  # on by default; the flag turns it off
    args = cli.build_parser().parse_args(["benchmark", "--grad-overlap", "0"])
    assert "grad_overlap" in cli.explicit_cli_keys(args) and args.grad_overlap == 0


def test_superset_keys_have_b200_defaults_and_validate(tmp_path):
    cfg = C.Config(base_dict(tmp_path))
    assert cfg.grad_allreduce == "fused" and cfg.halo_exchange == "fused"
    assert cfg.grad_overlap is True and cfg.allow_fallback is False and cfg.datagen_device == "auto"
    off = C.Config(base_dict(tmp_path, grad_overlap=0, allow_fallback=1, grad_allreduce="nccl", halo_exchange="nccl",
                             gn_stats="per_shard", unet_base_width=32))
    assert off.grad_overlap is False and off.allow_fallback is True and off.unet_base_width == 32
    for bad in (dict(grad_allreduce="mpi"), dict(halo_exchange="rdma"), dict(unet_base_width=0),
                dict(datagen_device="tpu")):
        with pytest.raises((ValueError, KeyError)):
            C.Config(base_dict(tmp_path, **bad))


@pytest.mark.parametrize("scale,bottleneck,layers", [(7, 3, 4), (8, 3, 5), (9, 3, 6), (5, 2, 3)])
def test_network_depth_follows_scale_and_bottleneck(tmp_path, scale, bottleneck, layers):
    cfg = C.Config(base_dict(tmp_path, problem_scale=scale, unet_bottleneck_dim=bottleneck))
    assert cfg.unet_layers == layers and cfg.vol_size == 2 ** scale


def test_cli_flags_for_the_fused_paths_reach_the_config(tmp_path):
    base = tmp_path / "b.yml"
    base.write_text(yaml.safe_dump(base_dict(tmp_path, problem_scale=5)))
    parser = cli.build_parser()
    ns = parser.parse_args(["benchmark", "-c", str(base), "--grad-overlap", "0", "--allow-fallback", "1",
                            "--halo-exchange", "nccl", "--dc-num-shards", "1", "1", "2"])
    assert ns.grad_overlap == 0 and ns.allow_fallback == 1 and ns.halo_exchange == "nccl"
    assert ns.dc_num_shards == [1, 1, 2]


def test_validation_cache_budget_flag_parses_as_a_number(tmp_path):
    base = tmp_path / "b.yml"
    base.write_text(yaml.safe_dump(base_dict(tmp_path, problem_scale=5)))
    ns = cli.build_parser().parse_args(["benchmark", "-c", str(base), "--val-cache-gb", "0.5"])
    assert ns.val_cache_gb == 0.5
    assert C.Config(base_dict(tmp_path, val_cache_gb=ns.val_cache_gb)).val_cache_gb == 0.5
    assert C.Config(base_dict(tmp_path, val_cache_gb=2)).val_cache_gb == 2.0      # an integer in the YAML is fine
    with pytest.raises(ValueError, match="non-negative number"):
        C.Config(base_dict(tmp_path, val_cache_gb=True))                          # a boolean is a typo here
