"""Rank / world size / local rank from the environment of each supported launcher, before any process group exists
(role of ScaFFold/utils/distributed.py:28-160 and the launcher matrices of ScaFFold/cli.py:584-662)."""
import pytest

from scaffold_b200.utils import dist as D

ALL_VARS = set(D._RANK_VARS) | set(D._SIZE_VARS) | set(D._LOCAL_RANK_VARS) | set(D._LOCAL_SIZE_VARS)


@pytest.fixture
def clean_env(monkeypatch):
    for v in ALL_VARS:
        monkeypatch.delenv(v, raising=False)
    return monkeypatch


LAUNCHERS = {
    "torchrun": dict(RANK="5", WORLD_SIZE="8", LOCAL_RANK="1", LOCAL_WORLD_SIZE="4"),
    "openmpi": dict(OMPI_COMM_WORLD_RANK="5", OMPI_COMM_WORLD_SIZE="8", OMPI_COMM_WORLD_LOCAL_RANK="1",
                    OMPI_COMM_WORLD_LOCAL_SIZE="4"),
    "mvapich": dict(MV2_COMM_WORLD_RANK="5", MV2_COMM_WORLD_SIZE="8", MV2_COMM_WORLD_LOCAL_RANK="1",
                    MV2_COMM_WORLD_LOCAL_SIZE="4"),
    "pals": dict(PALS_RANKID="5", PALS_NRANKS="8", PALS_LOCAL_RANKID="1", PALS_LOCAL_SIZE="4"),
    "slurm": dict(SLURM_PROCID="5", SLURM_NTASKS="8", SLURM_LOCALID="1", SLURM_NTASKS_PER_NODE="4"),
    "slurm_tasklist": dict(SLURM_PROCID="5", SLURM_NTASKS="8", SLURM_LOCALID="1", SLURM_TASKS_PER_NODE="4(x2)"),
}


@pytest.mark.parametrize("name", sorted(LAUNCHERS))
def test_each_launcher_environment_gives_the_same_answers(clean_env, name):
    for k, v in LAUNCHERS[name].items():
        clean_env.setenv(k, v)
    assert (D.get_world_rank(), D.get_world_size(), D.get_local_rank(), D.get_local_size()) == (5, 8, 1, 4)


def test_single_process_defaults_and_priority(clean_env):
    assert (D.get_world_rank(), D.get_world_size(), D.get_local_rank()) == (0, 1, 0)
    clean_env.setenv("SLURM_PROCID", "3")
    clean_env.setenv("RANK", "1")                      # torchrun's variables win over the scheduler's
    assert D.get_world_rank() == 1
    clean_env.setenv("RANK", "not a number")           # unreadable: the next launcher in the list decides
    assert D.get_world_rank() == 3


def test_tolerant_integer_parse():
    assert D._to_int("4") == 4 and D._to_int(" 4 ") == 4 and D._to_int("4(x2)") == 4 and D._to_int("16,16") == 16
    assert D._to_int(None) is None and D._to_int("") is None and D._to_int("x4") is None


def test_launcher_world_size_check_is_silent_without_a_group(clean_env):
    clean_env.setenv("WORLD_SIZE", "8")
    D.check_launcher_world_size()                      # no process group: nothing to compare


def test_cpu_only_machine_gets_the_cpu_device(monkeypatch):
    import torch
    monkeypatch.setattr(torch.cuda, "is_available", lambda: False)
    assert D.get_device() == torch.device("cpu")
    with pytest.raises(ValueError, match="unknown rendezvous"):
        monkeypatch.setattr(D.dist, "is_initialized", lambda: False)
        D.initialize_dist(rendezvous="carrier pigeon")
