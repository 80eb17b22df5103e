"""Control-plane sequencing on fake communicators (no process group): who decides, what is broadcast,
and how one rank's failure reaches every rank. Role of the reference's tests with fake MPI communicators
(tests/datagen/test_mpi_consensus.py)."""
import hashlib
from pathlib import Path

import numpy as np
import pytest

from scaffold_b200.utils import dist as D


class FakeWorld:
    """Replays one collective program for ``size`` ranks sequentially: every rank's contribution is recorded
    first (pass 1), then each rank re-runs and receives everybody's (pass 2)."""

    def __init__(self, size):
        self.size = size
        self.rank = 0
        self.gathered = {}
        self.bcast = {}
        self.calls = 0
        self.replay = False

    def patch(self, monkeypatch):
        monkeypatch.setattr(D, "get_world_rank", lambda: self.rank)
        monkeypatch.setattr(D, "get_world_size", lambda: self.size)
        monkeypatch.setattr(D, "allgather_obj", self.allgather)
        monkeypatch.setattr(D, "bcast_obj", self.broadcast)

    def allgather(self, obj):
        slot = self.gathered.setdefault(self.calls, [None] * self.size)
        slot[self.rank] = obj
        self.calls += 1
        return list(slot)

    def broadcast(self, obj, src=0):
        if self.rank == src:
            self.bcast[self.calls] = obj
        out = self.bcast.get(self.calls)
        self.calls += 1
        return out

    def run(self, program):
        """Run ``program(rank)`` for every rank twice; return the second pass's outcomes (value or exception)."""
        outcomes = []
        for final in (False, True):
            outcomes = []
            for r in range(self.size):
                self.rank, self.calls = r, 0
                try:
                    outcomes.append(program(r))
                except Exception as exc:  # noqa: BLE001
                    outcomes.append(exc)
        return outcomes


def test_consensus_with_one_failing_rank_raises_everywhere(monkeypatch):
    world = FakeWorld(4)
    world.patch(monkeypatch)

    def program(rank):
        D.consensus(rank != 2, f"volume {rank} could not be written")
        return "ok"
    out = world.run(program)
    assert all(isinstance(o, D.RemoteError) for o in out)
    assert all("rank 2: volume 2 could not be written" in str(o) for o in out)
    assert "rank 1" not in str(out[0])


def test_consensus_passes_when_every_rank_succeeded(monkeypatch):
    world = FakeWorld(3)
    world.patch(monkeypatch)
    assert world.run(lambda r: D.consensus(True) or "ok") == ["ok"] * 3


def test_root_failure_is_rebuilt_with_its_class_and_origin_on_every_rank(monkeypatch):
    world = FakeWorld(3)
    world.patch(monkeypatch)

    def program(rank):
        def decide():
            raise FileNotFoundError("no fractal library at /data/fr")
        return D.run_on_root(decide)
    out = world.run(program)
    assert all(isinstance(o, FileNotFoundError) for o in out)
    assert all("[rank 0]" in str(o) and "no fractal library" in str(o) for o in out)


def test_root_decides_and_the_others_never_run_the_decision(monkeypatch):
    world = FakeWorld(4)
    world.patch(monkeypatch)
    ran = []

    def program(rank):
        def decide():
            ran.append(rank)
            return {"run_dir": "/runs/000", "run_iter": 3}
        return D.run_on_root(decide)
    out = world.run(program)
    assert set(ran) == {0}
    assert all(o == {"run_dir": "/runs/000", "run_iter": 3} for o in out)


def test_unknown_exception_classes_become_remote_errors():
    err = D.rebuild_error({"type": "CheckpointSaveError", "module": "x", "message": "disk full", "rank": 5})
    assert isinstance(err, D.RemoteError) and "rank 5" in str(err) and "CheckpointSaveError" in str(err)
    err = D.rebuild_error({"type": "ValueError", "module": "builtins", "message": "bad", "rank": 1})
    assert isinstance(err, ValueError)


def test_id_digest_guard_names_the_disagreeing_ranks(monkeypatch):
    from scaffold_b200.data.dataset import FractalDataset
    world = FakeWorld(3)
    world.patch(monkeypatch)
    lists = [["0", "1", "2"], ["0", "1", "2"], ["0", "1", "2", "3"]]  # rank 2 sees an extra volume

    def program(rank):
        ds = object.__new__(FractalDataset)
        ds.ids, ds.images_dir = lists[rank], Path("/data/volumes/training")
        ds.check_ids_across_ranks()
        return "ok"
    out = world.run(program)
    assert all(isinstance(o, RuntimeError) and "ranks [2] disagree" in str(o) for o in out)
    lists[2] = ["0", "1", "2"]
    world2 = FakeWorld(3)
    world2.patch(monkeypatch)
    assert world2.run(program) == ["ok"] * 3
    assert FractalDataset.ids_digest(type("X", (), {"ids": ["0", "1"]})()) == hashlib.sha256(b"0\n1").digest()


def test_unpadded_sampler_gives_every_sample_to_exactly_one_replica():
    from scaffold_b200.train.trainer import UnpaddedDistributedSampler
    for n, world in ((5, 2), (7, 3), (2, 4), (8, 8)):
        seen = []
        for r in range(world):
            s = UnpaddedDistributedSampler(range(n), world, r)
            assert len(s) == len(list(s))
            seen += list(s)
        assert sorted(seen) == list(range(n))  # no padding, no duplicates: validation sums are exact


def test_round_size_and_attempt_counters_are_per_rank(tmp_path):
    from scaffold_b200.data import category_search as cs
    assert cs.load_attempt_counter(tmp_path, 3) == 0
    cs.store_attempt_counter(tmp_path, 3, 41)
    cs.store_attempt_counter(tmp_path, 1, 7)
    assert cs.load_attempt_counter(tmp_path, 3) == 41 and cs.load_attempt_counter(tmp_path, 1) == 7
    # proposals depend on (seed, rank, attempt) only: a restarted rank continues its own stream
    a = cs.propose_params(11, 3, 41)
    assert np.array_equal(a, cs.propose_params(11, 3, 41)) and not np.array_equal(a, cs.propose_params(11, 1, 41))
    assert 1 <= cs.round_size(5, 0, 0, 64, 4) <= 64
