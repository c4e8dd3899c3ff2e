"""Artifact archives: round trips, atomic replacement, integrity checks."""
import zipfile

import numpy as np
import pytest
import torch

from shadowspill_b200.artifacts import (ArtifactError, TensorChunk, archive_kind, load_archive,
                                        load_artifact, save_archive, save_artifact)
from shadowspill_b200.communication.info import CommunicationInfo
from shadowspill_b200.frontend.capture import BatchGeometry, StepDataOrdering, build_step
from shadowspill_b200.models.config import preset
from shadowspill_b200.planning.plan import MemoryBudgets, SearchOptions, sweep_programs


def _program():
    geo = BatchGeometry(microbatch_tokens=256, n_microbatches=2, slots=16, mean_seqlen=64)
    return build_step(preset("llama3-tiny"), geo, StepDataOrdering(), dtype=torch.float32)[0]


def test_program_plan_and_sweep_round_trip(tmp_path):
    prog = _program()
    assert save_artifact(prog, tmp_path / "p.ssa") == "program"
    again = load_artifact(tmp_path / "p.ssa", "program")
    assert again.to_json() == prog.to_json()
    total = sum(o.bytes for o in prog.objects)
    sweep = sweep_programs([prog], MemoryBudgets(2 * total, 64 << 20, headroom_bytes=0),
                           CommunicationInfo(), SearchOptions(workers=1))
    save_artifact(sweep, tmp_path / "s.ssa")
    got = load_artifact(tmp_path / "s.ssa")
    assert got.best.to_json() == sweep.best.to_json() and got.errors == sweep.errors
    save_artifact(sweep.best, tmp_path / "plan.ssa")
    assert archive_kind(tmp_path / "plan.ssa") == "plan"
    with pytest.raises(ArtifactError):
        load_artifact(tmp_path / "plan.ssa", "program")
    save_artifact(MemoryBudgets(1 << 30, 2 << 30), tmp_path / "b.ssa")
    assert load_artifact(tmp_path / "b.ssa").spill_bytes == 2 << 30
    save_artifact(CommunicationInfo(world_size=4), tmp_path / "c.ssa")
    assert load_artifact(tmp_path / "c.ssa").world_size == 4


def test_equal_payloads_are_stored_once_and_verified(tmp_path):
    blob = b"x" * 4096
    path = save_archive(tmp_path / "a.ssa", "program", {"k": 1}, {"one": blob, "two": blob, "three": b"y"})
    with zipfile.ZipFile(path) as z:
        assert sum(n.startswith("payloads/") for n in z.namelist()) == 2
    meta, payloads = load_archive(path)
    assert meta == {"k": 1} and payloads["one"] == payloads["two"] == blob
    # flip one payload byte: the digest check must refuse the archive
    raw = bytearray(path.read_bytes())
    at = raw.find(b"x" * 64)
    raw[at] ^= 1
    bad = tmp_path / "bad.ssa"
    bad.write_bytes(bytes(raw))
    with pytest.raises((ArtifactError, zipfile.BadZipFile)):
        load_archive(bad)


def test_failed_save_leaves_the_old_archive(tmp_path):
    path = save_archive(tmp_path / "a.ssa", "budgets", {"v": 1})
    with pytest.raises(ArtifactError):
        save_archive(path, "budgets", {"v": 2}, {"big": b"0" * 100_000}, max_bytes=1000)
    assert load_archive(path)[0] == {"v": 1}
    assert [p.name for p in tmp_path.iterdir()] == ["a.ssa"]           # no temporary left behind


def test_tensor_chunk(tmp_path):
    data = np.arange(100, dtype=np.float32)
    save_artifact(TensorChunk("layer0.wqkv", "float32", (20, 10), 50, data), tmp_path / "t.ssa")
    c = load_artifact(tmp_path / "t.ssa")
    assert c.name == "layer0.wqkv" and c.start == 50 and np.array_equal(c.data, data)
    with pytest.raises(ArtifactError):
        TensorChunk("w", "float32", (4, 4), 10, np.zeros(10, np.float32))
