"""Slurm job facts are read, bounded and never trusted beyond what they say."""
import json

import pytest

from shadowspill_b200.orchestration import slurm


def test_hostlist_expansion():
    assert slurm.expand_hostlist("node[01-03,07],gpu5") == ["node01", "node02", "node03", "node07", "gpu5"]
    assert slurm.expand_hostlist("a1") == ["a1"] and slurm.expand_hostlist("") == []
    with pytest.raises(ValueError):
        slurm.expand_hostlist("n[0-99999]")


def test_detect_and_clamp():
    assert slurm.detect({}) is None
    env = {"SLURM_JOB_ID": "4242", "SLURM_JOB_NODELIST": "b200-[1-2]", "SLURM_CPUS_ON_NODE": "48",
           "SLURM_MEM_PER_NODE": "204800", "SLURM_GPUS_ON_NODE": "4", "SLURM_JOB_UID": "1000",
           "SLURMD_NODENAME": "b200-2"}
    job = slurm.detect(env)
    assert job.job_id == 4242 and sorted(job.nodes) == ["b200-1", "b200-2"] and job.nodes["b200-2"].gpus == 4
    inv = {"gpus": 8, "gpu_names": ["B200"] * 8, "cpus": 224, "host_total_gib": 2000.0, "host_free_gib": 1900.0}
    got = slurm.clamp_inventory(inv, job, "b200-2")
    assert got["gpus"] == 4 and len(got["gpu_names"]) == 4 and got["cpus"] == 48
    assert got["host_free_gib"] == 200.0 and got["slurm_job"] == "4242"
    assert slurm.clamp_inventory(inv, None) is inv
    assert slurm._gpu_count("gpu:b200:4") == 4 and slurm._gpu_count("0,1,2") == 3 and slurm._gpu_count("") == 0


def test_parse_job_checks_identity_and_size():
    doc = {"jobs": [{"job_id": 7, "user_id": 1000, "nodes": "n[1-2]", "tres_per_node": "gres/gpu:8",
                     "job_resources": {"nodes": {"allocation": [
                         {"name": "n1", "cpus": {"count": 32}, "memory": {"allocated": 65536}},
                         {"name": "n2", "cpus": {"count": 32}, "memory": {"allocated": 65536}}]}}}], "errors": []}
    job = slurm.parse_job(json.dumps(doc).encode(), job_id=7, user_id=1000)
    assert job.nodes["n2"].cpus == 32 and job.nodes["n1"].memory_mib == 65536 and job.nodes["n1"].gpus == 8
    for kw in ({"job_id": 8, "user_id": 1000}, {"job_id": 7, "user_id": 1}):
        with pytest.raises(ValueError):
            slurm.parse_job(json.dumps(doc).encode(), **kw)
    with pytest.raises(ValueError):
        slurm.parse_job(json.dumps({"jobs": [], "errors": []}).encode(), job_id=7, user_id=1000)
    with pytest.raises(ValueError):
        slurm.parse_job(json.dumps({"jobs": doc["jobs"], "errors": [{"error": "x"}]}).encode(), job_id=7, user_id=1000)
    with pytest.raises(ValueError):
        slurm.parse_job(b" " * (slurm.MAX_RESPONSE_BYTES + 1), job_id=7, user_id=1000)
