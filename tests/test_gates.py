"""The numerical gate passes on the CPU plumbing configuration and reports its evidence."""
from shadowspill_b200.qualification.gates import compare_tensors, numerical_gate


def test_numerical_gate_on_cpu():
    rec = numerical_gate("llama3-tiny", "cpu", updates=5)
    assert rec["passed"], rec["failures"]
    assert rec["weights"]["rel_l2"] < 1e-4 and rec["replay_max_abs"] == 0.0
    assert len(rec["losses"]) == 5


def test_compare_tensors_flags_sign_flips():
    import torch
    a = torch.tensor([1.0, -1.0, 0.5, 1e-6])
    b = torch.tensor([1.0, 1.0, 0.5, -1e-6])
    m = compare_tensors(a, b, lr=1e-3)
    assert m["sign_agreement"] < 0.99 and m["near_zero_abs"] < 1e-5


def test_torch_twin_gate_on_cpu():
    """The same gate in fp32 on the CPU is exact to rounding: the planned program and the
    plain-PyTorch twin are two implementations of one model."""
    from shadowspill_b200.models.config import preset
    from shadowspill_b200.qualification.gates import torch_twin_gate
    rec = torch_twin_gate(preset("llama3-tiny"), "cpu", updates=3, tokens=256)
    assert rec["passed"], rec["failures"]
    assert rec["weights"]["rel_l2"] < 1e-4 and rec["fetch_bytes"] > 0


import pytest  # noqa: E402


@pytest.mark.gpu
@pytest.mark.parametrize("family,frontend", [("llama3", "stages"), ("llama3", "graph"), ("qwen35", "stages"),
                                             ("qwen35", "graph"), ("olmoe", "stages"), ("olmoe", "graph")])
def test_planned_bf16_training_matches_the_fp32_pytorch_twin(family, frontend):
    """Five updates of two microbatches, bf16 kernels under a spilling plan, against fp32 eager
    PyTorch + torch.optim.AdamW: weights within rel-L2 2.5 %, cosine 0.999, sign agreement 99 %."""
    from shadowspill_b200.ops import _lib
    from shadowspill_b200.qualification.gates import torch_twin_gate, twin_config
    rec = torch_twin_gate(twin_config(family), "cuda", updates=5, microbatches=2, tokens=1024, frontend=frontend)
    _lib.check_status()
    assert rec["passed"], (rec["failures"], rec["weights"], rec["losses"])
    assert rec["frontend"] == frontend and rec["fetch_bytes"] > 0


def test_divergence_probe_agrees_on_cpu_and_names_a_flipped_bit():
    """Two runs from one seed agree bit for bit on CPU; a single flipped bit in the second run's
    state is found at the update where it happened, with the tensor named."""
    from shadowspill_b200.qualification.nondeterminism import probe
    clean = probe("llama3-tiny", "cpu", updates=2)
    assert clean["diverged_at"] is None and clean["same_plan"] and len(clean["losses"]) == 2
    assert all(a == b for a, b in clean["losses"])
    dirty = probe("llama3-tiny", "cpu", updates=3, perturb_at=2)
    assert dirty["diverged_at"] == 2 and dirty["tensors"][0]["differing"] == 1
    assert dirty["tensors"][0]["tensor"].startswith("embed") and dirty["tensors"][0]["first_index"] == 0


def test_gate_launcher_runs_the_suite_and_the_probe_as_gates(capsys):
    """``gates suite`` runs pytest in child processes and records their last lines; ``gates
    determinism`` runs the divergence probe; the exit status is the conjunction."""
    import json
    from shadowspill_b200.qualification import gates
    rec = gates.suite_gate("cpu", extra=("-k", "test_blake3_known_vectors"))
    assert rec["passed"] and rec["runs"][0]["marker"] == "not gpu" and "passed" in rec["runs"][0]["summary"]
    bad = gates.suite_gate("cpu", extra=("-k", "no_such_test_anywhere"))
    assert not bad["passed"]                       # pytest exits 5 when nothing was collected
    assert gates.main(["determinism", "--device", "cpu"]) == 0
    out = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert out["gate"] == "determinism" and out["passed"] and out["diverged_at"] is None


def test_recorded_floors_are_found_by_hardware_and_configuration():
    from shadowspill_b200.qualification.gates import recorded_floor
    assert recorded_floor("NVIDIA B200", "llama3-8b", 24, 128, 65536) == 15_800.0
    assert recorded_floor("NVIDIA B200", "llama3-8b", 48, 128, 65536) is None       # another budget: no floor
    assert recorded_floor("NVIDIA H100", "llama3-8b", 24, 128, 65536) is None       # another GPU: no floor
