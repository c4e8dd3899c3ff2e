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
