"""Chunked, boundary-masked gated delta rule against the token-by-token recurrence."""
import pytest
import torch

from shadowspill_b200.ops import reference as ref
from shadowspill_b200.ops import sequence as seq


def _case(T, bounds, Hk=2, Hv=4, dk=32, dv=32, seed=0, device="cpu"):
    g = torch.Generator().manual_seed(seed)
    q = seq.l2_normalize(torch.randn(T, Hk, dk, generator=g))
    k = seq.l2_normalize(torch.randn(T, Hk, dk, generator=g))
    v = torch.randn(T, Hv, dv, generator=g)
    beta = torch.sigmoid(torch.randn(T, Hv, generator=g))
    gl = -torch.nn.functional.softplus(torch.randn(T, Hv, generator=g)) * 0.3
    t = [x.to(device) for x in (q, k, v, beta, gl)]
    return t, torch.tensor(bounds, dtype=torch.int32, device=device)


@pytest.mark.parametrize("T,bounds", [
    (256, [0, 256]),                                  # one sequence, whole chunks
    (200, [0, 7, 64, 65, 130, 200]),                  # boundaries inside chunks and on a chunk edge, ragged end
    (192, [0, 1, 2, 3, 100, 192]),                    # one-token sequences
])
def test_chunked_matches_token_recurrence(T, bounds):
    (q, k, v, beta, g), cu = _case(T, bounds)
    want = ref.gated_delta_rule(q, k, v, beta, g, cu)
    got = seq.gated_delta_rule_chunked(q, k, v, beta, g, bounds, 64)
    assert torch.allclose(got, want, rtol=2e-4, atol=2e-5)
    padded_cu = torch.cat([cu, cu[-1:].repeat(5)])    # slot padding of a packed batch
    again = seq.gated_delta_rule_chunked(q, k, v, beta, g, None, 64, cu_seqlens=padded_cu)
    assert torch.allclose(again, want, rtol=2e-4, atol=2e-5)


def test_chunked_gradients_match_token_recurrence():
    T, bounds = 150, [0, 40, 41, 110, 150]
    (q, k, v, beta, g), cu = _case(T, bounds, seed=3)
    dout = torch.randn(T, 4, 32)
    leaves_a = [t.clone().requires_grad_(True) for t in (q, k, v, beta, g)]
    seq.gated_delta_rule_chunked(*leaves_a, bounds, 32).backward(dout)
    leaves_b = [t.clone().requires_grad_(True) for t in (q, k, v, beta, g)]
    ref.gated_delta_rule(*leaves_b, cu).backward(dout)
    for name, a, b in zip("q k v beta g".split(), leaves_a, leaves_b):
        assert torch.allclose(a.grad, b.grad, rtol=2e-3, atol=2e-5), name


def test_linear_scan_adjoint():
    torch.manual_seed(0)
    n, H, dk, dv = 5, 3, 8, 32
    A = (torch.randn(n, H, dk, dk) * 0.3).requires_grad_(True)
    B = torch.randn(n, H, dk, dv).requires_grad_(True)
    S = seq._LinearScan.apply(A.transpose(-1, -2), B)
    X = torch.zeros(H, dk, dv)
    want = []
    for c in range(n):
        want.append(X)
        X = A[c] @ X + B[c]
    want = torch.stack(want)
    assert torch.allclose(S, want, atol=1e-6)
    w = torch.randn_like(S)
    gA, gB = torch.autograd.grad((S * w).sum(), (A, B))
    hA, hB = torch.autograd.grad((want * w).sum(), (A, B))
    assert torch.allclose(gA, hA, atol=1e-5) and torch.allclose(gB, hB, atol=1e-5)
