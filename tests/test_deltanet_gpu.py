"""DeltaNet elementwise kernels (conv+SiLU, L2 norm, gated RMSNorm) against the fp32
PyTorch definitions, forward and backward."""
import pytest
import torch

from shadowspill_b200.ops import sequence as seq

pytestmark = pytest.mark.gpu


def _rel(a, b):
    a, b = a.detach().float(), b.detach().float()
    return float((a - b).norm() / b.norm().clamp_min(1e-9))


def _positions(bounds, device):
    pos = torch.zeros(bounds[-1], dtype=torch.int32, device=device)
    for s, e in zip(bounds[:-1], bounds[1:]):
        pos[s:e] = torch.arange(e - s, device=device, dtype=torch.int32)
    return pos


@pytest.mark.parametrize("K", [4, 2, 7])
def test_conv_silu_forward_backward(K):
    torch.manual_seed(0)
    bounds = [0, 1, 4, 300, 301, 777, 1024]         # includes sequences shorter than the window
    T, C, full = 1024, 640, 896
    buf = (torch.randn(T, full, device="cuda") * 0.7).bfloat16()
    w = (torch.randn(C, K, device="cuda") * 0.4).bfloat16()
    dy = torch.randn(T, C, device="cuda").bfloat16()
    pos = _positions(bounds, "cuda")
    xk = buf[:, :C].clone().requires_grad_(True)     # contiguous copy and strided view both work
    xv = buf.clone().requires_grad_(True)
    wk = w.clone().requires_grad_(True)
    y = seq.causal_conv_silu(xv[:, :C], wk, bounds, pos)
    y.backward(dy)
    xr = buf[:, :C].float().requires_grad_(True)
    wr = w.float().requires_grad_(True)
    want = seq.causal_conv_silu(xr, wr, bounds)
    want.backward(dy.float())
    assert _rel(y, want) < 6e-3
    assert _rel(xv.grad[:, :C], xr.grad) < 1e-2
    assert float(xv.grad[:, C:].abs().max()) == 0.0
    assert _rel(wk.grad, wr.grad) < 1e-2
    y2 = seq.causal_conv_silu(xk, w, bounds, pos)
    assert torch.equal(y2, y)


def test_l2_normalize_forward_backward():
    torch.manual_seed(1)
    x = torch.randn(3000, 6, 128, device="cuda").bfloat16()
    dy = torch.randn_like(x)
    xk = x.clone().requires_grad_(True)
    y = seq.l2_normalize(xk)
    y.backward(dy)
    xr = x.float().requires_grad_(True)
    want = seq.l2_normalize(xr)
    want.backward(dy.float())
    assert _rel(y, want) < 5e-3 and _rel(xk.grad, xr.grad) < 1e-2
    assert abs(float(y.float().square().sum(-1).mean()) - 1.0) < 1e-2


@pytest.mark.parametrize("zero_centered", [False, True])
def test_gated_rmsnorm_forward_backward(zero_centered):
    torch.manual_seed(2)
    x = torch.randn(2000, 8, 128, device="cuda").bfloat16()
    gate = torch.randn_like(x)
    w = (torch.randn(128, device="cuda") * 0.2 + (0.0 if zero_centered else 1.0)).bfloat16()
    dy = torch.randn_like(x)
    xk, gk, wk = (t.clone().requires_grad_(True) for t in (x, gate, w))
    y = seq.gated_rmsnorm(xk, gk, wk, 1e-6, zero_centered)
    y.backward(dy)
    xr, gr, wr = (t.float().requires_grad_(True) for t in (x, gate, w))
    want = seq.gated_rmsnorm(xr, gr, wr, 1e-6, zero_centered)
    want.backward(dy.float())
    assert _rel(y, want) < 6e-3
    assert _rel(xk.grad, xr.grad) < 1.5e-2 and _rel(gk.grad, gr.grad) < 1.5e-2
    assert _rel(wk.grad, wr.grad) < 1.5e-2


def test_linear_scan_kernel_matches_loop():
    torch.manual_seed(0)
    n, H, dk, dv = 9, 5, 64, 64
    A = torch.randn(n, H, dk, dk, device="cuda") * 0.1
    B = torch.randn(n, H, dk, dv, device="cuda")
    for reverse in (False, True):
        got = seq._LinearScan.run(A, B, reverse)
        want = seq._LinearScan.run(A.cpu(), B.cpu(), reverse)
        assert _rel(got.cpu(), want) < 1e-5


def test_gated_delta_rule_on_gpu_matches_token_recurrence():
    from shadowspill_b200.ops import reference as ref
    torch.manual_seed(1)
    T, Hk, Hv, dk = 704, 2, 4, 64
    bounds = [0, 5, 300, 301, 640, 704]
    q = seq.l2_normalize(torch.randn(T, Hk, dk))
    k = seq.l2_normalize(torch.randn(T, Hk, dk))
    v = torch.randn(T, Hv, dk)
    beta = torch.sigmoid(torch.randn(T, Hv))
    g = -torch.nn.functional.softplus(torch.randn(T, Hv)) * 0.3
    cu = torch.tensor(bounds + [T] * 4, dtype=torch.int32)
    dout = torch.randn(T, Hv, dk)
    cpu = [t.clone().requires_grad_(True) for t in (q, k, v, beta, g)]
    want = ref.gated_delta_rule(*cpu, torch.tensor(bounds))
    want.backward(dout)
    dev = [t.clone().cuda().requires_grad_(True) for t in (q, k, v, beta, g)]
    got = seq.gated_delta_rule_chunked(*dev, None, 64, cu_seqlens=cu.cuda())
    got.backward(dout.cuda())
    assert _rel(got.cpu(), want) < 2e-3            # TF32 products
    for name, a, b in zip("q k v beta g".split(), dev, cpu):
        assert _rel(a.grad.cpu(), b.grad) < 1e-2, name
