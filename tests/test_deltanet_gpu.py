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


def _delta_case(T, Hk, Hv, bounds, seed):
    g = torch.Generator().manual_seed(seed)
    nrm = lambda x: x / x.norm(dim=-1, keepdim=True)
    q = nrm(torch.randn(T, Hk, 128, generator=g)).bfloat16()
    k = nrm(torch.randn(T, Hk, 128, generator=g)).bfloat16()
    v = torch.randn(T, Hv, 128, generator=g).bfloat16()
    beta = torch.sigmoid(torch.randn(T, Hv, generator=g))
    gl = -torch.nn.functional.softplus(torch.randn(T, Hv, generator=g)) * 0.3
    dout = (torch.randn(T, Hv, 128, generator=g) * 0.5).bfloat16()
    cu = torch.tensor(bounds + [T] * 3, dtype=torch.int32)
    return q, k, v, beta, gl, dout, cu


@pytest.mark.parametrize("T,Hk,Hv,bounds", [
    (333, 2, 4, [0, 5, 130, 131, 300, 333]),        # T not a multiple of 64, boundaries at odd offsets
    (200, 1, 3, [0, 77, 200]),                      # three V heads per QK head: a pair and a single
    (256, 2, 2, [0, 64, 191, 256]),                 # one V head per QK head, a boundary on a chunk edge
])
def test_delta_rule_kernels_match_the_token_recurrence(T, Hk, Hv, bounds):
    """The tcgen05 chunk kernels (forward and every gradient) against the token-by-token
    recurrence evaluated in fp32 on the CPU from the same bf16 inputs."""
    from shadowspill_b200.ops import _lib, delta_rule, reference as ref
    q, k, v, beta, gl, dout, cu = _delta_case(T, Hk, Hv, bounds, seed=T)
    cpu = [t.float().clone().requires_grad_(True) for t in (q, k, v, beta, gl)]
    want = ref.gated_delta_rule(*cpu, torch.tensor(bounds))
    want.backward(dout.float())
    dev = [t.clone().cuda().requires_grad_(True) for t in (q, k, v, beta, gl)]
    assert delta_rule.supported(dev[0], dev[1], dev[2])
    got = seq.gated_delta_rule_chunked(*dev, None, 64, cu_seqlens=cu.cuda())
    got.backward(dout.cuda())
    torch.cuda.synchronize()
    _lib.check_status()
    assert _rel(got.cpu(), want) < 1.5e-2                      # bf16 operands, fp32 accumulation
    for name, a, b in zip("q k v beta g".split(), dev, cpu):
        assert _rel(a.grad.cpu(), b.grad) < 3e-2, name


def test_delta_rule_kernels_at_the_model_head_counts():
    """16 QK heads, 32 V heads (the 9B configuration), against the PyTorch chunked form on the GPU."""
    from shadowspill_b200.ops import _lib
    T, bounds = 640, [0, 1, 250, 577, 640]
    q, k, v, beta, gl, dout, cu = _delta_case(T, 16, 32, bounds, seed=3)
    a = [t.clone().cuda().requires_grad_(True) for t in (q, k, v, beta, gl)]
    b = [t.clone().cuda().float().requires_grad_(True) for t in (q, k, v, beta, gl)]
    got = seq.gated_delta_rule_chunked(*a, None, 64, cu_seqlens=cu.cuda())
    want = seq._gated_delta_rule_torch(*b, None, 64, cu_seqlens=cu.cuda())
    got.backward(dout.cuda())
    want.backward(dout.cuda().float())
    torch.cuda.synchronize()
    _lib.check_status()
    assert _rel(got, want) < 1.5e-2
    for name, x, y in zip("q k v beta g".split(), a, b):
        assert _rel(x.grad, y.grad) < 3e-2, name


@pytest.mark.gpu
def test_head_groups_compute_the_same_rule_in_pieces():
    """Running the rule in groups of key heads (less intermediate memory) gives the same output
    and gradients as all heads at once."""
    from shadowspill_b200.ops import delta_rule as dr
    torch.manual_seed(3)
    dev = torch.device("cuda")
    T, Hk, H = 640, 4, 8
    q = torch.nn.functional.normalize(torch.randn(T, Hk, 128, device=dev), dim=-1).bfloat16()
    k = torch.nn.functional.normalize(torch.randn(T, Hk, 128, device=dev), dim=-1).bfloat16()
    v = (torch.randn(T, H, 128, device=dev) * 0.5).bfloat16()
    beta = torch.sigmoid(torch.randn(T, H, device=dev))
    g = -torch.rand(T, H, device=dev) * 0.2
    cu = torch.tensor([0, 201, 640] + [640] * 6, dtype=torch.int32, device=dev)
    dout = torch.randn(T, H, 128, device=dev).bfloat16()
    whole = dr.gated_delta_rule(q, k, v, beta, g, cu)
    grads = dr.backward(q, k, v, beta, g, cu, dout)
    dr.set_head_groups(2)
    try:
        pieces = dr.gated_delta_rule(q, k, v, beta, g, cu)
        grads2 = dr.backward(q, k, v, beta, g, cu, dout)
    finally:
        dr.set_head_groups(1)
    assert torch.equal(whole, pieces)
    for a, b in zip(grads, grads2):
        assert torch.equal(a, b)
