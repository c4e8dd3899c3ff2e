"""sm_100a kernels against plain-PyTorch fp32 references of the same op."""
import pytest
import torch

from shadowspill_b200.ops import _lib, functional as F, reference as R

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _rand(*shape, scale=1.0, dtype=torch.bfloat16):
    return (torch.randn(*shape, device=DEV, dtype=torch.float32) * scale).to(dtype)


def _rel(a, b):
    return float((a.float() - b.float()).norm() / (b.float().norm() + 1e-12))


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, True), (True, False)])
@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (256, 512, 256), (1000, 520, 328),
                                   (4096, 4096, 1024), (64, 136, 72)])
def test_gemm_layouts(a_mn, b_mn, M, N, K):
    a = _rand(K, M) if a_mn else _rand(M, K)
    b = _rand(K, N) if b_mn else _rand(N, K)
    out = F.gemm(a, b, a_mn=a_mn, b_mn=b_mn)
    _lib.check_status()
    am = a.float().t() if a_mn else a.float()
    bm = b.float() if b_mn else b.float().t()
    ref = am @ bm
    assert _rel(out, ref) < 5e-3


@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
def test_gemm_accumulate_and_dtype(out_dtype):
    M, N, K = 512, 384, 640
    a, b = _rand(M, K), _rand(N, K)
    c0 = _rand(M, N, dtype=out_dtype)
    c = c0.clone()
    F.gemm(a, b, out=c, accumulate=True, alpha=0.5)
    _lib.check_status()
    ref = c0.float() + 0.5 * (a.float() @ b.float().t())
    assert _rel(c, ref) < 5e-3
    # strided output view (column slice of a wider buffer)
    wide = torch.zeros(M, N + 64, device=DEV, dtype=out_dtype)
    F.gemm(a, b, out=wide[:, :N])
    assert _rel(wide[:, :N], a.float() @ b.float().t()) < 5e-3
    assert float(wide[:, N:].abs().max()) == 0.0


def test_gemm_bn128_and_large_k():
    a, b = _rand(384, 8192, scale=0.1), _rand(128, 8192, scale=0.1)
    out = F.gemm(a, b, bn=128, out_dtype=torch.float32)
    _lib.check_status()
    assert _rel(out, a.float() @ b.float().t()) < 2e-3


@pytest.mark.parametrize("D", [128, 4096, 2048 + 8])
@pytest.mark.parametrize("zc", [False, True])
def test_rmsnorm(D, zc):
    T = 333
    x, w, d = _rand(T, D), _rand(D, scale=0.2), _rand(T, D)
    x_ref = x.clone()
    y_ref, r_ref = R.rmsnorm_fwd(x_ref, w, 1e-5, zc, d)
    x2 = x.clone()
    y, r = F.rmsnorm_fwd(x2, w, 1e-5, zc, delta=d)
    assert torch.equal(x2, x_ref)
    assert _rel(y, y_ref) < 4e-3 and _rel(r, r_ref) < 1e-4
    gy = _rand(T, D)
    dx_ref, dw_ref = R.rmsnorm_bwd(x_ref, w, gy, r_ref, zc)
    dw = torch.zeros(D, device=DEV, dtype=torch.float32)
    dx = F.rmsnorm_bwd(x2, w, gy, r, dw, zc)
    assert _rel(dx, dx_ref) < 4e-3 and _rel(dw, dw_ref) < 1e-3
    base = _rand(T, D)
    acc = base.clone()
    F.rmsnorm_bwd(x2, w, gy, r, None, zc, dx=acc, accumulate=True)
    assert _rel(acc, base.float() + dx_ref) < 4e-3


@pytest.mark.parametrize("rot", [128, 32])
def test_rope_roundtrip_and_reference(rot):
    T, H, dh = 257, 6, 128
    buf = _rand(T, 64 + H * dh)
    pos = torch.randint(0, 8000, (T,), device=DEV, dtype=torch.int32)
    ref = R.rope_(buf.clone().cpu(), pos.cpu(), 64, H, dh, rot, 5e5).to(DEV)
    got = F.rope_(buf.clone(), pos, col0=64, heads=H, dh=dh, rot=rot, theta=5e5)
    assert _rel(got, ref) < 4e-3
    back = F.rope_(got.clone(), pos, col0=64, heads=H, dh=dh, rot=rot, theta=5e5, inverse=True)
    assert _rel(back, buf) < 8e-3
    assert torch.equal(got[:, :64], buf[:, :64])


def test_swiglu():
    T, Fw = 300, 1032
    gu, dh = _rand(T, 2 * Fw), _rand(T, Fw)
    assert _rel(F.swiglu_fwd(gu), R.swiglu_fwd(gu)) < 4e-3
    assert _rel(F.swiglu_bwd(gu, dh), R.swiglu_bwd(gu, dh)) < 4e-3


def test_embedding():
    V, D, T = 1000, 256, 777
    W = _rand(V, D)
    ids = torch.randint(0, V, (T,), device=DEV)
    assert torch.equal(F.embedding_fwd(ids, W), W[ids])
    g = _rand(T, D)
    for dt, tol in ((torch.float32, 1e-5), (torch.bfloat16, 2e-2)):
        dW = torch.zeros(V, D, device=DEV, dtype=dt)
        F.embedding_bwd(ids, g, dW)
        ref = torch.zeros(V, D, device=DEV).index_add_(0, ids, g.float())
        assert _rel(dW, ref) < tol


@pytest.mark.parametrize("V", [4096, 128256, 1003 * 8])
def test_cross_entropy_block(V):
    Rr = 64
    logits = _rand(Rr, V, scale=2.0)
    tgt = torch.randint(0, V, (Rr,), device=DEV)
    tgt[::7] = -1
    w = torch.rand(Rr, device=DEV)
    ref_logits = logits.clone()
    loss_ref, lse_ref = R.cross_entropy_(ref_logits, tgt, w, 0.5, True)
    loss = torch.zeros(1, device=DEV)
    lse = torch.empty(Rr, device=DEV)
    F.cross_entropy_(logits, tgt, w, loss, grad_scale=0.5, lse=lse)
    assert abs(float(loss) - float(loss_ref)) < 2e-3 * abs(float(loss_ref))
    assert _rel(lse, lse_ref) < 1e-5
    assert _rel(logits, ref_logits) < 1e-2
    assert float(logits[::7].abs().max()) == 0.0


def test_adamw_nearest_matches_reference():
    n = 100003
    p, g = _rand(n), _rand(n, scale=0.1)
    m, v = _rand(n, scale=0.01), _rand(n, scale=0.001).abs()
    pr, mr, vr = p.clone(), m.clone(), v.clone()
    kw = dict(lr=1e-2, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1, step=3)
    R.adamw_(pr, g, mr, vr, **kw)
    F.adamw_(p, g, m, v, stochastic_param=False, stochastic_state=False, **kw)
    for a, b in ((p, pr), (m, mr), (v, vr)):
        # identical up to one bf16 ulp on a handful of elements (fp32 op order)
        assert _rel(a, b) < 2e-3


def test_adamw_stochastic_rounding_is_unbiased_and_shard_invariant():
    n = 1 << 16
    p0 = torch.full((n,), 1.0, device=DEV, dtype=torch.bfloat16)
    g = torch.full((n,), 1.0, device=DEV, dtype=torch.bfloat16)
    kw = dict(lr=1e-4, beta1=0.0, beta2=0.0, eps=1e-8, weight_decay=0.0, step=1, seed=7)
    p = p0.clone(); m = torch.zeros_like(p); v = torch.zeros_like(p)
    F.adamw_(p, g, m, v, **kw)
    # exact update 1 - 1e-4 is not representable in bf16 (ulp 2^-8 below 1): SR must
    # hit it on average, nearest rounding would stay at 1.0
    assert abs(float(p.float().mean()) - (1 - 1e-4)) < 2e-5
    assert p.unique().numel() == 2
    # same bits when the range is updated as two shards with global offsets
    q = p0.clone(); m2 = torch.zeros_like(q); v2 = torch.zeros_like(q)
    h = n // 2
    F.adamw_(q[:h], g[:h], m2[:h], v2[:h], offset=0, **kw)
    F.adamw_(q[h:], g[h:], m2[h:], v2[h:], offset=h, **kw)
    assert torch.equal(p, q)


def test_sumsq():
    x = _rand(1 << 20)
    partials = torch.empty(256, device=DEV)
    out = torch.zeros(1, device=DEV)
    F.sumsq(x, partials, out)
    assert abs(float(out) - float(x.float().square().sum())) < 1e-3 * float(out)
