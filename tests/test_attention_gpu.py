"""tcgen05 packed causal attention against the fp32 PyTorch definition."""
import pytest
import torch

from shadowspill_b200.ops import _lib, attention, reference as R

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _case(T, lens, Hq, Hkv, dh, seed=0):
    g = torch.Generator(device="cpu").manual_seed(seed)
    q = (torch.randn(T, Hq, dh, generator=g) * 0.8).to(torch.bfloat16).to(DEV)
    k = (torch.randn(T, Hkv, dh, generator=g) * 0.8).to(torch.bfloat16).to(DEV)
    v = (torch.randn(T, Hkv, dh, generator=g)).to(torch.bfloat16).to(DEV)
    cu = [0]
    for n in lens:
        cu.append(cu[-1] + n)
    while cu[-1] < T:
        cu.append(T)
    cu += [T, T]   # empty slots are allowed
    return q, k, v, torch.tensor(cu, dtype=torch.int32, device=DEV)


def _rel(a, b):
    return float((a.float() - b.float()).norm() / (b.float().norm() + 1e-12))


CASES = [
    (256, [256], 2, 1, 128),
    (640, [100, 37, 300, 131], 4, 2, 128),
    (1024, [1, 2, 513, 380], 8, 2, 128),
    (2048, [2048], 4, 4, 128),
    (384, [200, 184], 4, 1, 256),
    (1024, [700, 324], 2, 2, 256),
    (512, [130, 382], 4, 2, 64),
]


@pytest.mark.parametrize("T,lens,Hq,Hkv,dh", CASES)
def test_forward(T, lens, Hq, Hkv, dh, monkeypatch):
    monkeypatch.setenv("SS_ATTENTION", "native")
    q, k, v, cu = _case(T, lens, Hq, Hkv, dh)
    out, lse = attention.forward(q, k, v, cu, max(lens))
    _lib.check_status()
    ref, lse_ref = R.attention_varlen(q, k, v, cu)
    assert _rel(out, ref) < 1e-2
    valid = torch.isfinite(lse_ref)
    assert float((lse[valid] - lse_ref[valid]).abs().max()) < 2e-2


@pytest.mark.parametrize("T,lens,Hq,Hkv,dh", CASES)
def test_backward(T, lens, Hq, Hkv, dh, monkeypatch):
    monkeypatch.setenv("SS_ATTENTION", "native")
    q, k, v, cu = _case(T, lens, Hq, Hkv, dh, seed=1)
    out, lse = attention.forward(q, k, v, cu, max(lens))
    dout = (torch.randn(T, Hq, dh, device=DEV) * 0.5).to(torch.bfloat16)
    dq, dk, dv = attention.backward(q, k, v, out, lse, dout, cu, max(lens))
    _lib.check_status()
    out_ref, lse_ref = R.attention_varlen(q, k, v, cu)
    dq_r, dk_r, dv_r = R.attention_varlen_bwd(q, k, v, out_ref, lse_ref, dout, cu)
    assert _rel(dq, dq_r) < 2e-2
    assert _rel(dk, dk_r) < 2e-2
    assert _rel(dv, dv_r) < 2e-2
