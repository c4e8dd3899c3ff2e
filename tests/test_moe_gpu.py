"""Mixture-of-experts kernels (router, layout, grouped tcgen05 GEMMs, combine) on a B200."""
import pytest
import torch
import torch.nn.functional as TF

from shadowspill_b200.models.autograd_ops import GradSink
from shadowspill_b200.ops import _lib, moe

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _rel(a, b):
    return float((a.float() - b.float()).norm() / (b.float().norm() + 1e-12))


@pytest.mark.parametrize("renorm", [True, False])
@pytest.mark.parametrize("T,E,k", [(1000, 8, 2), (777, 128, 8), (64, 256, 8)])
def test_route_matches_topk(T, E, k, renorm):
    logits = torch.randn(T, E, device=DEV)
    ids, wts, counts = moe.route(logits, k, renorm)
    if renorm:
        v, i = torch.topk(logits, k, dim=-1)
        w = torch.softmax(v, -1)
    else:
        w, i = torch.topk(torch.softmax(logits, -1), k, dim=-1)
    assert torch.equal(ids.long(), i)
    assert float((wts - w).abs().max()) < 1e-5
    assert torch.equal(counts.long(), torch.bincount(i.reshape(-1), minlength=E))


def _reference(h, logits, w13, w2, k, renorm):
    T, D = h.shape
    E = w13.shape[0]
    if renorm:
        v, ids = torch.topk(logits, k, dim=-1)
        w = torch.softmax(v, -1)
    else:
        w, ids = torch.topk(torch.softmax(logits, -1), k, dim=-1)
    out = torch.zeros(T, D, device=h.device, dtype=torch.float32)
    for e in range(E):
        sel = ids == e
        rows = sel.any(-1).nonzero()[:, 0]
        if rows.numel() == 0:
            continue
        gu = h[rows].float() @ w13[e].float().t()
        F_ = gu.shape[1] // 2
        hm = (TF.silu(gu[:, :F_]).to(torch.bfloat16).float() * gu[:, F_:]).to(torch.bfloat16).float()
        out = out.index_add(0, rows, (hm @ w2[e].float().t()) * (w * sel).sum(-1)[rows, None])
    return out


@pytest.mark.parametrize("T,D,Fe,E,k", [(512, 256, 128, 8, 2), (1500, 512, 256, 16, 4)])
def test_experts_forward_backward(T, D, Fe, E, k):
    torch.manual_seed(0)
    h = (torch.randn(T, D, device=DEV) * 0.5).to(torch.bfloat16)
    logits = torch.randn(T, E, device=DEV)
    logits[:, E - 1] = -50.0                        # one expert receives no tokens
    w13 = (torch.randn(E, 2 * Fe, D, device=DEV) * 0.05).to(torch.bfloat16)
    w2 = (torch.randn(E, D, Fe, device=DEV) * 0.05).to(torch.bfloat16)
    G = {"w13": torch.full_like(w13, 7.0), "w2": torch.full_like(w2, 7.0)}
    hq, lq = h.clone().requires_grad_(True), logits.clone().requires_grad_(True)
    out = moe.experts(hq, lq, w13, w2, k, True, GradSink(G, first=True))
    dout = (torch.randn(T, D, device=DEV) * 0.1).to(torch.bfloat16)
    out.backward(dout)
    _lib.check_status()
    hr, lr = h.float().requires_grad_(True), logits.clone().requires_grad_(True)
    w13r, w2r = w13.float().requires_grad_(True), w2.float().requires_grad_(True)
    ref = _reference(hr, lr, w13r, w2r, k, True)
    ref.backward(dout.float())
    assert _rel(out, ref) < 2e-2
    assert _rel(hq.grad, hr.grad) < 3e-2
    assert _rel(lq.grad, lr.grad) < 5e-2
    assert _rel(G["w13"], w13r.grad) < 3e-2 and _rel(G["w2"], w2r.grad) < 3e-2
    assert float(G["w13"][E - 1].abs().max()) == 0.0      # the idle expert's gradient is zero
    # a second contribution accumulates
    out2 = moe.experts(h.clone().requires_grad_(True), logits, w13, w2, k, True, GradSink(G, first=False))
    out2.backward(dout)
    assert _rel(G["w2"], 2 * w2r.grad) < 3e-2
