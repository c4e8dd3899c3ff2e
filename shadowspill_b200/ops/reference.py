"""Plain-PyTorch definitions of every model op.

These are the numerical oracles for the CUDA kernels and the execution path on
CPU. They restate the semantics of the reference's pure-PyTorch decoders
(packages/workloads/src/shadowspill_workloads/models/shared/decoder.py:18-330 and
models/qwen35/implementations/pytorch/delta_rule/reference.py:8-132) and run in
fp32 internally, casting at the same points the kernels do.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F


def gemm(a: torch.Tensor, b: torch.Tensor, *, a_mn: bool, b_mn: bool, out: torch.Tensor | None,
         accumulate: bool, alpha: float, out_dtype: torch.dtype) -> torch.Tensor:
    am = a.float().t() if a_mn else a.float()          # [M, K]
    bm = b.float() if b_mn else b.float().t()          # [K, N]
    res = (am @ bm) * alpha
    if out is None:
        return res.to(out_dtype)
    if accumulate:
        res = res + out.float()
    out.copy_(res.to(out.dtype))
    return out


def rmsnorm_fwd(x, w, eps, zero_centered=False, delta=None):
    """Returns (y, rstd); folds ``delta`` into ``x`` in place first when given."""
    if delta is not None:
        x.copy_((x.float() + delta.float()).to(x.dtype))
    xf = x.float()
    rstd = torch.rsqrt(xf.square().mean(dim=-1) + eps)
    scale = (1.0 + w.float()) if zero_centered else w.float()
    y = (xf * rstd[:, None] * scale).to(x.dtype)
    return y, rstd


def rmsnorm_bwd(x, w, gy, rstd, zero_centered=False):
    """Returns (dx fp32, dw fp32)."""
    xf, gf = x.float(), gy.float()
    scale = (1.0 + w.float()) if zero_centered else w.float()
    xh = xf * rstd[:, None]
    gw = gf * scale
    mean = (gw * xh).mean(dim=-1, keepdim=True)
    dx = rstd[:, None] * (gw - xh * mean)
    dw = (gf * xh).sum(dim=0)
    return dx, dw


def rope_(buf, positions, col0, heads, dh, rot, theta, inverse=False):
    """In-place half-split rotary on columns [col0, col0 + heads*dh) of ``buf`` [T, C]."""
    T = buf.shape[0]
    half = rot // 2
    inv = theta ** (-torch.arange(0, half, dtype=torch.float32, device=buf.device) * 2.0 / rot)
    ang = positions.float()[:, None] * inv[None, :]
    cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]
    if inverse:
        sin = -sin
    view = buf[:, col0:col0 + heads * dh].reshape(T, heads, dh)
    a = view[..., :half].float()
    b = view[..., half:rot].float()
    oa = a * cos - b * sin
    ob = b * cos + a * sin
    view = view.clone()
    view[..., :half] = oa.to(buf.dtype)
    view[..., half:rot] = ob.to(buf.dtype)
    buf[:, col0:col0 + heads * dh] = view.reshape(T, heads * dh)
    return buf


def swiglu_fwd(gu):
    F_ = gu.shape[-1] // 2
    g, u = gu[..., :F_], gu[..., F_:]
    return (F.silu(g.float()).to(gu.dtype).float() * u.float()).to(gu.dtype)


def swiglu_bwd(gu, dh):
    F_ = gu.shape[-1] // 2
    g, u, d = gu[..., :F_].float(), gu[..., F_:].float(), dh.float()
    sig = torch.sigmoid(g)
    dg = d * u * (sig * (1 + g * (1 - sig)))
    du = d * g * sig
    return torch.cat([dg, du], dim=-1).to(gu.dtype)


def embedding_fwd(ids, W):
    return W[ids.clamp(0, W.shape[0] - 1)]


def embedding_bwd(ids, g, dW):
    dW.index_add_(0, ids, g.to(dW.dtype))
    return dW


def cross_entropy_(logits, targets, weights, grad_scale=1.0, write_grad=True):
    """Weighted-sum cross entropy over a logits block; rewrites ``logits`` with
    its gradient when asked. Returns (loss_sum fp32 scalar, lse fp32[R])."""
    lf = logits.float()
    lse = torch.logsumexp(lf, dim=-1)
    V = logits.shape[-1]
    valid = (targets >= 0) & (targets < V)
    w = torch.ones_like(lse) if weights is None else weights.float()
    w = torch.where(valid, w, torch.zeros_like(w))
    tgt = targets.clamp(0, V - 1)
    picked = lf.gather(1, tgt[:, None])[:, 0]
    loss = (w * (lse - picked)).sum()
    if write_grad:
        p = torch.exp(lf - lse[:, None])
        p.scatter_add_(1, tgt[:, None], -torch.ones_like(picked)[:, None])
        logits.copy_((p * (w * grad_scale)[:, None]).to(logits.dtype))
    return loss, lse


def clipped_policy_(logits, targets, weights, old_logp, advantage, clip, ref_logp=None,
                    ref_beta=0.0, grad_scale=1.0, write_grad=True):
    """Weighted-sum clipped policy objective over a logits block (autograd-derived
    gradient written in place). Returns (loss_sum, logp[R])."""
    lf = logits.float().detach().requires_grad_(write_grad)
    V = logits.shape[-1]
    valid = (targets >= 0) & (targets < V)
    w = torch.ones(logits.shape[0], device=logits.device) if weights is None else weights.float()
    w = torch.where(valid, w, torch.zeros_like(w))
    tgt = targets.clamp(0, V - 1)
    logp = lf.gather(1, tgt[:, None])[:, 0] - torch.logsumexp(lf, dim=-1)
    r = torch.exp(logp - old_logp.float())
    A = advantage.float()
    per = -torch.minimum(r * A, r.clamp(1 - clip, 1 + clip) * A)
    if ref_logp is not None:
        d = ref_logp.float() - logp
        per = per + ref_beta * (torch.exp(d) - d - 1)
    loss = (w * per).sum()
    if write_grad:
        (g,) = torch.autograd.grad(loss * grad_scale, lf)
        logits.copy_(g.to(logits.dtype))
    return loss.detach(), logp.detach()


def adamw_(p, g, m, v, *, lr, beta1, beta2, eps, weight_decay, step, grad_scale=1.0):
    """Round-to-nearest AdamW in fp32 math on tensors of any dtype (in place)."""
    gf = g.float() * grad_scale
    mf = beta1 * m.float() + (1 - beta1) * gf
    vf = beta2 * v.float() + (1 - beta2) * gf * gf
    b1 = 1 - beta1 ** step
    b2 = 1 - beta2 ** step
    pf = p.float() * (1 - lr * weight_decay)
    pf = pf - lr * (mf / b1) / ((vf / b2).sqrt() + eps)
    p.copy_(pf.to(p.dtype)); m.copy_(mf.to(m.dtype)); v.copy_(vf.to(v.dtype))


RULES = ("adamw", "sgd", "lion")


def update_rule_(rule, p, g, m, v, *, lr, beta1, beta2, eps, weight_decay, step, grad_scale=1.0):
    """The update rules other than AdamW, in fp32 math with round-to-nearest stores, on tensors of
    any dtype and device (plain tensor operations: these are not hot paths).

    ``sgd``: momentum ``m <- beta1 m + g``, ``p <- p - lr (m + wd p)`` (``torch.optim.SGD`` with
    momentum ``beta1``, no dampening; the decay is added to the step, not to the gradient).
    ``lion``: ``u = sign(beta1 m + (1 - beta1) g)``, ``p <- p - lr (u + wd p)``,
    ``m <- beta2 m + (1 - beta2) g`` (Chen et al. 2023). ``v`` is not used by either."""
    if hasattr(rule, "apply"):
        # the update of a torch.optim optimizer captured as a graph (frontend/optimizer_capture.py);
        # its own hyperparameters are constants of that graph, the learning rate follows the run
        return rule.apply(p, g, m, v, lr=lr, step=step, grad_scale=grad_scale)
    if rule == "adamw":
        return adamw_(p, g, m, v, lr=lr, beta1=beta1, beta2=beta2, eps=eps, weight_decay=weight_decay,
                      step=step, grad_scale=grad_scale)
    gf = g.float() * grad_scale
    pf, mf = p.float(), m.float()
    if rule == "sgd":
        mf = beta1 * mf + gf
        pf = pf - lr * (mf + weight_decay * pf)
    elif rule == "lion":
        u = torch.sign(beta1 * mf + (1 - beta1) * gf)
        pf = pf - lr * (u + weight_decay * pf)
        mf = beta2 * mf + (1 - beta2) * gf
    else:
        raise ValueError(f"unknown update rule {rule!r}; known: {RULES}")
    p.copy_(pf.to(p.dtype)); m.copy_(mf.to(m.dtype))


def attention_varlen(q, k, v, cu_seqlens, scale=None):
    """Packed causal GQA: q [T,Hq,dh], k/v [T,Hkv,dh]; each [cu[i],cu[i+1]) is its
    own causal sequence. Returns (out [T,Hq,dh], lse fp32 [Hq,T])."""
    T, Hq, dh = q.shape
    Hkv = k.shape[1]
    rep = Hq // Hkv
    scale = scale if scale is not None else 1.0 / math.sqrt(dh)
    out = torch.zeros_like(q)
    lse = torch.full((Hq, T), float("-inf"), dtype=torch.float32, device=q.device)
    bounds = cu_seqlens.tolist()
    for s, e in zip(bounds[:-1], bounds[1:]):
        if e <= s:
            continue
        qs = q[s:e].float().transpose(0, 1)                               # [Hq, L, dh]
        ks = k[s:e].float().transpose(0, 1).repeat_interleave(rep, dim=0)
        vs = v[s:e].float().transpose(0, 1).repeat_interleave(rep, dim=0)
        sc = (qs @ ks.transpose(1, 2)) * scale
        L = e - s
        mask = torch.ones(L, L, dtype=torch.bool, device=q.device).tril()
        sc = sc.masked_fill(~mask, float("-inf"))
        lse[:, s:e] = torch.logsumexp(sc, dim=-1)
        out[s:e] = (torch.softmax(sc, dim=-1) @ vs).transpose(0, 1).to(q.dtype)
    return out, lse


def attention_varlen_bwd(q, k, v, out, lse, dout, cu_seqlens, scale=None):
    """Returns (dq, dk, dv) in the input dtypes."""
    T, Hq, dh = q.shape
    Hkv = k.shape[1]
    rep = Hq // Hkv
    scale = scale if scale is not None else 1.0 / math.sqrt(dh)
    dq = torch.zeros_like(q); dk = torch.zeros_like(k); dv = torch.zeros_like(v)
    bounds = cu_seqlens.tolist()
    for s, e in zip(bounds[:-1], bounds[1:]):
        if e <= s:
            continue
        L = e - s
        qs = q[s:e].float().transpose(0, 1)
        ks = k[s:e].float().transpose(0, 1).repeat_interleave(rep, dim=0)
        vs = v[s:e].float().transpose(0, 1).repeat_interleave(rep, dim=0)
        do = dout[s:e].float().transpose(0, 1)
        o = out[s:e].float().transpose(0, 1)
        sc = (qs @ ks.transpose(1, 2)) * scale
        mask = torch.ones(L, L, dtype=torch.bool, device=q.device).tril()
        sc = sc.masked_fill(~mask, float("-inf"))
        p = torch.exp(sc - lse[:, s:e, None])
        dvs = p.transpose(1, 2) @ do
        dp = do @ vs.transpose(1, 2)
        delta = (do * o).sum(-1, keepdim=True)
        ds = p * (dp - delta) * scale
        dqs = ds @ ks
        dks = ds.transpose(1, 2) @ qs
        dq[s:e] = dqs.transpose(0, 1).to(q.dtype)
        dk[s:e] = dks.reshape(Hkv, rep, L, dh).sum(1).transpose(0, 1).to(k.dtype)
        dv[s:e] = dvs.reshape(Hkv, rep, L, dh).sum(1).transpose(0, 1).to(v.dtype)
    return dq, dk, dv


def l2_normalize(x, eps=1e-6):
    xf = x.float()
    return (xf * torch.rsqrt(xf.square().sum(-1, keepdim=True) + eps)).to(x.dtype)


def gated_delta_rule(q, k, v, beta, g, cu_seqlens):
    """Token-by-token gated delta rule (the recurrence the chunked kernel must
    match). q,k [T,Hk,dk] (already L2-normalised), v [T,Hv,dv], beta,g [T,Hv];
    g is the log-decay (<= 0). QK heads are repeat-interleaved to V heads.
    Returns out [T,Hv,dv] in v.dtype."""
    T, Hk, dk = q.shape
    Hv, dv = v.shape[1], v.shape[2]
    rep = Hv // Hk
    qf = q.float().repeat_interleave(rep, dim=1) * dk ** -0.5
    kf = k.float().repeat_interleave(rep, dim=1)
    vf, bf, gf = v.float(), beta.float(), g.float()
    out = torch.zeros(T, Hv, dv, dtype=torch.float32, device=q.device)
    bounds = cu_seqlens.tolist()
    for s, e in zip(bounds[:-1], bounds[1:]):
        S = torch.zeros(Hv, dk, dv, dtype=torch.float32, device=q.device)
        for t in range(s, e):
            S = S * torch.exp(gf[t])[:, None, None]
            u = bf[t][:, None] * (vf[t] - torch.einsum("hk,hkv->hv", kf[t], S))
            S = S + kf[t][:, :, None] * u[:, None, :]
            out[t] = torch.einsum("hk,hkv->hv", qf[t], S)
    return out.to(v.dtype)


def causal_conv_silu(x, w, cu_seqlens):
    """Depthwise causal conv1d (kernel K) + SiLU over packed sequences.
    x [T,C], w [C,K]; the window never crosses a sequence boundary."""
    T, C = x.shape
    K = w.shape[1]
    out = torch.zeros_like(x)
    bounds = cu_seqlens.tolist()
    for s, e in zip(bounds[:-1], bounds[1:]):
        if e <= s:
            continue
        seg = x[s:e].float().t()[None]                       # [1, C, L]
        y = F.conv1d(F.pad(seg, (K - 1, 0)), w.float()[:, None, :], groups=C)[0].t()
        out[s:e] = F.silu(y).to(x.dtype)
    return out


def router_topk(logits, top_k, renormalize=True):
    """top-k then softmax over the selected logits (Qwen-MoE convention).
    Returns (weights fp32 [T,k], ids int64 [T,k], counts int64 [E])."""
    vals, ids = torch.topk(logits.float(), top_k, dim=-1)
    if renormalize:
        w = torch.softmax(vals, dim=-1)
    else:
        w = torch.softmax(logits.float(), dim=-1).gather(1, ids)
    counts = torch.bincount(ids.reshape(-1), minlength=logits.shape[-1])
    return w, ids, counts
