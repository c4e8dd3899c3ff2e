"""Sequence-mixer ops of the hybrid (Gated DeltaNet) layers, written as
differentiable PyTorch so that ``torch.autograd`` supplies their backward pass.

``gated_delta_rule_chunked`` evaluates the gated delta rule in chunks of 64 tokens
(the WY / UT-transform form): inside a chunk everything is dense matrix algebra,
and only the ``[dk, dv]`` state is carried from chunk to chunk. With
``a_t = exp(g_t)`` and ``G_t`` the running product of ``a`` inside the chunk,

    A[t,i] = beta_t (G_t/G_i) (k_t . k_i)  for i < t          (strictly lower)
    T      = (I + A)^-1
    U      = T (beta V) - T (beta G K) S_in                    (the "new values")
    O      = (G Q) S_in + tril((G_t/G_i) Q K^T) U
    S_out  = G_C S_in + ((G_C/G) K)^T U

which equals the token recurrence in :func:`..reference.gated_delta_rule`
(the reference's definition: packages/workloads/src/shadowspill_workloads/models/
qwen35/implementations/pytorch/delta_rule/reference.py:8-41). Sequences of a packed
batch are independent: the state starts at zero at every boundary.
"""
from __future__ import annotations

import torch
import torch.nn.functional as TF


def l2_normalize(x: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    xf = x.float()
    return (xf * torch.rsqrt(xf.square().sum(-1, keepdim=True) + eps)).to(x.dtype)


def causal_conv_silu(x: torch.Tensor, w: torch.Tensor, bounds: list[int]) -> torch.Tensor:
    """Depthwise causal conv1d (kernel ``w.shape[1]``) + SiLU; ``x`` [T,C], ``w`` [C,K].
    The window never crosses a sequence boundary (``bounds`` = cu_seqlens as a list)."""
    T, C = x.shape
    K = w.shape[1]
    xf = x.float()
    # shifted copies: y[t] = sum_j w[:, K-1-j] * x[t-j], with x[t-j] zero before the sequence start
    pos = torch.zeros(T, dtype=torch.long, device=x.device)
    for s, e in zip(bounds[:-1], bounds[1:]):
        if e > s:
            pos[s:e] = torch.arange(e - s, device=x.device)
    y = torch.zeros_like(xf)
    wf = w.float()
    for j in range(K):
        shifted = torch.roll(xf, shifts=j, dims=0) if j else xf
        valid = (pos >= j).to(xf.dtype)[:, None]
        y = y + shifted * valid * wf[:, K - 1 - j][None, :]
    return TF.silu(y).to(x.dtype)


def _chunk_sequence(q, k, v, beta, g, C):
    """One sequence, heads batched. q,k [L,H,dk] fp32 (q pre-scaled), v [L,H,dv], beta,g [L,H]."""
    L, H, dk = q.shape
    dv = v.shape[-1]
    n = -(-L // C)
    pad = n * C - L
    if pad:
        zp = lambda t: TF.pad(t, (0, 0) * (t.dim() - 1) + (0, pad))
        q, k, v, beta, g = zp(q), zp(k), zp(v), zp(beta), zp(g)
    # [n, H, C, ...]
    rs = lambda t: t.reshape(n, C, H, -1).permute(0, 2, 1, 3)
    q, k, v = rs(q), rs(k), rs(v)
    beta = beta.reshape(n, C, H).permute(0, 2, 1)
    gam = g.reshape(n, C, H).permute(0, 2, 1).cumsum(-1)            # log G_t
    ratio = torch.exp((gam[..., :, None] - gam[..., None, :]).clamp(max=0.0))   # G_t/G_i, i<=t
    lower = torch.ones(C, C, device=q.device, dtype=torch.bool).tril()
    strict = lower & ~torch.eye(C, device=q.device, dtype=torch.bool)
    kk = k @ k.transpose(-1, -2)
    A = (beta[..., :, None] * ratio * kk).masked_fill(~strict, 0.0)
    eye = torch.eye(C, device=q.device, dtype=q.dtype).expand(n, H, C, C)
    Tm = torch.linalg.solve_triangular(eye + A, eye, upper=False)
    Gt = torch.exp(gam)[..., None]                                   # G_t
    W = Tm @ (beta[..., None] * Gt * k)                              # [n,H,C,dk]
    U0 = Tm @ (beta[..., None] * v)                                  # [n,H,C,dv]
    M = (ratio * (q @ k.transpose(-1, -2))).masked_fill(~lower, 0.0)
    Qg = Gt * q
    Gc = torch.exp(gam[..., -1])[..., None, None]                    # G_C
    Kd = torch.exp(gam[..., -1:] - gam)[..., None] * k               # (G_C/G_i) k_i
    S = q.new_zeros(H, dk, dv)
    outs = []
    for c in range(n):
        U = U0[c] - W[c] @ S
        outs.append(Qg[c] @ S + M[c] @ U)
        S = Gc[c] * S + Kd[c].transpose(-1, -2) @ U
    out = torch.stack(outs, 0).permute(0, 2, 1, 3).reshape(n * C, H, dv)
    return out[:L]


def gated_delta_rule_chunked(q, k, v, beta, g, bounds: list[int], chunk: int = 64) -> torch.Tensor:
    """q,k [T,Hk,dk] (L2-normalised), v [T,Hv,dv], beta,g [T,Hv] (g = log decay <= 0).
    QK heads are repeat-interleaved to the V heads. Returns [T,Hv,dv] in ``v.dtype``."""
    Hk, dk = q.shape[1], q.shape[2]
    Hv = v.shape[1]
    rep = Hv // Hk
    qf = q.float().repeat_interleave(rep, dim=1) * dk ** -0.5
    kf = k.float().repeat_interleave(rep, dim=1)
    vf, bf, gf = v.float(), beta.float(), g.float()
    pieces = []
    for s, e in zip(bounds[:-1], bounds[1:]):
        if e > s:
            pieces.append(_chunk_sequence(qf[s:e], kf[s:e], vf[s:e], bf[s:e], gf[s:e], chunk))
    return torch.cat(pieces, 0).to(v.dtype)


def gated_rmsnorm(x: torch.Tensor, gate: torch.Tensor, w: torch.Tensor, eps: float,
                  zero_centered: bool = False) -> torch.Tensor:
    """RMSNorm over the last dimension followed by a SiLU gate (reference:
    models/shared/decoder.py GatedRMSNorm)."""
    xf = x.float()
    r = torch.rsqrt(xf.square().mean(-1, keepdim=True) + eps)
    scale = (1.0 + w.float()) if zero_centered else w.float()
    return (xf * r * scale * TF.silu(gate.float())).to(x.dtype)
