"""Autograd twin of the dense decoder: the same parameters, plain PyTorch ops,
gradients by ``torch.autograd``. It is the independent oracle for the
hand-written stage backward passes (the role the reference gives its
pure-PyTorch implementations, e.g.
packages/workloads/src/shadowspill_workloads/models/llama3/implementations/pytorch.py).
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as TF

from .config import DecoderConfig
from .decoder import BatchMeta


def _rms(x, w, eps, zero_centered):
    xf = x.float()
    r = torch.rsqrt(xf.square().mean(-1, keepdim=True) + eps)
    scale = (1 + w.float()) if zero_centered else w.float()
    return (xf * r * scale).to(x.dtype)


def _rope(x, positions, rot, theta):
    # x [T, H, dh]
    half = rot // 2
    inv = theta ** (-torch.arange(0, half, dtype=torch.float32, device=x.device) * 2.0 / rot)
    ang = positions.float()[:, None] * inv[None]
    cos, sin = ang.cos()[:, None], ang.sin()[:, None]
    a, b, rest = x[..., :half].float(), x[..., half:rot].float(), x[..., rot:]
    return torch.cat([(a * cos - b * sin).to(x.dtype), (b * cos + a * sin).to(x.dtype), rest], -1)


def _attention(q, k, v, cu):
    T, Hq, dh = q.shape
    rep = Hq // k.shape[1]
    outs = []
    b = cu.tolist()
    for s, e in zip(b[:-1], b[1:]):
        if e <= s:
            continue
        qs = q[s:e].transpose(0, 1)[None]
        ks = k[s:e].transpose(0, 1).repeat_interleave(rep, 0)[None]
        vs = v[s:e].transpose(0, 1).repeat_interleave(rep, 0)[None]
        o = TF.scaled_dot_product_attention(qs.float(), ks.float(), vs.float(), is_causal=True)
        outs.append(o[0].transpose(0, 1).to(q.dtype))
    return torch.cat(outs, 0)


def dense_layer(cfg: DecoderConfig, P: dict, x, meta: BatchMeta):
    T = x.shape[0]
    dh, Hq, Hkv = cfg.head_dim, cfg.n_heads, cfg.n_kv_heads
    h = _rms(x, P["attn_norm"], cfg.norm_epsilon, cfg.zero_centered_norm)
    qkv = h @ P["wqkv"].t()
    q = qkv[:, :Hq * dh].reshape(T, Hq, dh)
    k = qkv[:, Hq * dh:(Hq + Hkv) * dh].reshape(T, Hkv, dh)
    v = qkv[:, (Hq + Hkv) * dh:].reshape(T, Hkv, dh)
    if cfg.qk_norm:
        q = _rms(q, P["q_norm"], cfg.norm_epsilon, cfg.zero_centered_norm)
        k = _rms(k, P["k_norm"], cfg.norm_epsilon, cfg.zero_centered_norm)
    q = _rope(q, meta.positions, cfg.rotary_width, cfg.rope_base)
    k = _rope(k, meta.positions, cfg.rotary_width, cfg.rope_base)
    a = _attention(q, k, v, meta.cu_seqlens).reshape(T, Hq * dh)
    x = x + a @ P["wo"].t()
    h = _rms(x, P["mlp_norm"], cfg.norm_epsilon, cfg.zero_centered_norm)
    gu = h @ P["w13"].t()
    F_ = cfg.d_ff
    hm = TF.silu(gu[:, :F_].float()).to(x.dtype) * gu[:, F_:]
    return x + hm @ P["w2"].t()


def loss(cfg: DecoderConfig, params: dict[str, torch.Tensor], meta: BatchMeta) -> torch.Tensor:
    """Weighted-sum next-token loss of the dense decoder; ``params`` maps
    ``"<stage>.<param>"`` to tensors (possibly requiring grad)."""
    def stage(name):
        pre = name + "."
        return {k[len(pre):]: v for k, v in params.items() if k.startswith(pre)}
    x = stage("embed")["embed"][meta.tokens]
    for i in range(cfg.n_layers):
        x = dense_layer(cfg, stage(f"layer{i}"), x, meta)
    hp = stage("head")
    h = _rms(x, hp["final_norm"], cfg.norm_epsilon, cfg.zero_centered_norm)
    out_w = stage("embed")["embed"] if cfg.tied_embeddings else hp["head"]
    logits = (h @ out_w.t()).float()
    lse = torch.logsumexp(logits, -1)
    tgt = meta.targets.clamp(min=0)
    picked = logits.gather(1, tgt[:, None])[:, 0]
    w = torch.where(meta.targets >= 0, meta.weights.float(), torch.zeros_like(lse))
    return (w * (lse - picked)).sum()


# ---------------------------------------------------------------------------- hybrid / mixture
def hybrid_layer(cfg: DecoderConfig, P: dict, x, meta: BatchMeta, index: int):
    """Plain-PyTorch twin of ``HybridLayerStage``: same math, ordinary autograd."""
    from ..ops import sequence as seq
    T = x.shape[0]
    dh, Hq, Hkv = cfg.head_dim, cfg.n_heads, cfg.n_kv_heads
    h = _rms(x, P["attn_norm"], cfg.norm_epsilon, cfg.zero_centered_norm)
    if cfg.layer_kind(index) == "attention":
        qg = h @ P["wq"].t()
        q, gate = (qg[:, :Hq * dh], qg[:, Hq * dh:]) if cfg.gated_attention else (qg, None)
        k = h @ P["wk"].t()
        if cfg.qk_norm and cfg.qk_norm_full_width:
            q = _rms(q, P["q_norm"], cfg.norm_epsilon, cfg.zero_centered_norm)
            k = _rms(k, P["k_norm"], cfg.norm_epsilon, cfg.zero_centered_norm)
        q = q.reshape(T, Hq, dh)
        k = k.reshape(T, Hkv, dh)
        v = (h @ P["wv"].t()).reshape(T, Hkv, dh)
        if cfg.qk_norm and not cfg.qk_norm_full_width:
            q = _rms(q, P["q_norm"], cfg.norm_epsilon, cfg.zero_centered_norm)
            k = _rms(k, P["k_norm"], cfg.norm_epsilon, cfg.zero_centered_norm)
        q = _rope(q, meta.positions, cfg.rotary_width, cfg.rope_base)
        k = _rope(k, meta.positions, cfg.rotary_width, cfg.rope_base)
        a = _attention(q, k, v, meta.cu_seqlens).reshape(T, Hq * dh)
        if gate is not None:
            a = a * torch.sigmoid(gate.float()).to(a.dtype)
        mix = a @ P["wo"].t()
    else:
        Hk, Hv, dk = cfg.dn_qk_heads, cfg.dn_v_heads, cfg.dn_head_dim
        kw, vw = Hk * dk, Hv * dk
        cw = 2 * kw + vw
        bounds = meta.cu_seqlens.tolist()
        qkvz = h @ P["w_qkvz"].t()
        ba = h @ P["w_ba"].t()
        conv = seq.causal_conv_silu(qkvz[:, :cw], P["conv_w"], bounds)
        q = seq.l2_normalize(conv[:, :kw].reshape(T, Hk, dk))
        k = seq.l2_normalize(conv[:, kw:2 * kw].reshape(T, Hk, dk))
        v = conv[:, 2 * kw:].reshape(T, Hv, dk)
        beta = torch.sigmoid(ba[:, :Hv].float())
        g = -torch.exp(P["A_log"].float()) * TF.softplus(ba[:, Hv:].float() + P["dt_bias"].float())
        mixed = seq.gated_delta_rule_chunked(q, k, v, beta, g, bounds, cfg.dn_chunk)
        normed = seq.gated_rmsnorm(mixed, qkvz[:, cw:].reshape(T, Hv, dk), P["lin_norm"],
                                   cfg.norm_epsilon, cfg.zero_centered_norm)
        mix = normed.reshape(T, vw) @ P["w_out"].t()
    x = x + mix
    h = _rms(x, P["mlp_norm"], cfg.norm_epsilon, cfg.zero_centered_norm)

    def mlp(inp, w13, w2):
        gu = inp @ w13.t()
        F_ = gu.shape[-1] // 2
        return (TF.silu(gu[:, :F_].float()).to(inp.dtype) * gu[:, F_:]) @ w2.t()

    if cfg.is_moe:
        logits = (h @ P["router"].t()).float()
        if cfg.router_renormalize:
            vals, ids = torch.topk(logits, cfg.top_k, dim=-1)
            wts = torch.softmax(vals, -1)
        else:
            wts, ids = torch.topk(torch.softmax(logits, -1), cfg.top_k, dim=-1)
        ff = torch.zeros_like(h)
        for e in range(cfg.n_experts):          # dense reference: every expert sees its tokens
            sel = (ids == e)
            rows = sel.any(-1).nonzero()[:, 0]
            if rows.numel() == 0:
                continue
            w = (wts * sel).sum(-1)[rows].to(h.dtype)
            ff = ff.index_add(0, rows, mlp(h[rows], P["w13"][e], P["w2"][e]) * w[:, None])
        if cfg.d_shared_expert:
            sh = mlp(h, P["sw13"], P["sw2"])
            if cfg.gated_shared_expert:
                sh = sh * torch.sigmoid(h.float() @ P["shared_gate"].float()).to(h.dtype)[:, None]
            ff = ff + sh
    else:
        ff = mlp(h, P["w13"], P["w2"])
    return x + ff


def model_loss(cfg: DecoderConfig, params: dict[str, torch.Tensor], meta: BatchMeta,
               stages=None) -> torch.Tensor:
    """Weighted-sum loss of any catalog family (dense layers use ``dense_layer``).
    ``stages`` overrides the stage list whose layer classes pick the layer form."""
    from .decoder import DenseLayerStage, build_stages

    def stage(name):
        pre = name + "."
        return {k[len(pre):]: v for k, v in params.items() if k.startswith(pre)}
    stages = stages or build_stages(cfg)
    x = stage("embed")["embed"][meta.tokens]
    for i in range(cfg.n_layers):
        P = stage(f"layer{i}")
        x = dense_layer(cfg, P, x, meta) if isinstance(stages[i + 1], DenseLayerStage) \
            else hybrid_layer(cfg, P, x, meta, i)
    hp = stage("head")
    h = _rms(x, hp["final_norm"], cfg.norm_epsilon, cfg.zero_centered_norm)
    out_w = stage("embed")["embed"] if cfg.tied_embeddings else hp["head"]
    logits = (h @ out_w.t()).float()
    lse = torch.logsumexp(logits, -1)
    tgt = meta.targets.clamp(min=0)
    picked = logits.gather(1, tgt[:, None])[:, 0]
    w = torch.where(meta.targets >= 0, meta.weights.float(), torch.zeros_like(lse))
    return (w * (lse - picked)).sum()
