"""Model families as plain ``nn.Module`` trees over the ``ss`` operators.

These are what the graph frontend exports: a ``DecoderLM`` is an embedding, a
``ModuleList`` of layers (the repeated child that the partitioner turns into stages)
and a head that returns the weighted-sum loss. Parameter names and shapes are those
of the stage classes in :mod:`shadowspill_b200.models` (``wqkv``, ``w13``, ...), so a
state dict, a checkpoint or a Hugging Face conversion fits either form.

Reference models: packages/workloads/src/shadowspill_workloads/models/llama3/
implementations/mlops.py:29-161 (dense), models/shared/delta_net.py:13-89 (Gated
DeltaNet), models/qwen35/implementations/mlops.py:30-100 (gated attention).
"""
from __future__ import annotations

import torch
from torch import nn

from ..models.config import DecoderConfig
from . import ops as _ops  # noqa: F401  (registers torch.ops.ss)

S = torch.ops.ss


def _param(shape, init: str = "normal", std: float = 0.02, dtype=None, trainable: bool = True) -> nn.Parameter:
    p = nn.Parameter(torch.empty(shape, dtype=dtype), requires_grad=trainable)
    p.ss_init, p.ss_std = init, std
    return p


class Embedding(nn.Module):
    def __init__(self, cfg: DecoderConfig, dtype, trainable: bool = True):
        super().__init__()
        self.embed = _param((cfg.vocab_size, cfg.d_model), std=cfg.initializer_range, dtype=dtype,
                            trainable=trainable)

    def forward(self, tokens):
        return S.embedding(tokens, self.embed)


class _Norms:
    """Shared helpers of the layer modules."""
    lora = None
    adapted: frozenset = frozenset()

    def _norm(self, x, w):
        c = self.cfg
        return S.rmsnorm(x, w, c.norm_epsilon, c.zero_centered_norm)[0]

    def _lin(self, x, name: str):
        """``x W^T``, plus ``(alpha / r) (x A^T) B^T`` where ``W`` carries adapter factors."""
        y = S.linear(x, getattr(self, name))
        if name in self.adapted:
            low = S.linear(S.linear(x, getattr(self, f"{name}_lora_a")), getattr(self, f"{name}_lora_b"))
            y = y + low * self.lora.scale
        return y

    def _adapt(self, lora, dtype) -> None:
        """Adds the low-rank factors of every targeted matrix (and expert bank) of this layer and,
        unless the base trains too, freezes everything else: frozen parameters get no gradient
        object, no moments and no update task (models/lora.py; the reference's ``configure_lora``,
        packages/workloads/src/shadowspill_workloads/lora/__init__.py:16)."""
        if lora is None:
            return
        self.lora = lora
        base = dict(self.named_parameters(recurse=False))
        adapted = set()
        for name, p in base.items():
            is_bank = p.dim() == 3
            if name not in lora.targets or p.dim() < 2 or (is_bank and not lora.routed_experts):
                continue
            lead = tuple(p.shape[:-2])
            setattr(self, f"{name}_lora_a", _param(lead + (lora.rank, p.shape[-1]), std=self.cfg.initializer_range,
                                                   dtype=dtype))
            setattr(self, f"{name}_lora_b", _param(lead + (p.shape[-2], lora.rank), "zeros", dtype=dtype))
            adapted.add(name)
        self.adapted = frozenset(adapted)
        if not lora.train_base:
            for p in base.values():
                p.requires_grad_(False)

    def _mlp(self, x):
        h = self._norm(x, self.mlp_norm)
        c = self.cfg
        if not c.is_moe:
            return x + self._lin(S.swiglu(self._lin(h, "w13")), "w2")
        logits = S.linear(h, self.router).float()
        if c.router_scoring == "sigmoid":
            # scores in (0, 1); a frozen per-expert bias takes part in the selection only; the picked
            # scores are renormalised and scaled (GLM / DeepSeek-style routing without an auxiliary loss)
            scores = torch.sigmoid(logits)
            ids = torch.topk(scores + self.router_bias.float(), c.top_k, dim=-1).indices
            picked = torch.gather(scores, 1, ids)
            wts = picked / (picked.sum(-1, keepdim=True) + 1e-20) * c.routed_scaling_factor
            if "w13" in self.adapted:
                out = S.moe_experts_routed_lora(h, ids.to(torch.int32), wts, self.w13, self.w2, self.w13_lora_a,
                                                self.w13_lora_b, self.w2_lora_a, self.w2_lora_b, float(self.lora.scale))
            else:
                out = S.moe_experts_routed(h, ids.to(torch.int32), wts, self.w13, self.w2)
        elif "w13" in self.adapted:     # both banks carry per-expert factors (see graph_stage.supports)
            out = S.moe_experts_lora(h, logits, self.w13, self.w2, self.w13_lora_a, self.w13_lora_b,
                                     self.w2_lora_a, self.w2_lora_b, c.top_k, c.router_renormalize,
                                     float(self.lora.scale))
        else:
            out = S.moe_experts(h, logits, self.w13, self.w2, c.top_k, c.router_renormalize)
        if c.d_shared_expert:
            shared = self._lin(S.swiglu(self._lin(h, "sw13")), "sw2")
            if c.gated_shared_expert:
                shared = shared * torch.sigmoid(h.float() @ self.shared_gate.float()).to(h.dtype)[:, None]
            out = out + shared
        return x + out


class DenseLayer(nn.Module, _Norms):
    """Pre-norm GQA attention + SwiGLU; q/k/v and gate/up are fused projections."""

    def __init__(self, cfg: DecoderConfig, dtype):
        super().__init__()
        self.cfg = cfg
        D, dh, Hq, Hkv, Ff = cfg.d_model, cfg.head_dim, cfg.n_heads, cfg.n_kv_heads, cfg.d_ff
        std = cfg.initializer_range
        ninit = "zeros" if cfg.zero_centered_norm else "ones"
        self.attn_norm = _param((D,), ninit, dtype=dtype)
        self.wqkv = _param(((Hq + 2 * Hkv) * dh, D), std=std, dtype=dtype)
        self.wo = _param((D, Hq * dh), std=std, dtype=dtype)
        self.mlp_norm = _param((D,), ninit, dtype=dtype)
        self.w13 = _param((2 * Ff, D), std=std, dtype=dtype)
        self.w2 = _param((D, Ff), std=std, dtype=dtype)
        if cfg.qk_norm:
            self.q_norm = _param((dh,), ninit, dtype=dtype)
            self.k_norm = _param((dh,), ninit, dtype=dtype)

    def forward(self, x, positions, cu_seqlens):
        c = self.cfg
        T = x.shape[0]
        dh, Hq, Hkv = c.head_dim, c.n_heads, c.n_kv_heads
        h = self._norm(x, self.attn_norm)
        qkv = S.linear(h, self.wqkv)
        if c.qk_norm:
            qn = self._norm(qkv[:, :Hq * dh].reshape(T * Hq, dh), self.q_norm).reshape(T, Hq * dh)
            kn = self._norm(qkv[:, Hq * dh:(Hq + Hkv) * dh].reshape(T * Hkv, dh), self.k_norm).reshape(T, Hkv * dh)
            qkv = torch.cat([qn, kn, qkv[:, (Hq + Hkv) * dh:]], dim=1)
        # q and k heads are adjacent in the fused projection: one rotary launch covers both
        qkv = S.rope(qkv, positions, Hq + Hkv, dh, c.rotary_width, c.rope_base, False)
        q = qkv[:, :Hq * dh].view(T, Hq, dh)
        k = qkv[:, Hq * dh:(Hq + Hkv) * dh].view(T, Hkv, dh)
        v = qkv[:, (Hq + Hkv) * dh:].view(T, Hkv, dh)
        att, _ = S.attention(q, k, v, cu_seqlens, T)
        x = x + S.linear(att.view(T, Hq * dh), self.wo)
        return self._mlp(x)


class HybridLayer(nn.Module, _Norms):
    """Gated DeltaNet or (gated) full attention mixer + dense SwiGLU feed-forward."""

    def __init__(self, cfg: DecoderConfig, index: int, dtype, lora=None):
        super().__init__()
        self.cfg, self.index = cfg, index
        self.mixer = cfg.layer_kind(index)
        c, std = cfg, cfg.initializer_range
        D, dh, Hq, Hkv = c.d_model, c.head_dim, c.n_heads, c.n_kv_heads
        ninit = "zeros" if c.zero_centered_norm else "ones"
        self.attn_norm = _param((D,), ninit, dtype=dtype)
        if self.mixer == "attention":
            self.wq = _param((Hq * dh * (2 if c.gated_attention else 1), D), std=std, dtype=dtype)
            self.wk = _param((Hkv * dh, D), std=std, dtype=dtype)
            self.wv = _param((Hkv * dh, D), std=std, dtype=dtype)
            self.wo = _param((D, Hq * dh), std=std, dtype=dtype)
            if c.qk_norm:
                qn, kn = (Hq * dh, Hkv * dh) if c.qk_norm_full_width else (dh, dh)
                self.q_norm = _param((qn,), ninit, dtype=dtype)
                self.k_norm = _param((kn,), ninit, dtype=dtype)
        else:
            self.key_width = c.dn_qk_heads * c.dn_head_dim
            self.value_width = c.dn_v_heads * c.dn_head_dim
            self.conv_width = 2 * self.key_width + self.value_width
            self.w_qkvz = _param((self.conv_width + self.value_width, D), std=std, dtype=dtype)
            self.w_ba = _param((2 * c.dn_v_heads, D), std=std, dtype=dtype)
            self.conv_w = _param((self.conv_width, c.dn_conv_width), std=0.3, dtype=dtype)
            self.A_log = _param((c.dn_v_heads,), "zeros", dtype=torch.float32)
            self.dt_bias = _param((c.dn_v_heads,), "zeros", dtype=torch.float32)
            self.lin_norm = _param((c.dn_head_dim,), ninit, dtype=dtype)
            self.w_out = _param((D, self.value_width), std=std, dtype=dtype)
        self.mlp_norm = _param((D,), ninit, dtype=dtype)
        if c.is_moe:
            self.router = _param((c.n_experts, D), std=std, dtype=dtype)
            self.w13 = _param((c.n_experts, 2 * c.d_expert, D), std=std, dtype=dtype)
            self.w2 = _param((c.n_experts, D, c.d_expert), std=std, dtype=dtype)
            if c.d_shared_expert:
                self.sw13 = _param((2 * c.d_shared_expert, D), std=std, dtype=dtype)
                self.sw2 = _param((D, c.d_shared_expert), std=std, dtype=dtype)
                if c.gated_shared_expert:
                    self.shared_gate = _param((D,), std=std, dtype=dtype)
        else:
            self.w13 = _param((2 * c.d_ff, D), std=std, dtype=dtype)
            self.w2 = _param((D, c.d_ff), std=std, dtype=dtype)
        self._adapt(lora, dtype)

    def _attention(self, h, positions, cu_seqlens):
        c = self.cfg
        T = h.shape[0]
        dh, Hq, Hkv = c.head_dim, c.n_heads, c.n_kv_heads
        qg = self._lin(h, "wq")
        q, gate = (qg[:, :Hq * dh], qg[:, Hq * dh:]) if c.gated_attention else (qg, None)
        k, v = self._lin(h, "wk"), self._lin(h, "wv")
        if c.qk_norm and c.qk_norm_full_width:
            q, k = self._norm(q, self.q_norm), self._norm(k, self.k_norm)
        elif c.qk_norm:
            q = self._norm(q.reshape(T * Hq, dh), self.q_norm).reshape(T, Hq * dh)
            k = self._norm(k.reshape(T * Hkv, dh), self.k_norm).reshape(T, Hkv * dh)
        q = S.rope(q, positions, Hq, dh, c.rotary_width, c.rope_base, False)
        k = S.rope(k, positions, Hkv, dh, c.rotary_width, c.rope_base, False)
        att, _ = S.attention(q.view(T, Hq, dh), k.view(T, Hkv, dh), v.view(T, Hkv, dh), cu_seqlens, T)
        att = att.reshape(T, Hq * dh)
        if gate is not None:
            att = att * torch.sigmoid(gate.float()).to(att.dtype)
        return self._lin(att, "wo")

    def _deltanet(self, h, positions, cu_seqlens):
        c = self.cfg
        T = h.shape[0]
        Hk, Hv, dk = c.dn_qk_heads, c.dn_v_heads, c.dn_head_dim
        kw, cw = self.key_width, self.conv_width
        qkvz = self._lin(h, "w_qkvz")
        ba = S.linear(h, self.w_ba)
        conv = S.conv_silu(qkvz[:, :cw], self.conv_w, positions, cu_seqlens)
        q = S.l2norm(conv[:, :kw].reshape(T, Hk, dk), 1e-6)
        k = S.l2norm(conv[:, kw:2 * kw].reshape(T, Hk, dk), 1e-6)
        v = conv[:, 2 * kw:].reshape(T, Hv, dk)
        beta = torch.sigmoid(ba[:, :Hv].float())
        g = -torch.exp(self.A_log.float()) * torch.nn.functional.softplus(ba[:, Hv:].float() + self.dt_bias.float())
        mixed = S.gated_delta_rule(q, k, v, beta, g, cu_seqlens, c.dn_chunk)
        gate = qkvz[:, cw:].reshape(T, Hv, dk)
        normed = S.gated_rmsnorm(mixed, gate, self.lin_norm, c.norm_epsilon, c.zero_centered_norm)
        return self._lin(normed.reshape(T, Hv * dk), "w_out")

    def forward(self, x, positions, cu_seqlens):
        h = self._norm(x, self.attn_norm)
        mix = (self._attention if self.mixer == "attention" else self._deltanet)(h, positions, cu_seqlens)
        return self._mlp(x + mix)


def _rotate_pairs(x, positions, theta: float):
    """Rotary embedding over interleaved (even, odd) input pairs, emitted as the real half followed
    by the imaginary half (the layout of the published GLM checkpoints)."""
    import math
    width = x.shape[-1]
    # 0, 1, ..., width/2 - 1 built from an input: a tensor created on a named device would pin the
    # exported graph to the device it was traced on
    one = positions[:1].to(torch.float32) * 0 + 1
    k = torch.cumsum(one.expand(width // 2), 0) - 1
    freq = torch.exp(k * (-2.0 * math.log(theta) / width))
    ang = positions.to(torch.float32)[:, None] * freq
    cos, sin = ang.cos().to(x.dtype), ang.sin().to(x.dtype)
    if x.dim() == 3:
        cos, sin = cos[:, None], sin[:, None]
    re, im = x[..., 0::2], x[..., 1::2]
    return torch.cat((re * cos - im * sin, im * cos + re * sin), -1)


class LatentAttentionLayer(nn.Module, _Norms):
    """Sparse multi-head latent attention + dense or routed feed-forward (GLM 5.3).

    Queries go through a low-rank latent (``q_a`` -> norm -> ``q_b``); keys and values share one
    compressed latent per token (``kv_a`` -> norm) plus one rotary key; the per-head key and value
    projections (``kv_b``) are absorbed into the query and the output, so attention itself runs in
    the latent space over the rows an indexer picked. A layer with ``indexer == "full"`` owns a
    frozen indexer and returns its picks; a ``"shared"`` layer reuses the picks it is given.
    Reference: packages/workloads/src/shadowspill_workloads/models/glm53/implementations/mlops/
    attention.py:92-176 (``SparseMLA``), :49-89 (``Indexer``)."""

    def __init__(self, cfg: DecoderConfig, index: int, dtype, lora=None):
        super().__init__()
        self.cfg, self.index = cfg, index
        c, std = cfg, cfg.initializer_range
        D, H = c.d_model, c.n_heads
        ninit = "ones"
        self.attn_norm = _param((D,), ninit, dtype=dtype)
        self.q_a = _param((c.q_lora_rank, D), std=std, dtype=dtype)
        self.q_a_norm = _param((c.q_lora_rank,), ninit, dtype=dtype)
        self.q_b = _param((H * (c.qk_nope_head_dim + c.qk_rope_head_dim), c.q_lora_rank), std=std, dtype=dtype)
        self.kv_a = _param((c.kv_lora_rank + c.qk_rope_head_dim, D), std=std, dtype=dtype)
        self.kv_a_norm = _param((c.kv_lora_rank,), ninit, dtype=dtype)
        self.kv_b = _param((H * (c.qk_nope_head_dim + c.v_head_dim), c.kv_lora_rank), std=std, dtype=dtype)
        self.wo = _param((D, H * c.v_head_dim), std=std, dtype=dtype)
        self.own_indexer = c.indexer_types[index] == "full"
        if self.own_indexer:          # never trained: it only selects
            self.ix_q = _param((c.index_n_heads * c.index_head_dim, c.q_lora_rank), std=std, dtype=dtype, trainable=False)
            self.ix_k = _param((c.index_head_dim, D), std=std, dtype=dtype, trainable=False)
            self.ix_k_norm = _param((c.index_head_dim,), "ones", dtype=dtype, trainable=False)
            self.ix_k_bias = _param((c.index_head_dim,), "zeros", dtype=dtype, trainable=False)
            self.ix_w = _param((c.index_n_heads, D), std=std, dtype=dtype, trainable=False)
        self.mlp_norm = _param((D,), ninit, dtype=dtype)
        self.moe = c.layer_is_moe(index)
        if self.moe:
            self.router = _param((c.n_experts, D), std=std, dtype=dtype)
            self.router_bias = _param((c.n_experts,), "zeros", dtype=torch.float32, trainable=False)
            self.w13 = _param((c.n_experts, 2 * c.d_expert, D), std=std, dtype=dtype)
            self.w2 = _param((c.n_experts, D, c.d_expert), std=std, dtype=dtype)
            if c.d_shared_expert:
                self.sw13 = _param((2 * c.d_shared_expert, D), std=std, dtype=dtype)
                self.sw2 = _param((D, c.d_shared_expert), std=std, dtype=dtype)
        else:
            self.w13 = _param((2 * c.d_ff, D), std=std, dtype=dtype)
            self.w2 = _param((D, c.d_ff), std=std, dtype=dtype)
        self._adapt(lora, dtype)

    def _mlp(self, x):
        if self.moe:
            return _Norms._mlp(self, x)
        h = self._norm(x, self.mlp_norm)
        return x + self._lin(S.swiglu(self._lin(h, "w13")), "w2")

    def _picks(self, h, q_res, positions, cu_seqlens):
        c = self.cfg
        T, r = h.shape[0], c.qk_rope_head_dim
        q = S.linear(q_res, self.ix_q).reshape(T, c.index_n_heads, c.index_head_dim)
        key = torch.nn.functional.layer_norm(S.linear(h, self.ix_k).float(), (c.index_head_dim,),
                                             self.ix_k_norm.float(), self.ix_k_bias.float(), 1e-6).to(h.dtype)
        q = torch.cat((_rotate_pairs(q[..., :r], positions, c.rope_base), q[..., r:]), -1)
        key = torch.cat((_rotate_pairs(key[..., :r], positions, c.rope_base), key[..., r:]), -1)
        # a handful of head weights per token: a plain product (no tile or alignment constraints)
        head_weights = h.float() @ self.ix_w.float().t()
        return S.index_topk(q, key, head_weights, cu_seqlens, c.index_topk)

    def forward(self, x, positions, cu_seqlens, picks=None):
        c = self.cfg
        T, H = x.shape[0], c.n_heads
        n, r, dv, L = c.qk_nope_head_dim, c.qk_rope_head_dim, c.v_head_dim, c.kv_lora_rank
        h = self._norm(x, self.attn_norm)
        q_res = S.rmsnorm(self._lin(h, "q_a"), self.q_a_norm, 1e-6, False)[0]
        qb = self._lin(q_res, "q_b").reshape(T, H, n + r)
        query, q_rope = qb[..., :n], qb[..., n:]
        kv = self._lin(h, "kv_a")
        latent = S.rmsnorm(kv[:, :L], self.kv_a_norm, 1e-6, False)[0]
        k_rope = _rotate_pairs(kv[:, L:], positions, c.rope_base)
        q_rope = _rotate_pairs(q_rope, positions, c.rope_base)
        if self.own_indexer:
            picks = self._picks(h, q_res, positions, cu_seqlens)
        w = self.kv_b.reshape(H, n + dv, L)
        wk, wv = w[:, :n], w[:, n:]
        q_latent = torch.einsum("thd,hdl->thl", query, wk)                   # key projection absorbed into the query
        adapted = "kv_b" in self.adapted
        if adapted:
            # the adapter of the absorbed projection, absorbed the same way: W + s B A splits into the key
            # rows and the value rows of B, and A (rank x latent) stays on the latent side
            fa = self.kv_b_lora_a
            fb = self.kv_b_lora_b.reshape(H, n + dv, fa.shape[0])
            bk, bv = fb[:, :n], fb[:, n:]
            q_latent = q_latent + (torch.einsum("thd,hdr->thr", query, bk) @ fa) * self.lora.scale
        attended = S.sparse_latent_attention(q_latent, latent, picks, q_rope, k_rope, float((n + r) ** -0.5))
        value = torch.einsum("thl,hdl->thd", attended, wv)                   # value projection applied after
        if adapted:
            value = value + torch.einsum("thr,hdr->thd", attended @ fa.t(), bv) * self.lora.scale
        x = x + self._lin(value.reshape(T, H * dv), "wo")
        return self._mlp(x), picks


class LatentAttentionGroup(nn.Module):
    """A layer with its own indexer and the layers after it that reuse its picks: one repeated
    child, hence one stage, so the picks never cross a stage boundary."""

    def __init__(self, cfg: DecoderConfig, indices: list[int], dtype, lora=None):
        super().__init__()
        self.members = nn.ModuleList([LatentAttentionLayer(cfg, i, dtype, lora) for i in indices])

    def forward(self, x, positions, cu_seqlens):
        picks = None
        for layer in self.members:
            x, picks = layer(x, positions, cu_seqlens, picks)
        return x


class Head(nn.Module):
    """Final norm + output projection + masked weighted-sum cross entropy in row blocks."""

    def __init__(self, cfg: DecoderConfig, dtype, block_rows: int = 2048, trainable: bool = True):
        super().__init__()
        self.cfg, self.block_rows = cfg, block_rows
        ninit = "zeros" if cfg.zero_centered_norm else "ones"
        self.final_norm = _param((cfg.d_model,), ninit, dtype=dtype, trainable=trainable)
        if not cfg.tied_embeddings:
            self.head = _param((cfg.vocab_size, cfg.d_model), std=cfg.initializer_range, dtype=dtype,
                               trainable=trainable)

    def forward(self, x, targets, weights, tied=None):
        c = self.cfg
        h = S.rmsnorm(x, self.final_norm, c.norm_epsilon, c.zero_centered_norm)[0]
        W = tied if c.tied_embeddings else self.head
        return S.head_loss(h, W, targets, weights, self.block_rows)[0]


class DecoderLM(nn.Module):
    """``forward(tokens, targets, weights, positions, cu_seqlens) -> loss[1]``."""

    def __init__(self, cfg: DecoderConfig, dtype=torch.bfloat16, head_block_rows: int = 2048, lora=None):
        """``lora`` (a ``models.lora.LoRAConfig``): every layer is the form with separate q / k / v
        projections (the adapter targets), carries the factors, and the base is frozen unless
        ``lora.train_base``."""
        super().__init__()
        self.cfg = cfg
        base = lora is None or lora.train_base
        self.embed = Embedding(cfg, dtype, base)
        layers = []
        if cfg.is_latent_attention:
            layers = [LatentAttentionGroup(cfg, group, dtype, lora) for group in cfg.layer_groups()]
        for i in range(0 if cfg.is_latent_attention else cfg.n_layers):
            plain = (cfg.layer_kind(i) == "attention" and not cfg.gated_attention and not cfg.is_moe
                     and lora is None)
            layers.append(DenseLayer(cfg, dtype) if plain else HybridLayer(cfg, i, dtype, lora))
        self.layers = nn.ModuleList(layers)
        self.head = Head(cfg, dtype, head_block_rows, base)

    def forward(self, tokens, targets, weights, positions, cu_seqlens):
        x = self.embed(tokens)
        for layer in self.layers:
            x = layer(x, positions, cu_seqlens)
        tied = self.embed.embed if self.cfg.tied_embeddings else None
        return self.head(x, targets, weights, tied)


def init_(module: nn.Module, seed: int = 0) -> None:
    """Seed-only initialisation following each parameter's ``ss_init`` / ``ss_std`` tags."""
    gen = torch.Generator().manual_seed(seed)
    with torch.no_grad():
        for p in module.parameters():
            kind = getattr(p, "ss_init", "normal")
            if kind == "ones":
                p.fill_(1.0)
            elif kind == "zeros":
                p.zero_()
            else:
                tmp = torch.empty(p.shape, dtype=torch.float32)
                tmp.normal_(0.0, getattr(p, "ss_std", 0.02), generator=gen)
                p.copy_(tmp)
