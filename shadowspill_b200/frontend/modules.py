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
        if "w13" in self.adapted:       # both banks carry per-expert factors (see graph_stage.supports)
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
        for i in range(cfg.n_layers):
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
