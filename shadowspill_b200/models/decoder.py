"""Decoder stages with hand-written forward and backward passes.

A model is a list of *stages* (embedding, one per decoder layer, head+loss).
Each stage owns a flat parameter layout and two executable forms of its
forward pass: one that keeps a chosen set of intermediates for the backward
pass (``save``) and one that keeps nothing but its input (``recompute``). This
is the unit the planner reasons about, as the reference's stage graph pairs are
(docs/architecture/graph-pair-construction.md:255-346), except that the
backward pass here is written by hand on top of the op library rather than
derived by AOTAutograd, so every temporary is explicit.

Math follows the reference models:
  Llama 3   packages/workloads/src/shadowspill_workloads/models/llama3/implementations/mlops.py:29-161
  Qwen 3    GQA with per-head q/k RMSNorm (models/shared/qwen_moe/attention.py:32)
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Callable

import torch

from ..ops import functional as F
from .config import DecoderConfig

ALIGN = 256  # byte alignment of every tensor inside a flat stage buffer


@dataclass(frozen=True)
class ParamSpec:
    name: str
    shape: tuple[int, ...]
    init: str = "normal"          # normal | ones | zeros
    std: float = 0.02
    dtype: torch.dtype | None = None   # None = the model dtype; fp32 exceptions set this
    trainable: bool = True
    # expert parallelism: this rank holds experts [lo, lo + shape[0]) of a bank whose whole
    # shape is ``global_shape``; such a tensor is never cut into flat 1/N shards or gathered
    global_shape: tuple[int, ...] | None = None
    expert_lo: int = 0

    @property
    def expert_sharded(self) -> bool:
        return self.global_shape is not None

    @property
    def numel(self) -> int:
        return math.prod(self.shape)


@dataclass
class BatchMeta:
    """One packed microbatch. All tensors live on the compute device."""
    tokens: torch.Tensor        # int64 [T]
    targets: torch.Tensor       # int64 [T]   (-1 where no loss)
    weights: torch.Tensor       # fp32  [T]   (0 where masked)
    positions: torch.Tensor     # int32 [T]
    cu_seqlens: torch.Tensor    # int32 [S+1]
    max_seqlen: int
    extras: dict = field(default_factory=dict)   # further inputs: fp32 [T] or [T, width] each

    @property
    def T(self) -> int:
        return self.tokens.numel()


def _round_up(n: int, a: int) -> int:
    return (n + a - 1) // a * a


class Stage:
    """Base class: parameter layout + flat-buffer views."""
    kind = "stage"

    def __init__(self, name: str, cfg: DecoderConfig):
        self.name = name
        self.cfg = cfg
        self.params: list[ParamSpec] = []
        # sharded storage keeps tensors smaller than this whole on every rank (0 = shard all)
        self.min_shard_bytes = 0

    # ---- layout
    def parameter_count(self) -> int:
        return sum(p.numel for p in self.params)

    @property
    def has_trainable(self) -> bool:
        return any(p.trainable for p in self.params)

    def layout(self, dtype: torch.dtype, vector_dtype: torch.dtype | None = None,
               trainable_only: bool = False):
        """[(spec, byte offset, dtype)], total bytes. ``vector_dtype`` overrides
        the dtype of 1-D parameters (gradient buffers keep those in fp32);
        ``trainable_only`` lays out gradient and optimizer-state buffers, which hold
        nothing for frozen parameters."""
        out, off = [], 0
        for p in self.params:
            if trainable_only and not p.trainable:
                continue
            dt = p.dtype or (vector_dtype if (vector_dtype and len(p.shape) == 1) else dtype)
            out.append((p, off, dt))
            off = _round_up(off + p.numel * dt.itemsize, ALIGN)
        return out, off

    def views(self, flat: torch.Tensor, dtype: torch.dtype,
              vector_dtype: torch.dtype | None = None,
              trainable_only: bool = False) -> dict[str, torch.Tensor]:
        """Named tensor views over a flat uint8 buffer."""
        lay, total = self.layout(dtype, vector_dtype, trainable_only)
        if flat.numel() < total:
            raise ValueError(f"{self.name}: buffer of {flat.numel()} B < layout {total} B")
        res = {}
        for p, off, dt in lay:
            res[p.name] = flat[off:off + p.numel * dt.itemsize].view(dt).view(p.shape)
        return res

    # ---- data-parallel sharded storage: every tensor is cut into `world` equal
    # padded slices (a multiple of 8 elements each); a rank stores slice `rank`.
    def shard_layout(self, dtype: torch.dtype, world: int, trainable_only: bool = False):
        """[(spec, byte offset, dtype, elements per shard)], total bytes of one shard."""
        out, off = [], 0
        for p in self.params:
            if trainable_only and not p.trainable:
                continue
            dt = p.dtype or dtype
            if p.expert_sharded or self.kept_whole(p, dtype):
                # the local bank is this rank's own; a small tensor is not worth cutting
                per = -(-p.numel // 8) * 8
            else:
                per = -(-(-(-p.numel // world)) // 8) * 8
            out.append((p, off, dt, per))
            off = _round_up(off + per * dt.itemsize, ALIGN)
        return out, off

    def kept_whole(self, p: ParamSpec, dtype: torch.dtype) -> bool:
        """Under sharded storage: is ``p`` stored whole on every rank (replicated, updated by
        every rank from the summed gradient) because it is smaller than ``min_shard_bytes``?"""
        return (not p.expert_sharded and self.min_shard_bytes > 0
                and p.numel * (p.dtype or dtype).itemsize < self.min_shard_bytes)

    def owned_span(self, p: ParamSpec, dtype: torch.dtype, world: int, rank: int) -> tuple[int, int]:
        """``[lo, hi)`` of ``p``'s flat elements that ``rank`` stores under sharded storage."""
        if world <= 1 or self.kept_whole(p, dtype):
            return 0, p.numel
        per = -(-(-(-p.numel // world)) // 8) * 8
        lo = min(p.numel, rank * per)
        return lo, min(p.numel, lo + per)

    def shard_views(self, flat: torch.Tensor, dtype: torch.dtype, world: int,
                    trainable_only: bool = False) -> dict[str, torch.Tensor]:
        lay, total = self.shard_layout(dtype, world, trainable_only)
        if flat.numel() < total:
            raise ValueError(f"{self.name}: buffer of {flat.numel()} B < shard layout {total} B")
        return {p.name: flat[off:off + per * dt.itemsize].view(dt) for p, off, dt, per in lay}

    def init_(self, P: dict[str, torch.Tensor], generator: torch.Generator) -> None:
        """Deterministic seed-only initialisation, independent of any sharding."""
        for p in self.params:
            t = P[p.name]
            if p.init == "ones":
                t.fill_(1.0)
            elif p.init == "zeros":
                t.zero_()
            elif p.expert_sharded:
                # draw the whole bank so that every rank consumes the same random stream
                # and the union of the ranks' slices equals the single-rank model
                full = torch.empty(p.global_shape, dtype=t.dtype if t.is_cuda else torch.float32,
                                   device=t.device)
                full.normal_(0.0, p.std, generator=generator)
                t.copy_(full[p.expert_lo:p.expert_lo + p.shape[0]])
            elif t.is_cuda:
                t.normal_(0.0, p.std, generator=generator)   # device generator, large models
            else:
                tmp = torch.empty(p.shape, dtype=torch.float32)
                tmp.normal_(0.0, p.std, generator=generator)
                t.copy_(tmp)

    # ---- execution (overridden)
    SAVE_SETS: dict[str, tuple[str, ...]] = {"recompute": ()}

    def activation_bytes(self, T: int, variant: str, itemsize: int = 2) -> int:
        return 0

    def workspace_bytes(self, T: int, itemsize: int = 2) -> int:
        return 0

    def flops(self, T: int, mean_seqlen: float) -> float:
        return 0.0


# ============================================================================ embedding
class EmbeddingStage(Stage):
    kind = "embedding"

    def __init__(self, name, cfg, trainable: bool = True):
        super().__init__(name, cfg)
        self.params = [ParamSpec("embed", (cfg.vocab_size, cfg.d_model), std=cfg.initializer_range,
                                 trainable=trainable)]

    def forward(self, P, x, meta: BatchMeta, keep=None, out=None):
        return F.embedding_fwd(meta.tokens, P["embed"], out=out), {}

    def backward(self, P, G, x, dy, meta: BatchMeta, saved, first: bool):
        if first:
            G["embed"].zero_()
        F.embedding_bwd(meta.tokens, dy, G["embed"])
        return None

    def flops(self, T, mean_seqlen):
        return 0.0


# ============================================================================ dense decoder layer
class DenseLayerStage(Stage):
    """Pre-norm GQA attention + SwiGLU MLP. q/k/v and gate/up are single fused
    projections; the two residual adds are folded into GEMM epilogues."""
    kind = "layer"
    # matrices whose first use in a forward pass is ``x @ W^T``: their all-gather can be fused into
    # that GEMM under sharded storage
    fused_gather_params = ("wqkv", "wo", "w13", "w2")
    SAVE_SETS = {
        "recompute": (),
        "save_attention": ("qkv", "attn", "lse"),
        # also keeps the gate/up projection: the backward pass then recomputes only the small
        # output-projection GEMM and the elementwise pieces (the gate/up GEMM is 85 % of the
        # recomputed FLOPs of save_attention)
        "save_attention_gu": ("qkv", "attn", "lse", "gu"),
        "save": ("h1", "rstd1", "qkv", "attn", "lse", "x_mid", "h2", "rstd2", "gu", "hmlp"),
    }

    def __init__(self, name, cfg):
        super().__init__(name, cfg)
        D, dh, Hq, Hkv, Ff = cfg.d_model, cfg.head_dim, cfg.n_heads, cfg.n_kv_heads, cfg.d_ff
        std = cfg.initializer_range
        norm_init = "zeros" if cfg.zero_centered_norm else "ones"
        self.qkv_width = (Hq + 2 * Hkv) * dh
        self.params = [
            ParamSpec("attn_norm", (D,), init=norm_init),
            ParamSpec("wqkv", (self.qkv_width, D), std=std),
            ParamSpec("wo", (D, Hq * dh), std=std),
            ParamSpec("mlp_norm", (D,), init=norm_init),
            ParamSpec("w13", (2 * Ff, D), std=std),
            ParamSpec("w2", (D, Ff), std=std),
        ]
        if cfg.qk_norm:
            self.params += [ParamSpec("q_norm", (dh,), init=norm_init),
                            ParamSpec("k_norm", (dh,), init=norm_init)]

    # ---- sizes
    def activation_bytes(self, T, variant, itemsize=2):
        c = self.cfg
        per_tok = {"h1": c.d_model, "qkv": self.qkv_width, "attn": c.n_heads * c.head_dim,
                   "x_mid": c.d_model, "h2": c.d_model, "gu": 2 * c.d_ff, "hmlp": c.d_ff}
        total = 0
        for n in self.SAVE_SETS[variant]:
            if n in per_tok:
                total += T * per_tok[n] * itemsize
            elif n == "lse":
                total += T * c.n_heads * 4
            else:
                total += T * 4
        return total

    def saved_shapes(self, T, variant, dtype=torch.bfloat16):
        """[(name, shape, dtype)] of the tensors a ``variant`` forward keeps."""
        c = self.cfg
        shapes = {"h1": (T, c.d_model), "qkv": (T, self.qkv_width),
                  "attn": (T, c.n_heads * c.head_dim), "x_mid": (T, c.d_model),
                  "h2": (T, c.d_model), "gu": (T, 2 * c.d_ff), "hmlp": (T, c.d_ff)}
        out = []
        for n in self.SAVE_SETS[variant]:
            if n in shapes:
                out.append((n, shapes[n], dtype))
            elif n == "lse":
                out.append((n, (c.n_heads, T), torch.float32))
            else:
                out.append((n, (T,), torch.float32))
        if c.qk_norm and "qkv" in self.SAVE_SETS[variant]:
            out += [("qk_raw", (T, (c.n_heads + c.n_kv_heads) * c.head_dim), dtype),
                    ("q_rstd", (T * c.n_heads,), torch.float32),
                    ("k_rstd", (T * c.n_kv_heads,), torch.float32)]
        return out

    def workspace_bytes(self, T, itemsize=2):
        c = self.cfg
        # backward peak: every intermediate of the forward plus dgu and dqkv
        fwd = self.activation_bytes(T, "save", itemsize)
        return fwd + T * (2 * c.d_ff + c.d_ff + self.qkv_width + c.n_heads * c.head_dim
                          + c.d_model) * itemsize

    def flops(self, T, mean_seqlen):
        c = self.cfg
        gemm = 2.0 * T * c.d_model * (self.qkv_width + c.n_heads * c.head_dim + 3 * c.d_ff)
        attn = 2.0 * 2.0 * T * (mean_seqlen / 2.0) * c.n_heads * c.head_dim
        return gemm + attn

    # ---- forward
    def _compute(self, P, x, meta: BatchMeta, have: dict, upto: str = "end", out=None, bufs=None):
        """Fill in every intermediate missing from ``have`` (recompute path). ``bufs``
        names preallocated destinations (the views of a saved-set object), so that a
        saving forward writes what it keeps exactly once, in place."""
        c = self.cfg
        T = x.shape[0]
        dh, Hq, Hkv = c.head_dim, c.n_heads, c.n_kv_heads
        I = dict(have)
        bufs = bufs or {}
        b = bufs.get
        if "qkv" not in I or "h1" not in I:
            h1, rstd1 = F.rmsnorm_fwd(x, P["attn_norm"], c.norm_epsilon, c.zero_centered_norm,
                                      out=b("h1"), rstd=b("rstd1"))
            I["h1"], I["rstd1"] = h1, rstd1
        if "qkv" not in I:
            qkv = F.linear_fwd(I["h1"], P["wqkv"], out=b("qkv"))
            if c.qk_norm:
                self._qk_norm_fwd(P, qkv, I)
            # q and k heads are adjacent in the fused projection: one rotary launch covers both
            F.rope_(qkv, meta.positions, col0=0, heads=Hq + Hkv, dh=dh, rot=c.rotary_width,
                    theta=c.rope_base)
            I["qkv"] = qkv
        qkv = I["qkv"]
        q = qkv[:, :Hq * dh].view(T, Hq, dh)
        k = qkv[:, Hq * dh:(Hq + Hkv) * dh].view(T, Hkv, dh)
        v = qkv[:, (Hq + Hkv) * dh:].view(T, Hkv, dh)
        if "attn" not in I:
            ao = b("attn")
            attn, lse = F.attention_varlen(q, k, v, meta.cu_seqlens, meta.max_seqlen,
                                           out=None if ao is None else ao.view(T, Hq, dh),
                                           lse=b("lse"))
            I["attn"], I["lse"] = attn.view(T, Hq * dh), lse
        if "x_mid" not in I:
            x_mid = out if out is not None else torch.empty_like(x)
            x_mid.copy_(x)
            F.linear_fwd(I["attn"], P["wo"], out=x_mid, accumulate=True)
            I["x_mid"] = x_mid
        if "h2" not in I or "gu" not in I:
            I["h2"], I["rstd2"] = F.rmsnorm_fwd(I["x_mid"], P["mlp_norm"], c.norm_epsilon,
                                                c.zero_centered_norm, out=b("h2"), rstd=b("rstd2"))
        if "gu" not in I:
            I["gu"] = F.linear_fwd(I["h2"], P["w13"], out=b("gu"))
        if "hmlp" not in I:
            I["hmlp"] = F.swiglu_fwd(I["gu"], out=b("hmlp"))
        return I

    def _qk_norm_fwd(self, P, qkv, I):
        c = self.cfg
        T = qkv.shape[0]
        dh, Hq, Hkv = c.head_dim, c.n_heads, c.n_kv_heads
        # keep the pre-norm q/k for the backward pass
        I["qk_raw"] = qkv[:, :(Hq + Hkv) * dh].clone()
        qv = qkv[:, :Hq * dh].reshape(T * Hq, dh)
        kv = qkv[:, Hq * dh:(Hq + Hkv) * dh].reshape(T * Hkv, dh)
        qn, I["q_rstd"] = F.rmsnorm_fwd(qv, P["q_norm"], c.norm_epsilon, c.zero_centered_norm)
        kn, I["k_rstd"] = F.rmsnorm_fwd(kv, P["k_norm"], c.norm_epsilon, c.zero_centered_norm)
        qkv[:, :Hq * dh] = qn.view(T, Hq * dh)
        qkv[:, Hq * dh:(Hq + Hkv) * dh] = kn.view(T, Hkv * dh)

    def forward(self, P, x, meta: BatchMeta, keep: tuple[str, ...] = (), out=None, saved_out=None):
        """Returns ``(y, saved)`` where ``saved`` holds the intermediates named in ``keep``.
        With ``saved_out`` (name -> preallocated tensor) they are produced in place."""
        I = self._compute(P, x, meta, {}, out=out, bufs=saved_out)
        y = I["x_mid"]
        saved = {}
        if "x_mid" in keep:
            # the output buffer is about to absorb the MLP branch; keep a copy
            if saved_out is not None and "x_mid" in saved_out:
                saved["x_mid"] = saved_out["x_mid"].copy_(y)
            else:
                saved["x_mid"] = y.clone()
        F.linear_fwd(I["hmlp"], P["w2"], out=y, accumulate=True)
        for n in keep:
            if n != "x_mid":
                saved[n] = I[n]
        if self.cfg.qk_norm and "qkv" in keep:
            for n in ("qk_raw", "q_rstd", "k_rstd"):
                saved[n] = I[n]
        return y, saved

    # ---- backward
    def backward(self, P, G, x, dy, meta: BatchMeta, saved: dict, first: bool):
        """``dy`` [T,D] is rewritten in place with the gradient of the stage input.
        Parameter gradients land in ``G`` (created when ``first``, else accumulated)."""
        c = self.cfg
        T = x.shape[0]
        dh, Hq, Hkv = c.head_dim, c.n_heads, c.n_kv_heads
        acc = not first
        I = self._compute(P, x, meta, saved)
        if first:
            G["attn_norm"].zero_(); G["mlp_norm"].zero_()
            if c.qk_norm:
                G["q_norm"].zero_(); G["k_norm"].zero_()
        # ---- MLP branch
        F.linear_wgrad(dy, I["hmlp"], out=G["w2"], accumulate=acc)
        dhmlp = F.linear_dgrad(dy, P["w2"])
        dgu = F.swiglu_bwd(I["gu"], dhmlp)
        del dhmlp
        F.linear_wgrad(dgu, I["h2"], out=G["w13"], accumulate=acc)
        dh2 = F.linear_dgrad(dgu, P["w13"])
        del dgu
        F.rmsnorm_bwd(I["x_mid"], P["mlp_norm"], dh2, I["rstd2"], G["mlp_norm"],
                      c.zero_centered_norm, dx=dy, accumulate=True)
        del dh2
        # ---- attention branch (dy now holds d x_mid)
        F.linear_wgrad(dy, I["attn"], out=G["wo"], accumulate=acc)
        dattn = F.linear_dgrad(dy, P["wo"])
        qkv = I["qkv"]
        q = qkv[:, :Hq * dh].view(T, Hq, dh)
        k = qkv[:, Hq * dh:(Hq + Hkv) * dh].view(T, Hkv, dh)
        v = qkv[:, (Hq + Hkv) * dh:].view(T, Hkv, dh)
        dqkv = torch.empty_like(qkv)
        dq = dqkv[:, :Hq * dh].view(T, Hq, dh)
        dk = dqkv[:, Hq * dh:(Hq + Hkv) * dh].view(T, Hkv, dh)
        dv = dqkv[:, (Hq + Hkv) * dh:].view(T, Hkv, dh)
        _attention_bwd(q, k, v, I["attn"].view(T, Hq, dh), I["lse"], dattn.view(T, Hq, dh),
                       meta, dq, dk, dv)
        del dattn
        F.rope_(dqkv, meta.positions, col0=0, heads=Hq + Hkv, dh=dh, rot=c.rotary_width,
                theta=c.rope_base, inverse=True)
        if c.qk_norm:
            self._qk_norm_bwd(P, G, dqkv, I)
        F.linear_wgrad(dqkv, I["h1"], out=G["wqkv"], accumulate=acc)
        dh1 = F.linear_dgrad(dqkv, P["wqkv"])
        del dqkv
        F.rmsnorm_bwd(x, P["attn_norm"], dh1, I["rstd1"], G["attn_norm"], c.zero_centered_norm,
                      dx=dy, accumulate=True)
        return dy

    def _qk_norm_bwd(self, P, G, dqkv, I):
        c = self.cfg
        T = dqkv.shape[0]
        dh, Hq, Hkv = c.head_dim, c.n_heads, c.n_kv_heads
        raw = I["qk_raw"]
        dqn = dqkv[:, :Hq * dh].reshape(T * Hq, dh)
        dkn = dqkv[:, Hq * dh:(Hq + Hkv) * dh].reshape(T * Hkv, dh)
        dq = F.rmsnorm_bwd(raw[:, :Hq * dh].reshape(T * Hq, dh), P["q_norm"], dqn, I["q_rstd"],
                           G["q_norm"], c.zero_centered_norm)
        dk = F.rmsnorm_bwd(raw[:, Hq * dh:].reshape(T * Hkv, dh), P["k_norm"], dkn, I["k_rstd"],
                           G["k_norm"], c.zero_centered_norm)
        dqkv[:, :Hq * dh] = dq.view(T, Hq * dh)
        dqkv[:, Hq * dh:(Hq + Hkv) * dh] = dk.view(T, Hkv * dh)


def _heads(t: torch.Tensor) -> torch.Tensor:
    return t


def _attention_bwd(q, k, v, out, lse, dout, meta, dq, dk, dv):
    if q.is_cuda:
        from ..ops import attention
        attention.backward(q, k, v, out, lse, dout, meta.cu_seqlens, meta.max_seqlen,
                           dq=dq, dk=dk, dv=dv)
    else:
        a, b, c_ = F.attention_varlen_bwd(q, k, v, out, lse, dout, meta.cu_seqlens,
                                          meta.max_seqlen)
        dq.copy_(a); dk.copy_(b); dv.copy_(c_)


# ============================================================================ head + loss
class HeadLossStage(Stage):
    """Final RMSNorm, LM head and masked weighted cross-entropy, evaluated in row
    blocks so that the ``[T, V]`` logits never exist at once (the reference's
    chunked head, models/shared/token_head.py:16,63-68). Forward and backward of
    this stage run as one task: the loss gradient is formed while the logits
    block is still on chip, then folded into the head-weight gradient and the
    hidden-state gradient by two GEMMs."""
    kind = "head"

    def __init__(self, name, cfg, block_rows: int = 2048, objective=None, trainable: bool = True):
        super().__init__(name, cfg)
        from .objectives import Objective
        self.block_rows = block_rows
        self.objective = objective or Objective()
        norm_init = "zeros" if cfg.zero_centered_norm else "ones"
        self.params = [ParamSpec("final_norm", (cfg.d_model,), init=norm_init, trainable=trainable)]
        if not cfg.tied_embeddings:
            self.params.append(ParamSpec("head", (cfg.vocab_size, cfg.d_model),
                                         std=cfg.initializer_range, trainable=trainable))

    def workspace_bytes(self, T, itemsize=2):
        c = self.cfg
        return (min(T, self.block_rows) * c.vocab_size + 2 * T * c.d_model) * itemsize

    def flops(self, T, mean_seqlen):
        return 2.0 * T * self.cfg.d_model * self.cfg.vocab_size

    def loss_and_backward(self, P, G, x, meta: BatchMeta, loss_sum: torch.Tensor, first: bool,
                          dx: torch.Tensor | None = None, train: bool = True,
                          grad_scale: float = 1.0, tied: dict | None = None):
        """Adds this microbatch's weighted loss into ``loss_sum`` (fp32[1]); when
        ``train``, accumulates parameter gradients and returns ``dx``. With tied
        embeddings the output matrix is the embedding: ``tied = {"params": embedding
        views, "grads": embedding gradient views or None, "first": bool}`` and the
        head's weight gradient is accumulated into the embedding's."""
        c = self.cfg
        T = x.shape[0]
        if c.tied_embeddings:
            W = tied["params"]["embed"]
            Gw = tied.get("grads")
            Gw = Gw["embed"] if Gw else None
            w_first = bool(tied.get("first", False))
        else:
            W = P["head"]
            Gw = G["head"] if (G and "head" in G) else None
            w_first = first
        h, rstd = F.rmsnorm_fwd(x, P["final_norm"], c.norm_epsilon, c.zero_centered_norm)
        dh = torch.empty_like(h) if train else None
        frozen = not G or "final_norm" not in G
        if train and first and not frozen:
            G["final_norm"].zero_()
        B = self.block_rows
        acc = not w_first
        ob, X = self.objective, meta.extras
        for r0 in range(0, T, B):
            r1 = min(T, r0 + B)
            logits = F.linear_fwd(h[r0:r1], W)
            if ob.kind == "clipped_policy":
                ref = X["reference_logprobs"][r0:r1] if ob.reference_beta > 0 else None
                F.clipped_policy_(logits, meta.targets[r0:r1], meta.weights[r0:r1],
                                  X["old_logprobs"][r0:r1], X["advantages"][r0:r1], loss_sum,
                                  clip=ob.clip_ratio, ref_logp=ref, ref_beta=ob.reference_beta,
                                  grad_scale=grad_scale, write_grad=train)
            else:
                F.cross_entropy_(logits, meta.targets[r0:r1], meta.weights[r0:r1], loss_sum,
                                 grad_scale=grad_scale, write_grad=train)
            if train:
                if Gw is not None:
                    F.linear_wgrad(logits, h[r0:r1], out=Gw, accumulate=acc)
                F.linear_dgrad(logits, W, out=dh[r0:r1])
                acc = True
            del logits
        if not train:
            return None
        dw = G["final_norm"] if not frozen else torch.zeros(c.d_model, dtype=torch.float32,
                                                            device=x.device)
        return F.rmsnorm_bwd(x, P["final_norm"], dh, rstd, dw, c.zero_centered_norm,
                             dx=dx, accumulate=False)

    output_width = 1          # per-row outputs of a forward-only program: log p(target)

    def outputs(self, P, x, meta: BatchMeta, tied: dict | None = None) -> torch.Tensor:
        logp = self.target_logprobs(P, x, meta, tied)
        return logp.masked_fill_(meta.targets < 0, 0.0).reshape(-1, 1)   # no target: reported as 0

    def target_logprobs(self, P, x, meta: BatchMeta, tied: dict | None = None) -> torch.Tensor:
        """log p(target) for every token (fp32 [T]), in the same row blocks."""
        c = self.cfg
        T = x.shape[0]
        if c.tied_embeddings:
            P = dict(P, head=tied["params"]["embed"])
        h, _ = F.rmsnorm_fwd(x, P["final_norm"], c.norm_epsilon, c.zero_centered_norm)
        out = torch.empty(T, dtype=torch.float32, device=x.device)
        for r0 in range(0, T, self.block_rows):
            r1 = min(T, r0 + self.block_rows)
            F.target_logprobs_(F.linear_fwd(h[r0:r1], P["head"]), meta.targets[r0:r1], out[r0:r1])
        return out


# ============================================================================ assembly
def build_stages(cfg: DecoderConfig, objective=None, lora=None,
                 expert_parallel: tuple[int, int] | None = None) -> list[Stage]:
    """``objective`` selects what the head evaluates; ``lora`` adds low-rank adapters to
    every layer (which then run through the autograd-derived layer stage) and freezes
    the embedding, the head and the base matrices unless ``lora.train_base``.
    ``expert_parallel = (ranks, rank)`` gives routed layers this rank's slice of the
    expert banks."""
    if cfg.family == "regression":
        from .regression import build_regression_stages
        if lora is not None or expert_parallel is not None:
            raise ValueError("the regression family has no adapters and no experts")
        return build_regression_stages(cfg)
    base_trainable = lora is None or lora.train_base
    stages: list[Stage] = [EmbeddingStage("embed", cfg, trainable=base_trainable)]
    for i in range(cfg.n_layers):
        kind = cfg.layer_kind(i)
        if kind == "deltanet" or cfg.is_moe or cfg.gated_attention or lora is not None:
            from .hybrid import make_layer
            coef = objective.moe_balance_coef if objective is not None and objective.moe_balance_coef > 0 else None
            stages.append(make_layer(f"layer{i}", cfg, i, lora, coef, expert_parallel))
        else:
            stages.append(DenseLayerStage(f"layer{i}", cfg))
    stages.append(HeadLossStage("head", cfg, objective=objective, trainable=base_trainable))
    return stages
