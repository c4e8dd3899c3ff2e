"""Hybrid and mixture decoder layers: Gated DeltaNet or (gated) GQA attention as the
sequence mixer, a dense SwiGLU MLP or routed experts (plus an optional shared
expert) as the channel mixer.

The forward pass is written once with differentiable ops; ``torch.autograd``
derives the backward pass per stage execution (recompute form: the backward task
re-runs the forward under autograd from the stage input). Matrix weight
gradients are written by the ``linear`` op directly into the stage's gradient
buffer; the few remaining parameters (convolution taps, ``A_log``, ``dt_bias``,
router-free gates) are leaf tensors whose ``.grad`` is folded in afterwards.

Architecture references:
  Gated DeltaNet   packages/workloads/src/shadowspill_workloads/models/shared/delta_net.py:13-89
  gated attention  models/qwen35/implementations/mlops.py:30-100
  routed experts   models/shared/qwen_moe/experts.py:31-72 (router -> top-k -> grouped
                   up/SwiGLU/down -> weighted combine)
"""
from __future__ import annotations

import torch
import torch.nn.functional as TF

from ..ops import sequence as seq_ops
from . import autograd_ops as A
from .config import DecoderConfig
from .decoder import BatchMeta, ParamSpec, Stage


class HybridLayerStage(Stage):
    kind = "layer"
    SAVE_SETS = {"recompute": ()}

    def __init__(self, name: str, cfg: DecoderConfig, index: int, lora=None,
                 expert_parallel: tuple[int, int] | None = None):
        super().__init__(name, cfg)
        self.index = index
        self.lora = lora
        self.ep_world, self.ep_rank = expert_parallel if (expert_parallel and cfg.is_moe) else (1, 0)
        if cfg.is_moe and cfg.n_experts % self.ep_world:
            raise ValueError("n_experts must be divisible by the expert-parallel ranks")
        self.ep_group = None      # bound by the executor: symmetric workspace + barriers
        self.aux_coef = float(cfg.router_aux_coef)   # router balance term; 0 = off
        self._aux: list[torch.Tensor] = []           # this execution's balance term (autograd)
        self.aux_sum: torch.Tensor | None = None     # running sum of applied balance losses
        self.mixer = cfg.layer_kind(index)
        c, std = cfg, cfg.initializer_range
        D, dh, Hq, Hkv = c.d_model, c.head_dim, c.n_heads, c.n_kv_heads
        norm_init = "zeros" if c.zero_centered_norm else "ones"
        P = [ParamSpec("attn_norm", (D,), init=norm_init)]
        if self.mixer == "attention":
            qw = Hq * dh * (2 if c.gated_attention else 1)
            P += [ParamSpec("wq", (qw, D), std=std), ParamSpec("wk", (Hkv * dh, D), std=std),
                  ParamSpec("wv", (Hkv * dh, D), std=std), ParamSpec("wo", (D, Hq * dh), std=std)]
            if c.qk_norm:
                qn, kn = (Hq * dh, Hkv * dh) if c.qk_norm_full_width else (dh, dh)
                P += [ParamSpec("q_norm", (qn,), init=norm_init), ParamSpec("k_norm", (kn,), init=norm_init)]
        else:
            self.key_width = c.dn_qk_heads * c.dn_head_dim
            self.value_width = c.dn_v_heads * c.dn_head_dim
            self.conv_width = 2 * self.key_width + self.value_width
            P += [ParamSpec("w_qkvz", (self.conv_width + self.value_width, D), std=std),
                  ParamSpec("w_ba", (2 * c.dn_v_heads, D), std=std),
                  ParamSpec("conv_w", (self.conv_width, c.dn_conv_width), std=0.3),
                  ParamSpec("A_log", (c.dn_v_heads,), init="zeros", dtype=torch.float32),
                  ParamSpec("dt_bias", (c.dn_v_heads,), init="zeros", dtype=torch.float32),
                  ParamSpec("lin_norm", (c.dn_head_dim,), init=norm_init),
                  ParamSpec("w_out", (D, self.value_width), std=std)]
        P.append(ParamSpec("mlp_norm", (D,), init=norm_init))
        if c.is_moe:
            el = c.n_experts // self.ep_world
            ep = ({} if self.ep_world == 1 else {"expert_lo": self.ep_rank * el})
            g13 = (c.n_experts, 2 * c.d_expert, D) if self.ep_world > 1 else None
            g2 = (c.n_experts, D, c.d_expert) if self.ep_world > 1 else None
            P += [ParamSpec("router", (c.n_experts, D), std=std),
                  ParamSpec("w13", (el, 2 * c.d_expert, D), std=std, global_shape=g13, **ep),
                  ParamSpec("w2", (el, D, c.d_expert), std=std, global_shape=g2, **ep)]
            if c.d_shared_expert:
                P += [ParamSpec("sw13", (2 * c.d_shared_expert, D), std=std),
                      ParamSpec("sw2", (D, c.d_shared_expert), std=std)]
                if c.gated_shared_expert:
                    P.append(ParamSpec("shared_gate", (D,), std=std))
        else:
            P += [ParamSpec("w13", (2 * c.d_ff, D), std=std), ParamSpec("w2", (D, c.d_ff), std=std)]
        self._banks = ["w13", "w2"] if c.is_moe else []
        self._adapted: set[str] = set()
        if lora is not None:
            from dataclasses import replace as _replace
            from .lora import factor_names
            extra = []
            for p in P:
                is_bank = p.name in self._banks
                if p.name not in lora.targets or len(p.shape) < 2 or (is_bank and not lora.routed_experts):
                    continue
                a, b = factor_names(p.name)
                lead = p.shape[:-2]
                extra += [ParamSpec(a, lead + (lora.rank, p.shape[-1]), std=std),
                          ParamSpec(b, lead + (p.shape[-2], lora.rank), init="zeros")]
                self._adapted.add(p.name)
            if not lora.train_base:
                P = [_replace(p, trainable=False) for p in P]
            P += extra
            self._banks += [n for e in extra for n in [e.name] if len(e.shape) == 3]
        self.params = P
        self._leaf = [p.name for p in P if p.name in ("conv_w", "A_log", "dt_bias", "shared_gate")]

    # ---- sizes (used for modelled costs until profiled)
    def workspace_bytes(self, T, itemsize=2):
        c = self.cfg
        width = (c.d_ff or c.top_k * c.d_expert + c.d_shared_expert)
        return T * (8 * c.d_model + 6 * width + 4 * c.n_heads * c.head_dim) * itemsize * 2

    def flops(self, T, mean_seqlen):
        c = self.cfg
        if self.mixer == "attention":
            mix = 2.0 * T * c.d_model * (c.n_heads * c.head_dim * (3 if c.gated_attention else 2)
                                         + 2 * c.n_kv_heads * c.head_dim)
            mix += 4.0 * T * (mean_seqlen / 2.0) * c.n_heads * c.head_dim
        else:
            mix = 2.0 * T * c.d_model * (self.conv_width + 2 * self.value_width)
            mix += 6.0 * T * c.dn_v_heads * c.dn_head_dim * c.dn_head_dim
        ff = 3 * (c.d_ff if not c.is_moe else c.top_k * c.d_expert + c.d_shared_expert)
        return mix + 2.0 * T * c.d_model * ff

    # ---- the layer
    def _lin(self, P, x, name: str, sink):
        """Projection ``name``, with its low-rank adapter when it has one."""
        if name in self._adapted:
            return A.lora_linear(x, P[name], P[f"{name}_lora_a"], P[f"{name}_lora_b"],
                                 self.lora.scale, sink, name)
        return A.linear(x, P[name], sink, name)

    def _attention(self, P, h, meta: BatchMeta, sink):
        c = self.cfg
        T = h.shape[0]
        dh, Hq, Hkv = c.head_dim, c.n_heads, c.n_kv_heads
        qg = self._lin(P, h, "wq", sink)
        q, gate = (qg[:, :Hq * dh], qg[:, Hq * dh:]) if c.gated_attention else (qg, None)
        k = self._lin(P, h, "wk", sink)
        v = self._lin(P, h, "wv", sink)
        if c.qk_norm and c.qk_norm_full_width:
            q = A.rmsnorm(q.contiguous(), P["q_norm"], c.norm_epsilon, c.zero_centered_norm, sink, "q_norm")
            k = A.rmsnorm(k.contiguous(), P["k_norm"], c.norm_epsilon, c.zero_centered_norm, sink, "k_norm")
        elif c.qk_norm:
            q = A.rmsnorm(q.reshape(T * Hq, dh), P["q_norm"], c.norm_epsilon, c.zero_centered_norm,
                          sink, "q_norm").reshape(T, Hq * dh)
            k = A.rmsnorm(k.reshape(T * Hkv, dh), P["k_norm"], c.norm_epsilon, c.zero_centered_norm,
                          sink, "k_norm").reshape(T, Hkv * dh)
        q = A.rope(q.contiguous(), meta.positions, Hq, dh, c.rotary_width, c.rope_base)
        k = A.rope(k.contiguous(), meta.positions, Hkv, dh, c.rotary_width, c.rope_base)
        att = A.attention(q.view(T, Hq, dh), k.view(T, Hkv, dh), v.view(T, Hkv, dh),
                          meta.cu_seqlens, meta.max_seqlen).reshape(T, Hq * dh)
        if gate is not None:
            att = att * torch.sigmoid(gate.float()).to(att.dtype)
        return self._lin(P, att.contiguous(), "wo", sink)

    def _deltanet(self, P, L, h, meta: BatchMeta, sink, bounds):
        c = self.cfg
        T = h.shape[0]
        Hk, Hv, dk = c.dn_qk_heads, c.dn_v_heads, c.dn_head_dim
        qkvz = self._lin(P, h, "w_qkvz", sink)
        ba = A.linear(h, P["w_ba"], sink, "w_ba")
        conv = seq_ops.causal_conv_silu(qkvz[:, :self.conv_width], L["conv_w"], bounds, meta.positions)
        q = seq_ops.l2_normalize(conv[:, :self.key_width].reshape(T, Hk, dk))
        k = seq_ops.l2_normalize(conv[:, self.key_width:2 * self.key_width].reshape(T, Hk, dk))
        v = conv[:, 2 * self.key_width:].reshape(T, Hv, dk)
        beta = torch.sigmoid(ba[:, :Hv].float())
        g = -torch.exp(L["A_log"].float()) * TF.softplus(ba[:, Hv:].float() + L["dt_bias"].float())
        mixed = seq_ops.gated_delta_rule_chunked(q, k, v, beta, g, bounds, c.dn_chunk, meta.cu_seqlens)
        gate = qkvz[:, self.conv_width:].reshape(T, Hv, dk)
        normed = seq_ops.gated_rmsnorm(mixed, gate, P["lin_norm_leaf"], c.norm_epsilon,
                                       c.zero_centered_norm)
        return self._lin(P, normed.reshape(T, Hv * dk).contiguous(), "w_out", sink)

    def _experts(self, P, L, h, sink):
        c = self.cfg
        T = h.shape[0]
        logits = A.linear(h, P["router"], sink, "router").float()
        if self.aux_coef > 0 and sink is not None:
            from .objectives import router_balance
            with torch.no_grad():
                top = torch.topk(logits if c.router_renormalize else torch.softmax(logits, -1),
                                 c.top_k, dim=-1).indices
                counts = torch.bincount(top.reshape(-1), minlength=c.n_experts)
            self._aux.append(router_balance(torch.softmax(logits, -1).sum(0), counts, T, c.top_k))
        routed_lora = bool(self._adapted & {"w13", "w2"})
        if self.ep_world > 1:
            if not h.is_cuda or routed_lora:
                raise NotImplementedError("expert parallelism runs on CUDA without routed adapters")
            if self.ep_group is not None:
                from ..parallel import expert_parallel as ep_ops
                out = ep_ops.experts(h, logits, P["w13"], P["w2"], self.ep_group,
                                     c.router_renormalize, sink)
            else:
                # unbound (task profiling on one rank): the local experts alone, same row count
                from ..ops import moe as moe_ops
                el = c.n_experts // self.ep_world
                lo = self.ep_rank * el
                out = moe_ops.experts(h, logits[:, lo:lo + el].contiguous(), P["w13"], P["w2"],
                                      c.top_k, c.router_renormalize, sink)
            return self._shared(P, L, h, sink, out)
        if h.is_cuda and not routed_lora:
            from ..ops import moe as moe_ops
            out = moe_ops.experts(h, logits, P["w13"], P["w2"], c.top_k, c.router_renormalize, sink)
            return self._shared(P, L, h, sink, out)
        if h.is_cuda:
            return self._shared(P, L, h, sink, self._experts_lora_cuda(P, h, logits, sink))
        if c.router_renormalize:
            vals, ids = torch.topk(logits, c.top_k, dim=-1)
            wts = torch.softmax(vals, dim=-1)
        else:
            probs = torch.softmax(logits, dim=-1)
            wts, ids = torch.topk(probs, c.top_k, dim=-1)
        flat_e = ids.reshape(-1)
        order = torch.argsort(flat_e, stable=True)
        counts = torch.bincount(flat_e, minlength=c.n_experts).tolist()
        tok = (order // c.top_k)
        w_sorted = wts.reshape(-1)[order].to(h.dtype)
        out = torch.zeros_like(h)
        pos = 0
        for e, n in enumerate(counts):
            if n == 0:
                continue
            rows = tok[pos:pos + n]
            xe = h.index_select(0, rows)
            gu = self._expert_lin(P, xe, "w13", e, sink)
            ye = self._expert_lin(P, A.swiglu(gu), "w2", e, sink)
            out = out.index_add(0, rows, ye * w_sorted[pos:pos + n, None])
            pos += n
        return self._shared(P, L, h, sink, out)

    def _expert_lin(self, P, x, name: str, e: int, sink):
        y = A.linear(x, P[name][e], sink, name, e)
        if name in self._adapted:
            a, b = f"{name}_lora_a", f"{name}_lora_b"
            y = y + A.linear(A.linear(x, P[a][e], sink, a, e), P[b][e], sink, b, e) * self.lora.scale
        return y

    def _experts_lora_cuda(self, P, h, logits, sink):
        """Routed experts with per-expert adapters: the same grouped tcgen05 GEMMs, composed
        from differentiable pieces (gather, grouped linear, combine) so that the adapter
        factors train while the banks stay frozen."""
        from ..ops import moe as moe_ops
        c = self.cfg
        ids, _, counts = moe_ops.route(logits.detach(), c.top_k, c.router_renormalize)
        wts = moe_ops._weights_from_logits(logits, ids.long(), c.router_renormalize)
        lay = moe_ops.Layout(ids, counts)
        xs = A.expert_gather(h, lay)

        def bank(x, name):
            y = A.grouped_linear(x, P[name], lay, sink, name)
            if name in self._adapted:
                a, b = f"{name}_lora_a", f"{name}_lora_b"
                low = A.grouped_linear(A.grouped_linear(x, P[a], lay, sink, a), P[b], lay, sink, b)
                y = y + low * self.lora.scale
            return y
        ys = bank(A.swiglu(bank(xs, "w13")), "w2")
        return A.expert_combine(ys, wts.float().contiguous(), lay)

    def _shared(self, P, L, h, sink, out):
        c = self.cfg
        if c.d_shared_expert:
            sh = self._lin(P, A.swiglu(self._lin(P, h, "sw13", sink)), "sw2", sink)
            if c.gated_shared_expert:
                sh = sh * torch.sigmoid(h.float() @ L["shared_gate"].float()).to(h.dtype)[:, None]
            out = out + sh
        return out

    def _layer(self, P, L, x, meta: BatchMeta, sink, bounds):
        c = self.cfg
        h = A.rmsnorm(x, P["attn_norm"], c.norm_epsilon, c.zero_centered_norm, sink, "attn_norm")
        mix = (self._attention(P, h, meta, sink) if self.mixer == "attention"
               else self._deltanet(P, L, h, meta, sink, bounds))
        x = x + mix
        h = A.rmsnorm(x, P["mlp_norm"], c.norm_epsilon, c.zero_centered_norm, sink, "mlp_norm")
        if c.is_moe:
            ff = self._experts(P, L, h, sink)
        else:
            ff = self._lin(P, A.swiglu(self._lin(P, h, "w13", sink)), "w2", sink)
        return x + ff

    def _leaves(self, P, grad: bool):
        """Parameters whose gradient comes from autograd's ``.grad``."""
        L = {n: (P[n].detach().requires_grad_(True) if grad else P[n]) for n in self._leaf}
        P = dict(P)
        if "lin_norm" in P:       # the gated norm is plain differentiable math
            leaf = P["lin_norm"].detach().requires_grad_(True) if grad else P["lin_norm"]
            P["lin_norm_leaf"] = leaf
            L["lin_norm"] = leaf
        return P, L

    # ---- stage interface
    def forward(self, P, x, meta: BatchMeta, keep=(), out=None):
        bounds = meta.cu_seqlens.tolist() if (self.mixer == "deltanet" and not x.is_cuda) else None
        with torch.no_grad(), seq_ops.tf32_matmul():
            P2, L = self._leaves(P, False)
            y = self._layer(P2, L, x, meta, None, bounds)
        if out is not None:
            out.copy_(y)
            y = out
        return y, {}

    def backward(self, P, G, x, dy, meta: BatchMeta, saved, first: bool):
        bounds = meta.cu_seqlens.tolist() if (self.mixer == "deltanet" and not x.is_cuda) else None
        sink = A.GradSink(G, first)
        if first and not x.is_cuda:
            for name in self._banks:          # experts without tokens still need defined gradients
                if name not in G:
                    continue
                G[name].zero_()
                for e in range(self.cfg.n_experts):
                    sink.written.add(f"{name}[{e}]")
        P2, L = self._leaves(P, True)
        xin = x.detach().requires_grad_(True)
        self._aux = []
        tf32 = seq_ops.tf32_matmul()
        tf32.__enter__()                  # also covers the autograd backward below
        with torch.enable_grad():
            y = self._layer(P2, L, xin, meta, sink, bounds)
        if self._aux:
            # the balance term joins the loss with this microbatch's share of the loss weight
            share = meta.weights.sum() * self.aux_coef
            aux = self._aux[0] * share
            if self.aux_sum is None:
                self.aux_sum = torch.zeros(1, dtype=torch.float32, device=x.device)
            self.aux_sum += aux.detach().float()
            torch.autograd.backward([y, aux], [dy, torch.ones_like(aux)])
            self._aux = []
        else:
            torch.autograd.backward(y, dy)
        tf32.__exit__()
        for name, leaf in L.items():
            sink.add_vector(name, leaf.grad if leaf.grad is not None else torch.zeros_like(leaf))
        dy.copy_(xin.grad)
        return dy


def make_layer(name: str, cfg: DecoderConfig, index: int, lora=None, aux_coef: float | None = None,
               expert_parallel: tuple[int, int] | None = None) -> Stage:
    st = HybridLayerStage(name, cfg, index, lora, expert_parallel)
    if aux_coef is not None and cfg.is_moe:
        st.aux_coef = float(aux_coef)
    return st
