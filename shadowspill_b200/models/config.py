"""Model family configurations and the named presets (``<family>-<size>``).

The catalog mirrors the reference's preset table
(packages/workloads/src/shadowspill_workloads/MODELS.md:38-59): same layer counts,
widths, head geometry, expert counts and vocabularies, so a preset name means
the same architecture in both systems.
"""
from __future__ import annotations

from dataclasses import asdict, dataclass, field, replace
from typing import Any


@dataclass(frozen=True)
class DecoderConfig:
    family: str
    n_layers: int
    d_model: int
    n_heads: int
    n_kv_heads: int
    head_dim: int
    d_ff: int
    vocab_size: int
    rope_base: float = 500_000.0
    rotary_fraction: float = 1.0          # Qwen 3.5 rotates a quarter of each head
    norm_epsilon: float = 1e-5
    zero_centered_norm: bool = False      # Qwen 3.5: weight stored as offset from one
    qk_norm: bool = False                 # Qwen 3 family: RMSNorm on each q/k head
    qk_norm_full_width: bool = False      # OLMoE: one RMSNorm over the whole q (and k) projection
    gated_attention: bool = False         # Qwen 3.5: sigmoid output gate on attention
    tied_embeddings: bool = False
    initializer_range: float = 0.02
    # hybrid linear attention (Gated DeltaNet)
    full_attention_interval: int = 0      # every k-th layer is full attention; 0 = all layers
    dn_qk_heads: int = 0
    dn_v_heads: int = 0
    dn_head_dim: int = 128
    dn_conv_width: int = 4
    dn_chunk: int = 64
    # mixture of experts
    n_experts: int = 0
    top_k: int = 0
    d_expert: int = 0
    d_shared_expert: int = 0              # 0 = no shared expert
    gated_shared_expert: bool = False
    router_renormalize: bool = True
    router_aux_coef: float = 0.0
    router_scoring: str = "softmax"       # "sigmoid" (GLM): scores + a selection-only bias, top-k renormalised
    routed_scaling_factor: float = 1.0
    first_dense_layers: int = 0           # GLM: the first k layers have a dense feed-forward
    # sparse multi-head latent attention (GLM 5.3): queries and keys/values through low-rank
    # latents, a frozen indexer that picks index_topk earlier tokens per query
    q_lora_rank: int = 0
    kv_lora_rank: int = 0
    qk_nope_head_dim: int = 0
    qk_rope_head_dim: int = 0
    v_head_dim: int = 0
    index_n_heads: int = 0
    index_head_dim: int = 0
    index_topk: int = 0
    indexer_types: tuple = ()             # per layer "full" (own indexer) or "shared" (reuses the last full one's picks)

    def __post_init__(self) -> None:
        if self.n_heads % self.n_kv_heads:
            raise ValueError("n_heads must be divisible by n_kv_heads")
        if self.router_scoring not in ("softmax", "sigmoid"):
            raise ValueError("router_scoring is 'softmax' or 'sigmoid'")
        if self.kv_lora_rank:
            kinds = tuple(self.indexer_types) or tuple("full" if (i < 3 or i % 4 == 2) else "shared"
                                                       for i in range(self.n_layers))
            if len(kinds) < self.n_layers or kinds[0] != "full" or any(k not in ("full", "shared") for k in kinds):
                raise ValueError("indexer_types must start with 'full' and name every layer 'full' or 'shared'")
            object.__setattr__(self, "indexer_types", tuple(kinds[:self.n_layers]))
            if self.qk_rope_head_dim % 2 or self.index_head_dim < self.qk_rope_head_dim or self.index_topk < 1:
                raise ValueError("sparse latent attention needs an even rope width inside the index width and index_topk >= 1")
        elif self.indexer_types:
            object.__setattr__(self, "indexer_types", tuple(self.indexer_types))
        if self.n_experts and not (0 < self.top_k <= self.n_experts):
            raise ValueError("top_k must be in [1, n_experts]")
        if self.full_attention_interval and not self.dn_v_heads:
            raise ValueError("hybrid models need DeltaNet head counts")

    @property
    def is_moe(self) -> bool:
        return self.n_experts > 0

    @property
    def is_latent_attention(self) -> bool:
        return self.kv_lora_rank > 0

    def layer_is_moe(self, index: int) -> bool:
        return self.is_moe and index >= self.first_dense_layers

    def layer_groups(self) -> list[list[int]]:
        """Layers that must share a stage: a layer whose sparse attention reuses the picks of an
        earlier indexer stays with that indexer's layer, so the picks never cross a stage boundary."""
        if not self.indexer_types:
            return [[i] for i in range(self.n_layers)]
        groups: list[list[int]] = []
        for i, kind in enumerate(self.indexer_types):
            if kind == "full" or not groups:
                groups.append([i])
            else:
                groups[-1].append(i)
        return groups

    @property
    def rotary_width(self) -> int:
        w = int(self.head_dim * self.rotary_fraction)
        return w - (w % 4)

    def layer_kind(self, index: int) -> str:
        """``attention`` or ``deltanet`` for layer ``index``."""
        k = self.full_attention_interval
        if k and (index + 1) % k != 0:
            return "deltanet"
        return "attention"

    def to_json(self) -> dict[str, Any]:
        d = asdict(self)
        d["indexer_types"] = list(self.indexer_types)       # what JSON gives back, so a round trip compares equal
        return d

    @staticmethod
    def from_json(d: dict[str, Any]) -> "DecoderConfig":
        d = dict(d)
        if "indexer_types" in d:
            d["indexer_types"] = tuple(d["indexer_types"] or ())
        return DecoderConfig(**d)

    def parameter_count(self) -> int:
        if self.is_latent_attention:          # defined as a module for the graph frontend only
            import torch
            from ..frontend.modules import DecoderLM
            with torch.device("meta"):
                return sum(p.numel() for p in DecoderLM(self).parameters())
        from .decoder import build_stages
        return sum(s.parameter_count() for s in build_stages(self))


def _llama(n_layers, d, h, kv, ff, vocab=128_256, hd=None, **kw):
    return DecoderConfig("llama3", n_layers, d, h, kv, hd or d // h, ff, vocab, **kw)


def _qwen3(n_layers, d, h, kv, hd, ff, vocab=151_936, **kw):
    return DecoderConfig("qwen3", n_layers, d, h, kv, hd, ff, vocab, rope_base=1_000_000.0,
                         norm_epsilon=1e-6, qk_norm=True, **kw)


def _qwen35(n_layers, d, h, kv, hd, ff, dnk, dnv, vocab=248_320, interval=4, dnhd=128, **kw):
    return DecoderConfig("qwen35", n_layers, d, h, kv, hd, ff, vocab, rope_base=10_000_000.0,
                         rotary_fraction=0.25, norm_epsilon=1e-6, zero_centered_norm=True,
                         qk_norm=True, gated_attention=True, full_attention_interval=interval,
                         dn_qk_heads=dnk, dn_v_heads=dnv, dn_head_dim=dnhd, **kw)


PRESETS: dict[str, DecoderConfig] = {
    # ---- Llama 3: GQA + dense SwiGLU
    "llama3-tiny": _llama(2, 128, 4, 2, 256, vocab=512),
    "llama3-plumbing": _llama(4, 256, 4, 2, 688, vocab=4096, rope_base=10_000.0),
    "llama3-numerical": _llama(12, 2048, 16, 4, 7168),
    "llama3-1b": _llama(16, 2048, 32, 8, 8192),
    "llama3-8b": _llama(32, 4096, 32, 8, 14336),
    # ---- Qwen 3: GQA with q/k norms + dense SwiGLU
    "qwen3-tiny": _qwen3(2, 128, 4, 2, 64, 256, vocab=512),
    "qwen3-1.7b": _qwen3(28, 2048, 16, 8, 128, 6144),
    "qwen3-8b": _qwen3(36, 4096, 32, 8, 128, 12288),
    "qwen3-32b": _qwen3(64, 5120, 64, 8, 128, 25600),
    # ---- Qwen 3.5: 3 Gated DeltaNet : 1 gated full attention
    "qwen35-tiny": _qwen35(2, 128, 4, 2, 32, 256, 2, 4, vocab=512, interval=2, dnhd=32),
    "qwen35-numerical": _qwen35(8, 1536, 12, 4, 128, 4608, 6, 12),
    "qwen35-2b": _qwen35(24, 2048, 8, 2, 256, 6144, 16, 16, tied_embeddings=True),
    "qwen35-9b": _qwen35(32, 4096, 16, 4, 256, 12288, 16, 32),
    "qwen35-27b": _qwen35(64, 5120, 24, 4, 256, 17408, 16, 48),
    # ---- OLMoE: GQA + routed SwiGLU experts
    "olmoe-tiny": DecoderConfig("olmoe", 2, 128, 4, 2, 32, 0, 512, rope_base=10_000.0,
                                qk_norm=True, qk_norm_full_width=True, n_experts=8, top_k=2,
                                d_expert=128, router_renormalize=False),
    "olmoe-numerical": DecoderConfig("olmoe", 16, 1024, 8, 8, 128, 0, 50_304, rope_base=10_000.0,
                                     qk_norm=True, qk_norm_full_width=True, n_experts=16, top_k=4,
                                     d_expert=1024, router_renormalize=False),
    "olmoe-7b-a1b": DecoderConfig("olmoe", 16, 2048, 16, 16, 128, 0, 50_304, rope_base=10_000.0,
                                  qk_norm=True, qk_norm_full_width=True, n_experts=64, top_k=8,
                                  d_expert=1024, router_renormalize=False),
    # ---- Qwen 3 MoE
    "qwen3moe-tiny": DecoderConfig("qwen3moe", 2, 128, 4, 2, 32, 0, 1024, rope_base=1_000_000.0,
                                   norm_epsilon=1e-6, qk_norm=True, n_experts=8, top_k=2,
                                   d_expert=128),
    "qwen3moe-30b-a3b": DecoderConfig("qwen3moe", 48, 2048, 32, 4, 128, 0, 151_936,
                                      rope_base=1_000_000.0, norm_epsilon=1e-6, qk_norm=True,
                                      n_experts=128, top_k=8, d_expert=768),
    # ---- Qwen 3.5 MoE: hybrid attention, routed + gated shared expert
    "qwen35moe-tiny": replace(_qwen35(2, 128, 4, 2, 32, 0, 2, 4, vocab=1024, interval=2, dnhd=32),
                              family="qwen35moe", n_experts=8, top_k=2, d_expert=128,
                              d_shared_expert=128, gated_shared_expert=True),
    "qwen35moe-35b-a3b": replace(_qwen35(40, 2048, 16, 2, 256, 0, 16, 32), family="qwen35moe",
                                 n_experts=256, top_k=8, d_expert=512, d_shared_expert=512,
                                 gated_shared_expert=True),
    # ---- GLM 5.3: sparse multi-head latent attention + sigmoid-scored routed experts
    # (published shape: packages/workloads/src/shadowspill_workloads/models/glm53/config.py:10-43)
    "glm53-tiny": DecoderConfig("glm53", 4, 128, 16, 16, 96, 128, 128, rope_base=8_000_000.0,
                                first_dense_layers=1, n_experts=4, top_k=2, d_expert=128, d_shared_expert=128,
                                router_scoring="sigmoid", routed_scaling_factor=2.5, q_lora_rank=32,
                                kv_lora_rank=64, qk_nope_head_dim=32, qk_rope_head_dim=64, v_head_dim=32,
                                index_n_heads=2, index_head_dim=64, index_topk=8,
                                indexer_types=("full", "shared", "full", "shared")),
    "glm53-published": DecoderConfig("glm53", 78, 6144, 64, 64, 256, 12288, 154_880, rope_base=8_000_000.0,
                                     first_dense_layers=3, n_experts=256, top_k=8, d_expert=2048,
                                     d_shared_expert=2048, router_scoring="sigmoid", routed_scaling_factor=2.5,
                                     q_lora_rank=2048, kv_lora_rank=512, qk_nope_head_dim=192,
                                     qk_rope_head_dim=64, v_head_dim=256, index_n_heads=32, index_head_dim=128,
                                     index_topk=2048),
    # ---- the small non-text model: Linear(16, 32) -> SiLU -> Linear(32, 8), fp32
    # (d_ff = input width, d_model = hidden width, vocab_size = output width; models/regression.py)
    "regression": DecoderConfig("regression", 0, 32, 1, 1, 1, 16, 8, initializer_range=0.25),
}


def preset(name: str) -> DecoderConfig:
    try:
        return PRESETS[name]
    except KeyError:
        raise KeyError(f"unknown model preset {name!r}; known: {sorted(PRESETS)}") from None
