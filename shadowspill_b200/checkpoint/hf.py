"""Hugging Face weight names <-> this framework's stage parameters.

``to_hf(cfg, state)`` turns ``{"<stage>.<param>": tensor}`` into a Hugging Face style
state dict and ``from_hf`` is the inverse; that is how pretrained weights enter a run.
``save_hf`` / ``load_hf`` read and write ``model.safetensors`` plus a ``config.json``
with the architecture fields. Rotary tables are computed, not stored, and the
rotate-half convention matches, so no projection is permuted.

Every parameter has one *source*: a checkpoint tensor as it is, several tensors joined
on dimension 0 (fused ``qkv`` / ``gate|up`` projections), per-expert matrices stacked
into a bank, or a per-head de-interleave. The Qwen 3.5 families differ in four ways
(reference: packages/workloads/src/shadowspill_workloads/models/qwen35/checkpoint.py:1-80,
models/qwen35moe/checkpoint.py:1-60, models/llama3/checkpoint.py:20-55):

* their text decoder's keys begin ``model.language_model.`` (the checkpoint is the
  vision-language model; vision tower and multi-token-prediction head are skipped);
* a full-attention block's ``q_proj`` carries the attention gate interleaved per head
  (``[q_h, gate_h]`` for each head); this framework keeps all queries, then all gates;
* a linear-attention block's ``w_qkvz`` is ``in_proj_qkv`` then ``in_proj_z``, ``w_ba``
  is ``in_proj_b`` then ``in_proj_a``; ``conv1d.weight`` has a singleton middle axis;
* the mixture family stores routed experts as fused banks ``mlp.experts.gate_up_proj``
  ``[E, 2I, H]`` / ``mlp.experts.down_proj`` ``[E, H, I]`` and a shared expert with its
  own sigmoid gate.
"""
from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path
from typing import Callable

import torch

from ..models.config import DecoderConfig
from ..models.decoder import DenseLayerStage, build_stages

_ARCH = {"llama3": "LlamaForCausalLM", "qwen3": "Qwen3ForCausalLM", "olmoe": "OlmoeForCausalLM",
         "qwen3moe": "Qwen3MoeForCausalLM", "qwen35": "Qwen3_5ForConditionalGeneration",
         "qwen35moe": "Qwen3_5MoeForConditionalGeneration", "glm53": "GlmMoeDsaForCausalLM"}
_IGNORED_PREFIXES = ("model.visual.", "mtp.")


def supported(cfg: DecoderConfig) -> bool:
    return cfg.family in _ARCH


def _prefix(cfg: DecoderConfig) -> str:
    return "model.language_model." if cfg.family in ("qwen35", "qwen35moe") else "model."


@dataclass
class Source:
    """Where one framework parameter comes from: ``names`` in the checkpoint, ``load`` joins
    them into the parameter, ``store`` cuts the parameter back into those tensors."""
    names: tuple[str, ...]
    load: Callable[[list[torch.Tensor]], torch.Tensor]
    store: Callable[[torch.Tensor], list[torch.Tensor]]


def _tensor(name: str) -> Source:
    return Source((name,), lambda ts: ts[0], lambda p: [p])


def _reshaped(name: str, stored: tuple[int, ...], ours: tuple[int, ...]) -> Source:
    return Source((name,), lambda ts: ts[0].reshape(ours), lambda p: [p.reshape(stored)])


def _joined(names: tuple[str, ...], rows: tuple[int, ...]) -> Source:
    return Source(names, lambda ts: torch.cat(ts, 0), lambda p: list(p.split(list(rows), dim=0)))


def _deinterleaved(name: str, heads: int, head_dim: int) -> Source:
    """Checkpoint rows ``[q_0, g_0, q_1, g_1, ...]`` (blocks of ``head_dim``) <-> all q, all g."""
    def load(ts):
        w = ts[0]
        w = w.reshape(heads, 2, head_dim, w.shape[-1])
        return torch.cat([w[:, 0].reshape(heads * head_dim, -1), w[:, 1].reshape(heads * head_dim, -1)], 0)

    def store(p):
        q, g = p.split(heads * head_dim, dim=0)
        w = torch.stack([q.reshape(heads, head_dim, -1), g.reshape(heads, head_dim, -1)], 1)
        return [w.reshape(2 * heads * head_dim, -1)]
    return Source((name,), load, store)


def _expert_bank(fmt: tuple[str, ...], n_experts: int, rows: tuple[int, ...]) -> Source:
    """Per-expert matrices (``fmt`` formatted with the expert index, joined on dim 0) stacked."""
    names = tuple(f.format(e=e) for e in range(n_experts) for f in fmt)
    k = len(fmt)

    def load(ts):
        return torch.stack([torch.cat(ts[e * k:(e + 1) * k], 0) for e in range(n_experts)])

    def store(p):
        out = []
        for e in range(n_experts):
            out += list(p[e].split(list(rows), dim=0))
        return out
    return Source(names, load, store)


def _layer_sources(cfg: DecoderConfig, i: int, stage) -> dict[str, Source]:
    pre = f"{_prefix(cfg)}layers.{i}."
    dh, Hq, Hkv, D = cfg.head_dim, cfg.n_heads, cfg.n_kv_heads, cfg.d_model
    S = {"attn_norm": _tensor(pre + "input_layernorm.weight"),
         "mlp_norm": _tensor(pre + "post_attention_layernorm.weight")}
    if cfg.layer_kind(i) == "attention":
        a = pre + "self_attn."
        S["wo"] = _tensor(a + "o_proj.weight")
        if isinstance(stage, DenseLayerStage):
            S["wqkv"] = _joined((a + "q_proj.weight", a + "k_proj.weight", a + "v_proj.weight"),
                                (Hq * dh, Hkv * dh, Hkv * dh))
        else:
            S["wq"] = (_deinterleaved(a + "q_proj.weight", Hq, dh) if cfg.gated_attention
                       else _tensor(a + "q_proj.weight"))
            S["wk"], S["wv"] = _tensor(a + "k_proj.weight"), _tensor(a + "v_proj.weight")
        if cfg.qk_norm:
            S["q_norm"], S["k_norm"] = _tensor(a + "q_norm.weight"), _tensor(a + "k_norm.weight")
    else:
        la = pre + "linear_attn."
        kw = cfg.dn_qk_heads * cfg.dn_head_dim
        vw = cfg.dn_v_heads * cfg.dn_head_dim
        conv = 2 * kw + vw
        S["w_qkvz"] = _joined((la + "in_proj_qkv.weight", la + "in_proj_z.weight"), (conv, vw))
        S["w_ba"] = _joined((la + "in_proj_b.weight", la + "in_proj_a.weight"),
                            (cfg.dn_v_heads, cfg.dn_v_heads))
        S["conv_w"] = _reshaped(la + "conv1d.weight", (conv, 1, cfg.dn_conv_width),
                                (conv, cfg.dn_conv_width))
        S["A_log"], S["dt_bias"] = _tensor(la + "A_log"), _tensor(la + "dt_bias")
        S["lin_norm"] = _tensor(la + "norm.weight")
        S["w_out"] = _tensor(la + "out_proj.weight")
    m = pre + "mlp."
    if cfg.is_moe:
        S["router"] = _tensor(m + "gate.weight")
        F = cfg.d_expert
        if cfg.family == "qwen35moe":
            S["w13"], S["w2"] = _tensor(m + "experts.gate_up_proj"), _tensor(m + "experts.down_proj")
        else:
            S["w13"] = _expert_bank((m + "experts.{e}.gate_proj.weight", m + "experts.{e}.up_proj.weight"),
                                    cfg.n_experts, (F, F))
            S["w2"] = _expert_bank((m + "experts.{e}.down_proj.weight",), cfg.n_experts, (D,))
        if cfg.d_shared_expert:
            Fs = cfg.d_shared_expert
            S["sw13"] = _joined((m + "shared_expert.gate_proj.weight", m + "shared_expert.up_proj.weight"),
                                (Fs, Fs))
            S["sw2"] = _tensor(m + "shared_expert.down_proj.weight")
            S["shared_gate"] = _reshaped(m + "shared_expert_gate.weight", (1, D), (D,))
    else:
        S["w13"] = _joined((m + "gate_proj.weight", m + "up_proj.weight"), (cfg.d_ff, cfg.d_ff))
        S["w2"] = _tensor(m + "down_proj.weight")
    return S


def _latent_layer_sources(cfg: DecoderConfig, i: int) -> dict[str, Source]:
    """GLM 5.3 (``glm_moe_dsa``) names of layer ``i`` (the reference's naming:
    packages/workloads/src/shadowspill_workloads/models/glm53/weights.py:3-9)."""
    pre = f"model.layers.{i}."
    a, ix, m = pre + "self_attn.", pre + "self_attn.indexer.", pre + "mlp."
    S = {"attn_norm": _tensor(pre + "input_layernorm.weight"),
         "mlp_norm": _tensor(pre + "post_attention_layernorm.weight"),
         "q_a": _tensor(a + "q_a_proj.weight"), "q_a_norm": _tensor(a + "q_a_layernorm.weight"),
         "q_b": _tensor(a + "q_b_proj.weight"), "kv_a": _tensor(a + "kv_a_proj_with_mqa.weight"),
         "kv_a_norm": _tensor(a + "kv_a_layernorm.weight"), "kv_b": _tensor(a + "kv_b_proj.weight"),
         "wo": _tensor(a + "o_proj.weight"),
         "ix_q": _tensor(ix + "wq_b.weight"), "ix_k": _tensor(ix + "wk.weight"),
         "ix_k_norm": _tensor(ix + "k_norm.weight"), "ix_k_bias": _tensor(ix + "k_norm.bias"),
         "ix_w": _tensor(ix + "weights_proj.weight")}
    if cfg.layer_is_moe(i):
        F, D = cfg.d_expert, cfg.d_model
        S["router"] = _tensor(m + "gate.weight")
        S["router_bias"] = _tensor(m + "gate.e_score_correction_bias")
        S["w13"] = _expert_bank((m + "experts.{e}.gate_proj.weight", m + "experts.{e}.up_proj.weight"),
                                cfg.n_experts, (F, F))
        S["w2"] = _expert_bank((m + "experts.{e}.down_proj.weight",), cfg.n_experts, (D,))
        if cfg.d_shared_expert:
            Fs = cfg.d_shared_expert
            S["sw13"] = _joined((m + "shared_experts.gate_proj.weight", m + "shared_experts.up_proj.weight"), (Fs, Fs))
            S["sw2"] = _tensor(m + "shared_experts.down_proj.weight")
    else:
        S["w13"] = _joined((m + "gate_proj.weight", m + "up_proj.weight"), (cfg.d_ff, cfg.d_ff))
        S["w2"] = _tensor(m + "down_proj.weight")
    return S


def _latent_sources(cfg: DecoderConfig, stages) -> dict[str, Source]:
    """The family is exported in stages of several layers: a stage parameter is traced back to its
    layer through the module path the export recorded for it (``layers.<group>.members.<j>.<name>``)."""
    if stages is None:
        from ..frontend.graph_stage import build_graph_stages
        stages = build_graph_stages(cfg, 256, 16)
    groups = cfg.layer_groups()
    out = {"embed.embed": _tensor("model.embed_tokens.weight"), "head.final_norm": _tensor("model.norm.weight"),
           "head.head": _tensor("lm_head.weight")}
    for st in stages[1:-1]:
        for local, target in zip(st.graph.param_names, st.graph.param_targets):
            parts = target.split(".")                    # layers, g, members, j, name
            layer = groups[int(parts[1])][int(parts[3])]
            out[f"{st.name}.{local}"] = _latent_layer_sources(cfg, layer)[parts[4]]
    return out


def parameter_sources(cfg: DecoderConfig, stages=None) -> dict[str, Source]:
    """``{"<stage>.<param>": Source}`` for every base (non-adapter) parameter of the model."""
    if not supported(cfg):
        raise ValueError(f"no Hugging Face mapping for family {cfg.family!r}")
    if cfg.is_latent_attention:
        return _latent_sources(cfg, stages)
    stages = stages or build_stages(cfg)
    pre = _prefix(cfg)
    out = {"embed.embed": _tensor(pre + "embed_tokens.weight"),
           "head.final_norm": _tensor(pre + "norm.weight")}
    if not cfg.tied_embeddings:
        out["head.head"] = _tensor("lm_head.weight")
    for i in range(cfg.n_layers):
        st = stages[i + 1]
        S = _layer_sources(cfg, i, st)
        for p in st.params:
            if "_lora_" in p.name:
                continue                  # adapters are not part of a base checkpoint
            if p.name not in S:
                raise KeyError(f"{st.name}.{p.name} has no Hugging Face source")
            out[f"{st.name}.{p.name}"] = S[p.name]
    return out


def to_hf(cfg: DecoderConfig, state: dict[str, torch.Tensor], stages=None) -> dict[str, torch.Tensor]:
    """``stages``: the run's own stage list when it differs from the default build (adapters
    switch dense layers to separate q/k/v projections); adapter factors are not exported."""
    out: dict[str, torch.Tensor] = {}
    for name, src in parameter_sources(cfg, stages).items():
        for hf_name, t in zip(src.names, src.store(state[name])):
            out[hf_name] = t.contiguous()
    return out


def from_hf(cfg: DecoderConfig, hf: dict[str, torch.Tensor], stages=None) -> dict[str, torch.Tensor]:
    if stages is None and cfg.is_latent_attention:
        from ..frontend.graph_stage import build_graph_stages
        stages = build_graph_stages(cfg, 256, 16)
    stages = stages or build_stages(cfg)
    shapes = {f"{st.name}.{p.name}": tuple(p.shape) for st in stages for p in st.params}
    out: dict[str, torch.Tensor] = {}
    used: set[str] = set()
    for name, src in parameter_sources(cfg, stages).items():
        names = src.names
        if name == "head.head" and "lm_head.weight" not in hf:
            names = (_prefix(cfg) + "embed_tokens.weight",)      # exported with shared matrices
        missing = [n for n in names if n not in hf]
        if missing:
            raise KeyError(f"{name}: checkpoint has no {missing[0]!r}")
        t = src.load([hf[n] for n in names])
        if tuple(t.shape) != shapes[name]:
            raise ValueError(f"{name}: checkpoint shape {tuple(t.shape)} != {shapes[name]}")
        out[name] = t
        used.update(names)
    extra = [k for k in hf if k not in used and not k.startswith(_IGNORED_PREFIXES)
             and not (cfg.tied_embeddings and k == "lm_head.weight")]
    if extra:
        raise ValueError(f"checkpoint tensors with no destination: {sorted(extra)[:4]}")
    return out


def hf_config(cfg: DecoderConfig) -> dict:
    d = {"architectures": [_ARCH.get(cfg.family, cfg.family)], "hidden_size": cfg.d_model,
         "num_hidden_layers": cfg.n_layers, "num_attention_heads": cfg.n_heads,
         "num_key_value_heads": cfg.n_kv_heads, "head_dim": cfg.head_dim,
         "intermediate_size": cfg.d_ff or cfg.d_expert, "vocab_size": cfg.vocab_size,
         "rope_theta": cfg.rope_base, "rms_norm_eps": cfg.norm_epsilon,
         "tie_word_embeddings": cfg.tied_embeddings, "torch_dtype": "bfloat16"}
    if cfg.is_moe:
        d.update(num_experts=cfg.n_experts, num_experts_per_tok=cfg.top_k,
                 moe_intermediate_size=cfg.d_expert, norm_topk_prob=cfg.router_renormalize)
        if cfg.d_shared_expert:
            d["shared_expert_intermediate_size"] = cfg.d_shared_expert
    if cfg.is_latent_attention:
        d.update(model_type="glm_moe_dsa", q_lora_rank=cfg.q_lora_rank, kv_lora_rank=cfg.kv_lora_rank,
                 qk_nope_head_dim=cfg.qk_nope_head_dim, qk_rope_head_dim=cfg.qk_rope_head_dim,
                 v_head_dim=cfg.v_head_dim, index_n_heads=cfg.index_n_heads, index_head_dim=cfg.index_head_dim,
                 index_topk=cfg.index_topk, indexer_types=list(cfg.indexer_types),
                 first_k_dense_replace=cfg.first_dense_layers, intermediate_size=cfg.d_ff,
                 n_routed_experts=cfg.n_experts, n_shared_experts=1 if cfg.d_shared_expert else 0,
                 routed_scaling_factor=cfg.routed_scaling_factor, scoring_func="sigmoid", topk_method="noaux_tc",
                 rope_parameters={"rope_type": "default", "rope_theta": cfg.rope_base})
    if cfg.full_attention_interval:
        d.update(full_attention_interval=cfg.full_attention_interval,
                 layer_types=["full_attention" if cfg.layer_kind(i) == "attention" else "linear_attention"
                              for i in range(cfg.n_layers)],
                 linear_num_key_heads=cfg.dn_qk_heads, linear_num_value_heads=cfg.dn_v_heads,
                 linear_key_head_dim=cfg.dn_head_dim, linear_value_head_dim=cfg.dn_head_dim,
                 linear_conv_kernel_dim=cfg.dn_conv_width)
    return d


def save_hf(cfg: DecoderConfig, state: dict[str, torch.Tensor], directory: str | Path, stages=None) -> Path:
    from safetensors.torch import save_file
    d = Path(directory)
    d.mkdir(parents=True, exist_ok=True)
    save_file({k: v.detach().cpu().contiguous() for k, v in to_hf(cfg, state, stages).items()},
              str(d / "model.safetensors"), metadata={"format": "pt"})
    (d / "config.json").write_text(json.dumps(hf_config(cfg), indent=1))
    return d


def load_hf(cfg: DecoderConfig, directory: str | Path, stages=None) -> dict[str, torch.Tensor]:
    from safetensors.torch import load_file
    d = Path(directory)
    files = sorted(d.glob("*.safetensors"))
    if not files:
        raise FileNotFoundError(f"no .safetensors file in {d}")
    hf: dict[str, torch.Tensor] = {}
    for f in files:
        hf.update(load_file(str(f)))
    return from_hf(cfg, hf, stages)


def stream_hf(cfg: DecoderConfig, directory: str | Path, stages=None):
    """Bounded loading: yields ``(stage name, {"<stage>.<param>": tensor})`` one stage at a time,
    reading only that stage's tensors from the ``*.safetensors`` files (memory-mapped, any number
    of shards), so that a checkpoint far larger than host memory's free part loads with one stage
    resident. The same checks as ``from_hf``: a missing source tensor, a shape that differs and a
    checkpoint tensor without a destination are errors (vision towers and extra prediction heads
    are skipped). Reference: the bounded checkpoint loading of the reference's initialisation
    (packages/workloads/src/shadowspill_workloads/initialization/: safetensors ranges, local files)."""
    from safetensors import safe_open
    d = Path(directory)
    files = sorted(d.glob("*.safetensors"))
    if not files:
        raise FileNotFoundError(f"no .safetensors file in {d}")
    if stages is None and cfg.is_latent_attention:
        from ..frontend.graph_stage import build_graph_stages
        stages = build_graph_stages(cfg, 256, 16)
    stages = stages or build_stages(cfg)
    where: dict[str, Path] = {}
    for f in files:
        with safe_open(str(f), framework="pt") as handle:
            for key in handle.keys():
                where[key] = f
    sources = parameter_sources(cfg, stages)
    used: set[str] = set()
    shapes = {f"{st.name}.{p.name}": tuple(p.shape) for st in stages for p in st.params}
    for st in stages:
        part: dict[str, torch.Tensor] = {}
        opened: dict[Path, object] = {}
        try:
            for p in st.params:
                name = f"{st.name}.{p.name}"
                src = sources.get(name)
                if src is None:
                    continue                            # adapters: not part of a base checkpoint
                names = src.names
                if name == "head.head" and "lm_head.weight" not in where:
                    names = (_prefix(cfg) + "embed_tokens.weight",)
                missing = [n for n in names if n not in where]
                if missing:
                    raise KeyError(f"{name}: checkpoint has no {missing[0]!r}")
                tensors = []
                for n in names:
                    f = where[n]
                    if f not in opened:
                        opened[f] = safe_open(str(f), framework="pt").__enter__()
                    tensors.append(opened[f].get_tensor(n))
                t = src.load(tensors)
                if tuple(t.shape) != shapes[name]:
                    raise ValueError(f"{name}: checkpoint shape {tuple(t.shape)} != {shapes[name]}")
                part[name] = t
                used.update(names)
        finally:
            for handle in opened.values():
                handle.__exit__(None, None, None)
        yield st.name, part
    extra = [k for k in where if k not in used and not k.startswith(_IGNORED_PREFIXES)
             and not (cfg.tied_embeddings and k == "lm_head.weight")]
    if extra:
        raise ValueError(f"checkpoint tensors with no destination: {sorted(extra)[:4]}")
