"""Hugging Face weight names <-> this framework's stage parameters.

``to_hf(cfg, state)`` turns ``{"<stage>.<param>": tensor}`` into a Hugging Face style
state dict (fused projections are cut back into ``q_proj / k_proj / v_proj`` and
``gate_proj / up_proj``; expert banks into per-expert matrices); ``from_hf`` is the
inverse and is how pretrained weights enter a run. ``save_hf`` / ``load_hf`` read and
write ``model.safetensors`` plus a ``config.json`` with the architecture fields.
Rotary tables are computed, not stored, and the rotate-half convention matches, so no
projection is permuted (as in the reference's per-family ``checkpoint.py``, e.g.
packages/workloads/src/shadowspill_workloads/models/llama3/checkpoint.py:20-55).

Covered: llama3, qwen3 (dense layers), olmoe / qwen3moe (routed layers). The Gated
DeltaNet families keep this framework's own names on export (their Hugging Face
layout interleaves projections per head group; not mapped yet).
"""
from __future__ import annotations

import json
from pathlib import Path

import torch

from ..models.config import DecoderConfig
from ..models.decoder import DenseLayerStage, build_stages

_ARCH = {"llama3": "LlamaForCausalLM", "qwen3": "Qwen3ForCausalLM", "olmoe": "OlmoeForCausalLM",
         "qwen3moe": "Qwen3MoeForCausalLM"}


def supported(cfg: DecoderConfig) -> bool:
    return cfg.family in _ARCH and not cfg.tied_embeddings


def _layer_to_hf(cfg: DecoderConfig, i: int, dense: bool, P: dict[str, torch.Tensor]) -> dict:
    pre = f"model.layers.{i}."
    dh, Hq, Hkv = cfg.head_dim, cfg.n_heads, cfg.n_kv_heads
    out = {pre + "input_layernorm.weight": P["attn_norm"],
           pre + "post_attention_layernorm.weight": P["mlp_norm"],
           pre + "self_attn.o_proj.weight": P["wo"]}
    if dense:
        q, k, v = P["wqkv"].split([Hq * dh, Hkv * dh, Hkv * dh], dim=0)
    else:
        q, k, v = P["wq"], P["wk"], P["wv"]
    out[pre + "self_attn.q_proj.weight"] = q
    out[pre + "self_attn.k_proj.weight"] = k
    out[pre + "self_attn.v_proj.weight"] = v
    if cfg.qk_norm:
        out[pre + "self_attn.q_norm.weight"] = P["q_norm"]
        out[pre + "self_attn.k_norm.weight"] = P["k_norm"]
    if cfg.is_moe:
        out[pre + "mlp.gate.weight"] = P["router"]
        F = cfg.d_expert
        for e in range(cfg.n_experts):
            ep = f"{pre}mlp.experts.{e}."
            out[ep + "gate_proj.weight"] = P["w13"][e, :F]
            out[ep + "up_proj.weight"] = P["w13"][e, F:]
            out[ep + "down_proj.weight"] = P["w2"][e]
    else:
        F = cfg.d_ff
        out[pre + "mlp.gate_proj.weight"] = P["w13"][:F]
        out[pre + "mlp.up_proj.weight"] = P["w13"][F:]
        out[pre + "mlp.down_proj.weight"] = P["w2"]
    return out


def to_hf(cfg: DecoderConfig, state: dict[str, torch.Tensor], stages=None) -> dict[str, torch.Tensor]:
    """``stages``: the run's own stage list when it differs from the default build (adapters
    switch dense layers to separate q/k/v projections); adapter factors are not exported."""
    if not supported(cfg):
        raise ValueError(f"no Hugging Face mapping for family {cfg.family!r}")
    stages = stages or build_stages(cfg)
    out = {"model.embed_tokens.weight": state["embed.embed"],
           "model.norm.weight": state["head.final_norm"], "lm_head.weight": state["head.head"]}
    for i in range(cfg.n_layers):
        st = stages[i + 1]
        P = {p.name: state[f"{st.name}.{p.name}"] for p in st.params if "_lora_" not in p.name}
        out.update(_layer_to_hf(cfg, i, isinstance(st, DenseLayerStage), P))
    return {k: v.contiguous() for k, v in out.items()}


def from_hf(cfg: DecoderConfig, hf: dict[str, torch.Tensor], stages=None) -> dict[str, torch.Tensor]:
    if not supported(cfg):
        raise ValueError(f"no Hugging Face mapping for family {cfg.family!r}")
    stages = stages or build_stages(cfg)
    head = hf.get("lm_head.weight", hf["model.embed_tokens.weight"])
    out = {"embed.embed": hf["model.embed_tokens.weight"], "head.final_norm": hf["model.norm.weight"],
           "head.head": head}
    for i in range(cfg.n_layers):
        st = stages[i + 1]
        pre = f"model.layers.{i}."
        g = lambda name: hf[pre + name]
        P = {"attn_norm": g("input_layernorm.weight"), "mlp_norm": g("post_attention_layernorm.weight"),
             "wo": g("self_attn.o_proj.weight")}
        q, k, v = (g(f"self_attn.{n}_proj.weight") for n in "qkv")
        if isinstance(st, DenseLayerStage):
            P["wqkv"] = torch.cat([q, k, v], 0)
        else:
            P["wq"], P["wk"], P["wv"] = q, k, v
        if cfg.qk_norm:
            P["q_norm"], P["k_norm"] = g("self_attn.q_norm.weight"), g("self_attn.k_norm.weight")
        if cfg.is_moe:
            P["router"] = g("mlp.gate.weight")
            P["w13"] = torch.stack([torch.cat([g(f"mlp.experts.{e}.gate_proj.weight"),
                                               g(f"mlp.experts.{e}.up_proj.weight")], 0)
                                    for e in range(cfg.n_experts)])
            P["w2"] = torch.stack([g(f"mlp.experts.{e}.down_proj.weight") for e in range(cfg.n_experts)])
        else:
            P["w13"] = torch.cat([g("mlp.gate_proj.weight"), g("mlp.up_proj.weight")], 0)
            P["w2"] = g("mlp.down_proj.weight")
        for p in st.params:
            if "_lora_" in p.name:
                continue                  # adapters are not part of a base checkpoint
            if p.name not in P:
                raise KeyError(f"{st.name}.{p.name} has no Hugging Face source")
            if tuple(P[p.name].shape) != tuple(p.shape):
                raise ValueError(f"{st.name}.{p.name}: checkpoint shape {tuple(P[p.name].shape)} != {p.shape}")
            out[f"{st.name}.{p.name}"] = P[p.name]
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
