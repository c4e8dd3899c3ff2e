"""Component registry: models, objectives, optimizers, preparations and policies
under versioned ids, plus the built-in components and the resolution of a
client's settings into per-rank worker setups.

Reference: packages/engine/src/shadowspill/training/components/{registry.py,
contracts.py:48-199} and training/preparation/setup.py (``resolve_training``).
"""
from __future__ import annotations

import dataclasses
import hashlib
import inspect
from dataclasses import dataclass, field
from typing import Any, Callable

from ..models.config import PRESETS, DecoderConfig, preset

GIB = 1 << 30


@dataclass(frozen=True)
class ComponentSource:
    distribution: str
    version: str
    sha256: str

    @staticmethod
    def of(obj) -> "ComponentSource":
        try:
            src = inspect.getsource(obj)
        except (OSError, TypeError):
            src = repr(obj)
        from .. import __version__
        return ComponentSource("shadowspill_b200", __version__, hashlib.sha256(src.encode()).hexdigest())


@dataclass
class Component:
    id: str
    kind: str
    create: Callable[..., Any]
    source: ComponentSource
    config_schema: dict[str, Any] = field(default_factory=dict)
    capabilities: tuple[str, ...] = ()


class Registry:
    KINDS = ("model", "objective", "optimizer", "preparation", "policy")

    def __init__(self):
        self._items: dict[tuple[str, str], Component] = {}

    def _add(self, kind: str, id_: str, create, **kw) -> Component:
        if "@" not in id_:
            raise ValueError("component ids are versioned: name@version")
        if (kind, id_) in self._items:
            raise ValueError(f"{kind} {id_!r} is already registered")
        c = Component(id_, kind, create, ComponentSource.of(create), **kw)
        self._items[(kind, id_)] = c
        return c

    def add_model(self, id_, create, **kw): return self._add("model", id_, create, **kw)
    def add_objective(self, id_, create, **kw): return self._add("objective", id_, create, **kw)
    def add_optimizer(self, id_, create, **kw): return self._add("optimizer", id_, create, **kw)
    def add_preparation(self, id_, create, **kw): return self._add("preparation", id_, create, **kw)
    def add_policy(self, id_, create, **kw): return self._add("policy", id_, create, **kw)

    def get(self, kind: str, id_: str) -> Component:
        try:
            return self._items[(kind, id_)]
        except KeyError:
            known = sorted(i for k, i in self._items if k == kind)
            raise KeyError(f"no {kind} component {id_!r}; known: {known}") from None

    def list(self, kind: str | None = None) -> list[dict[str, Any]]:
        return [{"id": c.id, "kind": c.kind, "source": dataclasses.asdict(c.source),
                 "capabilities": list(c.capabilities)}
                for (k, _), c in sorted(self._items.items()) if kind in (None, k)]


def default_registry() -> Registry:
    r = Registry()
    for name in PRESETS:
        caps = ("tensor",) if PRESETS[name].family == "regression" else ("text", "packed")
        r.add_model(f"{name}@1", (lambda n=name: preset(n)), capabilities=caps)
    r.add_model("shadowspill/regression@1", lambda: preset("regression"), capabilities=("tensor",))
    r.add_objective("shadowspill/cross_entropy@1", lambda **kw: {"kind": "cross_entropy", **kw},
                    capabilities=("text",))
    r.add_objective("shadowspill/clipped_policy@1",
                    lambda clip_ratio=0.2, reference_beta=0.0: {"kind": "clipped_policy",
                                                                "clip_ratio": clip_ratio,
                                                                "reference_beta": reference_beta},
                    capabilities=("text",))
    r.add_objective("shadowspill/weighted_squared_error@1",
                    lambda **kw: {"kind": "weighted_squared_error", **kw}, capabilities=("tensor",))
    r.add_objective("shadowspill/moe_balance@1", lambda coefficient=0.01: {"kind": "moe_balance",
                                                                           "coefficient": coefficient})
    r.add_objective("shadowspill/sum@1", lambda terms=(): {"kind": "sum", "terms": list(terms)})
    r.add_optimizer("adamw@1", lambda **kw: {"kind": "adamw", **kw})
    r.add_optimizer("mlops/adamw@1", lambda **kw: {"kind": "adamw", **kw})    # the reference's id
    r.add_optimizer("sgd@1", lambda **kw: {"kind": "sgd", **kw})              # momentum = beta1
    r.add_optimizer("lion@1", lambda **kw: {"kind": "lion", **kw})
    r.add_preparation("shadowspill/default@1", lambda **kw: kw)
    r.add_policy("shadowspill/text_chunks@1",
                 lambda projection=0, moe=0, rows=0, delta_heads=1: {"projection": projection, "moe": moe, "rows": rows,
                                                                     "delta_heads": delta_heads})
    r.add_policy("shadowspill/text_retention@1", lambda rule="cost-input": {"rule": rule})
    return r


_RETENTION_VARIANT = {"cost-input": "recompute", "cost-attention": "save_attention",
                      "attention-input": "save_attention"}


@dataclass
class ResolvedTraining:
    cfg: DecoderConfig
    workers: int
    setups: list[dict[str, Any]]              # one TrainingSetup (as JSON) per rank
    geometry: dict[str, Any]
    provenance: dict[str, str]
    budgets: dict[str, float]


def _lora_record(rec: dict | None, is_moe: bool = False) -> dict | None:
    """Client ``LoRA`` record -> ``models.lora.LoRAConfig`` JSON."""
    if not rec:
        return None
    from ..models.lora import DENSE_TARGETS, LoRAConfig
    groups = {"attention": ("wq", "wk", "wv", "wo", "w_qkvz", "w_out", "q_a", "q_b", "kv_a", "kv_b"),
              "mlp": ("w13", "w2", "sw13", "sw2"),
              "experts": ("w13", "w2")}
    wanted = rec.get("targets", ("attention", "experts"))
    targets: list[str] = []
    for t in wanted:                        # group names of the client record, or matrix names
        if t == "experts" and not is_moe:
            continue                        # a dense model has no routed banks to adapt
        for name in groups.get(t, (t,)):
            if name in DENSE_TARGETS and name not in targets:
                targets.append(name)
    return LoRAConfig(int(rec.get("rank", 16)), float(rec.get("alpha", 32.0)), tuple(targets),
                      "experts" in wanted, bool(rec.get("train_base", False))).to_json()


def _objective_record(rec: dict | None) -> dict | None:
    """Client ``Objective`` record (component id, config, summed terms) -> ``Objective`` JSON."""
    if not rec or rec.get("id", "shadowspill/cross_entropy@1") == "shadowspill/cross_entropy@1":
        return None
    from ..models.objectives import Objective
    if rec["id"] == "shadowspill/sum@1":
        head, head_cfg, balance = "shadowspill/cross_entropy@1", {}, 0.0
        for term in rec.get("terms", ()):
            if term.get("id") == "shadowspill/moe_balance@1":
                balance = float((term.get("config") or {}).get("coefficient", 0.01))
            else:
                head, head_cfg = term["id"], dict(term.get("config") or {})
        return Objective.from_component("shadowspill/sum@1", head=head, head_config=head_cfg,
                                        moe_balance=balance).to_json()
    return Objective.from_component(rec["id"], **dict(rec.get("config") or {})).to_json()


def resolve_training(body: dict[str, Any], registry: Registry, hardware: dict[str, Any]) -> ResolvedTraining:
    """Client settings -> per-rank worker setups, with the provenance of every default."""
    prov: dict[str, str] = {}
    m = body["model"]
    if m.get("config"):
        cfg = DecoderConfig.from_json(m["config"]); prov["model"] = "explicit config"
    else:
        name = m["name"] if "@" in m["name"] else m["name"] + "@1"
        cfg = registry.get("model", name).create(); prov["model"] = f"catalog {name}"
    registry.get("objective", body["objective"]["id"])
    opt = body["optimizer"]
    registry.get("optimizer", opt["id"])
    # gradients, moments and parameters are all kept in the model dtype (no master copies):
    # say so instead of silently ignoring a request for anything else
    model_dtype = m.get("dtype", "bfloat16")
    for key in ("gradient_dtype", "opt_state_dtype"):
        if opt.get(key, "bfloat16") not in ("bfloat16", model_dtype):
            raise ValueError(f"optimizer {key}={opt[key]!r} is not supported: gradients and moments are "
                             f"kept in the model dtype ({model_dtype})")
    if opt.get("master_dtype", "bfloat16") not in ("bfloat16", "float32", model_dtype):
        raise ValueError(f"optimizer master_dtype={opt['master_dtype']!r} is not supported")
    master_weights = opt.get("master_dtype", "bfloat16") == "float32" and model_dtype != "float32"
    res = body.get("resources", {})
    par = body.get("parallelism") or {}
    per_replica = int(par.get("ranks_per_replica", res.get("gpus", 1)))
    replicas = int(par.get("num_replicas", 1))
    if replicas > 1 and par.get("kind") == "expert_parallel":
        raise ValueError("expert parallelism runs as one replica")
    workers = per_replica * replicas
    backend = res.get("backend", "cuda")
    device = "cuda" if backend == "cuda" else "cpu"
    if device == "cuda" and workers > max(1, hardware.get("gpus", 0)):
        raise ValueError(f"{workers} workers requested, {hardware.get('gpus', 0)} GPUs present")
    mem = body.get("memory", {})
    device_gib, spill_gib = float(mem.get("device_gib", 0)), float(mem.get("spill_gib", 0))
    if device_gib <= 0:
        device_gib = 0.9 * hardware.get("device_gib", 180.0); prov["device_gib"] = "automatic 90 %"
    if mem.get("spill_pool", "host") == "file":
        import os
        if spill_gib <= 0 or not os.path.isdir(mem.get("spill_directory", "")):
            raise ValueError("a file spill pool needs spill_gib and an existing spill_directory on the node")
        prov["spill_pool"] = f"file in {mem['spill_directory']}"
    if mem.get("spill_pool") == "remote":
        if spill_gib <= 0 or ":" not in mem.get("spill_address", ""):
            raise ValueError("a remote spill pool needs spill_gib and spill_address = host:port")
        prov["spill_pool"] = f"memory daemon at {mem['spill_address']}"
    if spill_gib <= 0:
        spill_gib = 0.9 * hardware.get("host_free_gib", 64.0) / max(1, workers)
        prov["spill_gib"] = "automatic 90 % of free host memory"
    b = body.get("batch", {})
    T, tokens = int(b.get("microbatch_tokens", 8192)), int(b.get("tokens_per_step", 65536))
    slots = int(b.get("max_datums", 0)) or max(16, T // 32 + 1)
    if cfg.family == "regression":
        slots = max(slots, T + 1)             # every row is its own datum
        if m.get("dtype", "bfloat16") != "float32":
            raise ValueError("the regression family trains in float32: Model(..., dtype='float32')")
    prep = body.get("preparation", {})
    build, planning = prep.get("build", {}), prep.get("planning", {})
    saved_variant = build.get("saved_variant", "save_attention")
    head_chunks = moe_chunks = axis_rows = 0
    delta_heads = 1
    frontend = str(build.get("frontend", "stages"))
    if frontend not in ("stages", "graph"):
        raise ValueError(f"unknown build frontend {frontend!r} (stages | graph)")
    for pol in prep.get("policies", []):
        # every policy is a registered component; one that an extension package added may be a
        # preset of a built-in policy ("alias_of" names it, the rest is its configuration)
        made = registry.get("policy", pol.get("id", "")).create(**(pol.get("config") or {}))
        if isinstance(made, dict) and made.get("alias_of"):
            prov[f"policy {pol['id']}"] = f"preset of {made['alias_of']}"
            pol = {"id": made["alias_of"], "config": {k: v for k, v in made.items() if k != "alias_of"}}
        if pol.get("id") == "shadowspill/text_chunks@1":
            # "projection": row chunks of the output projection; "moe": expert groups a routed layer
            # is pipelined in under expert parallelism; "rows": token rows per chunk of the
            # token-local operators inside a layer stage (graph frontend; sequence mixers stay whole)
            head_chunks = int((pol.get("config") or {}).get("projection", 0) or 0)
            moe_chunks = int((pol.get("config") or {}).get("moe", 0) or 0)
            axis_rows = int((pol.get("config") or {}).get("rows", 0) or 0)
            delta_heads = int((pol.get("config") or {}).get("delta_heads", 1) or 1)   # key-head groups of the delta rule
            if axis_rows < 0:
                raise ValueError("text_chunks rows must not be negative")
            if axis_rows:
                frontend = "graph"            # axis chunks are a transform of the exported graphs
        if pol.get("id") == "shadowspill/text_retention@1":
            saved_variant = _RETENTION_VARIANT.get((pol.get("config") or {}).get("rule", ""), saved_variant)
    ex = body.get("execution", {})
    sr = opt.get("parameter_rounding", "stochastic") == "stochastic"
    search = {"workers": planning.get("workers", 0),
              "strategies": list(planning.get("strategies", ("stall", "traffic"))),
              "fetch_rules": list(planning.get("fetch_rules",
                                               ("demand", "latest-safe", "packed-fifo", "packed-fit"))),
              "max_repairs": planning.get("max_repairs", 16),
              "minimum_object_bytes_evict_eligible":
                  planning.get("minimum_object_bytes_evict_eligible", 1 << 20),
              "deterministic": planning.get("deterministic", False)}
    setups = []
    for rank in range(workers):
        setups.append({
            "model": cfg.to_json(), "device_gib": device_gib, "spill_gib": spill_gib,
            "tokens_per_step": tokens, "microbatch_tokens": T, "slots": slots,
            "lr": opt.get("lr", 1e-4), "beta1": opt.get("beta1", 0.9), "beta2": opt.get("beta2", 0.95),
            "eps": opt.get("eps", 1e-8), "weight_decay": opt.get("weight_decay", 0.0),
            "parameter_groups": [dict(g) for g in opt.get("parameter_groups", ())],
            "observe_norms": bool(ex.get("observe_norms", False)),
            "collective_overhead_us": float(planning.get("collective_overhead_us", 0.0)),
            "optimizer_rule": registry.get("optimizer", opt["id"]).create()["kind"],
            "seed": int(m.get("weights", {}).get("seed", ex.get("seed", 0))),
            "dtype": m.get("dtype", "bfloat16"), "stochastic_rounding": sr, "device": device,
            "device_index": rank if device == "cuda" else 0, "rank": rank, "world_size": workers,
            "ranks_per_replica": per_replica if replicas > 1 else 0,
            "min_shard_bytes": int(par.get("min_shard_bytes", 0)) if workers > 1 else 0,
            "head_chunks": head_chunks, "moe_chunks": moe_chunks, "master_weights": master_weights,
            "frontend": frontend, "axis_chunk_rows": axis_rows, "delta_head_groups": delta_heads,
            "walks": list(build.get("walks", ("breadth",))),
            "recompute_shares": list(build.get("recompute_shares", (100,))),
            "saved_variant": saved_variant,
            "profile": bool(prep.get("profiling", {}).get("enabled", True)) and not body.get("simulation_only"),
            "calibrate": bool(prep.get("calibrate", True)) and not body.get("simulation_only"),
            "search": search, "collectives": ex.get("collectives", "auto"),
            "operations": list(body.get("operations", ("step",))),
            "trace_capacity": 65536 if ex.get("runtime_trace") else 0, "nsys": ex.get("nsys"),
            "profiler_annotations": bool(ex.get("profiler_annotations", False)),
            "spill_pool": mem.get("spill_pool", "host"), "spill_directory": mem.get("spill_directory", ""),
            "spill_address": mem.get("spill_address", ""),
            "spill_chunk_bytes": int(mem.get("spill_chunk_bytes", 2 << 20)),
            "spill_queue_depth": int(mem.get("spill_queue_depth", 16)),
            "lora": _lora_record(m.get("lora"), cfg.is_moe), "objective": _objective_record(body.get("objective")),
            "expert_parallel": (body.get("parallelism") or {}).get("kind") == "expert_parallel",
            "pretrained": (m.get("weights", {}).get("location", "")
                           if m.get("weights", {}).get("source") == "checkpoint" else "")})
    ob = _objective_record(body.get("objective"))
    from ..frontend.capture import extra_fields_for
    from ..models.objectives import Objective as _Ob
    extra_fields = list(extra_fields_for(cfg, _Ob.from_json(ob) if ob else None))
    geometry = {"extra_fields": extra_fields,
                "microbatch_tokens": T, "microbatches": tokens // T, "slots": slots,
                "vocab_size": cfg.vocab_size, "workers": workers, "packing": b.get("packing", "best_fit"),
                "tokens_per_step": tokens * workers}
    return ResolvedTraining(cfg, workers, setups, geometry, prov,
                            {"device_gib": device_gib, "spill_gib": spill_gib})
