"""Build phase: model configuration + batch geometry -> ``Program``.

The step is unrolled over stages and microbatches in a chosen walk
(``StepDataOrdering``): *breadth* runs one stage across all microbatches before
the next stage, so a stage's weights are fetched once per pass; *depth* runs
each microbatch through the whole model. The last stage runs its forward
together with its backward (``pair_loss``), backward passes visit microbatches
in reverse (``reverse_breadth``), and each stage's optimizer task follows its
last backward (``stage_interleaved``) or all of them run at the end (``tail``).
These are the reference's walk and ordering knobs
(packages/engine/src/shadowspill/step/ordering.py:11,
docs/architecture/planning-pipeline.md:56-76).

Every stage execution is a task; every tensor that outlives a task is an
object: stage weights and AdamW moments (persistent: their home is the spill
pool), gradients, stage-boundary activations, saved sets of ``save`` variants,
the per-microbatch activation gradient, the packed batch and the loss.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import torch

from ..ir.program import ObjectSpec, Program, TaskSpec, UseSpec
from ..models.config import DecoderConfig
from ..models.decoder import ALIGN, Stage, build_stages

_DT = {torch.bfloat16: "bfloat16", torch.float32: "float32", torch.float16: "float16"}


@dataclass(frozen=True)
class StepDataOrdering:
    walk: str = "breadth"            # breadth | depth
    reverse_breadth: bool = True
    pair_loss: bool = True
    optimizer: str = "stage_interleaved"   # stage_interleaved | tail
    # sharded storage, breadth walk: run the microbatches in this many groups, each a full
    # forward + backward sweep over the layers. Live activations shrink with the group; the
    # weights are gathered once per group and pass (NVLink, cheap) and every group's gradient is
    # reduce-scattered into a shard-sized fp32 accumulator, which the update of the last group
    # reads. 1 = one sweep over all microbatches.
    microbatch_groups: int = 1
    # sharded storage, breadth walk: emit each weight gather one weight set before its first reader
    gather_ahead: bool = True

    def label(self) -> str:
        return f"{self.walk}/{self.optimizer}" + (f"/groups{self.microbatch_groups}" if self.microbatch_groups > 1 else "")


@dataclass
class BatchGeometry:
    microbatch_tokens: int
    n_microbatches: int
    slots: int = 64                  # sequence slots per microbatch (cu_seqlens has slots+1)
    mean_seqlen: float = 2048.0
    # further per-row fp32 fields the objective or the model reads: "name" or "name:width"
    extra_fields: tuple[str, ...] = ()

    @property
    def tokens(self) -> int:
        return self.microbatch_tokens * self.n_microbatches


def field_spec(field_name: str) -> tuple[str, int]:
    """``"name"`` -> ``(name, 1)``; ``"name:width"`` -> ``(name, width)``."""
    name, _, width = field_name.partition(":")
    return name, int(width) if width else 1


def extra_fields_for(cfg, objective) -> tuple[str, ...]:
    """Batch fields beyond tokens/targets/weights/positions for this model and objective."""
    fields = tuple(objective.extra_fields) if objective is not None else ()
    if cfg.family == "regression":
        from ..models.regression import batch_fields
        fields = batch_fields(cfg) + fields
    return fields


def batch_layout(T: int, slots: int, extras: tuple[str, ...] = ()
                 ) -> tuple[dict[str, tuple[int, int, str]], int]:
    """Byte layout of one packed microbatch object: name -> (offset, count, dtype)."""
    out, off = {}, 0
    fields = [("tokens", T, "int64", 8), ("targets", T, "int64", 8), ("weights", T, "float32", 4),
              ("positions", T, "int32", 4), ("cu_seqlens", slots + 1, "int32", 4)]
    for spec in extras:
        name, width = field_spec(spec)
        fields.append((name, T * width, "float32", 4))
    for name, count, dt, size in fields:
        out[name] = (off, count, dt)
        off = (off + count * size + ALIGN - 1) // ALIGN * ALIGN
    return out, off


def saved_layout(stage: Stage, T: int, variant: str, dtype: torch.dtype = torch.bfloat16):
    """[(name, shape, dtype, offset)], total bytes of a stage's saved set."""
    if not hasattr(stage, "saved_shapes"):
        return [], 0
    out, off = [], 0
    for name, shape, dt in stage.saved_shapes(T, variant, dtype):
        nbytes = int(torch.tensor([], dtype=dt).element_size())
        for d in shape:
            nbytes *= d
        out.append((name, shape, dt, off))
        off = (off + nbytes + ALIGN - 1) // ALIGN * ALIGN
    return out, off


@dataclass
class TrainingDescription:
    """Everything the executor needs to turn tasks back into stage calls."""
    cfg: DecoderConfig
    geometry: BatchGeometry
    ordering: StepDataOrdering
    dtype: torch.dtype = torch.bfloat16
    grad_dtype: torch.dtype = torch.bfloat16
    selection: dict[int, str] = field(default_factory=dict)   # stage index -> variant
    mode: str = "step"                # step | forward_backward | forward
    world_size: int = 1               # data-parallel ranks with sharded weights/optimizer state
    rank: int = 0
    objective: "Objective | None" = None
    lora: "LoRAConfig | None" = None
    expert_parallel: bool = False     # routed layers keep 1/world of the experts per rank
    # hierarchical data parallelism: ``world_size`` ranks share one sharded copy of the state and
    # ``replicas`` such groups run side by side (rank = replica * world_size + shard index);
    # gradients are summed over every rank, weights are gathered inside a replica
    replicas: int = 1
    # sharded storage keeps tensors smaller than this whole on every rank (0 = cut everything)
    min_shard_bytes: int = 0
    # rows of the output projection evaluated at once (the head never materialises all logits);
    # 0 = the stage's default. Fewer rows = less workspace, more launches.
    head_block_rows: int = 0
    # fp32 master copies of the trainable parameters: the optimizer updates them and rounds the
    # result into the model-dtype weights (unfused update path)
    master_weights: bool = False
    # "stages": the hand-written stage classes; "graph": torch.export -> partition -> AOT graph
    # pairs (frontend/graph_stage.py) for the models it covers, the stage classes otherwise
    frontend: str = "stages"
    # sharded storage on GPUs: leave the all-gather of a layer's matrices to the first GEMM that
    # consumes them in the forward pass (ops/csrc/gemm_tcgen05_2cta.cu, GATHER form). The first
    # forward task of the stage then also holds the shard, whose peers read it during that task.
    fused_gather: bool = False
    # graph frontend: token-local operators of a layer stage (projections, norms, MLP) run in row
    # chunks of this many tokens (frontend/chunking.py); 0 = whole microbatch at once
    axis_chunk_rows: int = 0

    def __post_init__(self) -> None:
        extras = extra_fields_for(self.cfg, self.objective)
        if tuple(self.geometry.extra_fields) != tuple(extras):
            from dataclasses import replace as _replace
            self.geometry = _replace(self.geometry, extra_fields=tuple(extras))

    @property
    def shard_rank(self) -> int:
        return self.rank % self.world_size

    @property
    def total_ranks(self) -> int:
        return self.world_size * self.replicas

    def stages(self):
        ep = (self.world_size, self.rank) if (self.expert_parallel and self.world_size > 1) else None
        if self.frontend == "graph" or self.cfg.is_latent_attention:
            from .graph_stage import build_graph_stages, supports
            if self.cfg.is_latent_attention and not supports(self.cfg, self.lora, ep, self.objective):
                raise ValueError(f"the {self.cfg.family} family is defined for the graph frontend only, which "
                                 "does not cover expert parallelism or the router-balance term yet")
            if supports(self.cfg, self.lora, ep, self.objective):
                stages = build_graph_stages(self.cfg, self.geometry.microbatch_tokens, self.geometry.slots,
                                            self.dtype, self.grad_dtype, self.head_block_rows,
                                            chunk_rows=self.axis_chunk_rows, lora=self.lora)
                for st in stages:
                    st.min_shard_bytes = int(self.min_shard_bytes)
                return stages
        elif self.frontend != "stages":
            raise ValueError(f"unknown frontend {self.frontend!r}")
        stages = build_stages(self.cfg, self.objective, self.lora, ep)
        for st in stages:
            st.min_shard_bytes = int(self.min_shard_bytes)
        if self.head_block_rows > 0 and hasattr(stages[-1], "block_rows"):
            stages[-1].block_rows = int(self.head_block_rows)
        return stages

    def variant(self, stage_index: int) -> str:
        return self.selection.get(stage_index, "recompute")


def estimate_duration_ns(flops: float, nbytes: float, tflops: float = 1100.0,
                         gbps: float = 5000.0) -> int:
    return int(max(flops / (tflops * 1e12), nbytes / (gbps * 1e9)) * 1e9) + 20_000


def exposed_collective_ns(nbytes: float, world: int) -> int:
    """What a collective on the communication stream costs the compute timeline. The planner's
    timeline is one lane: a task's duration is how long the next task waits for it. The peer
    kernels move ``(world - 1) / world`` of the bytes over NVLink (about 700 GB/s measured per
    direction) while the compute stream keeps running; a traced two-GPU step showed the compute
    stream idle for about a quarter of its collectives' time, which is the share charged here."""
    remote = nbytes * (world - 1) / max(1, world)
    return int(0.25 * remote / 700e9 * 1e9) + 20_000


def add_collective_overhead(program: Program, microseconds: float) -> int:
    """Adds ``microseconds`` to the planned duration of every task that runs on the communication
    stream (collectives and the sharded update); returns how many tasks that was. The figure comes
    from a traced step (``qualification/gap_report.py``): what such a task costs the compute lane
    beyond the modelled share of its NVLink time."""
    extra = int(microseconds * 1e3)
    touched = 0
    if extra <= 0:
        return 0
    for t in program.tasks:
        if t.kind == "collective" or t.variant == "adamw_dp":
            t.duration_ns += extra
            touched += 1
    return touched


def _build(desc: TrainingDescription) -> Program:
    cfg, geo, order = desc.cfg, desc.geometry, desc.ordering
    stages = desc.stages()
    S, n_mb, T = len(stages), geo.n_microbatches, geo.microbatch_tokens
    train = desc.mode != "forward"
    step = desc.mode in ("step", "optimizer")
    only_optimizer = desc.mode == "optimizer"
    step_mode = desc.mode == "step"
    isz = desc.dtype.itemsize
    prog = Program(metadata={"model": cfg.to_json(), "tokens": geo.tokens, "mode": desc.mode,
                             "microbatch_tokens": T, "n_microbatches": n_mb, "slots": geo.slots,
                             "ordering": order.label(), "dtype": _DT[desc.dtype],
                             "grad_dtype": _DT[desc.grad_dtype],
                             "selection": ",".join(f"{k}:{v}" for k, v in sorted(desc.selection.items()))
                             or "recompute",
                             "walk": order.walk, "optimizer_order": order.optimizer,
                             "objective": desc.objective.to_json() if desc.objective else None,
                             "lora": desc.lora.to_json() if desc.lora else None})
    W, M, V, G = [], [], [], []
    world = desc.world_size
    sharded = world > 1
    prog.metadata["world_size"] = world
    FULL: dict[tuple[int, str], int] = {}     # (stage, pass) -> gathered full-weight object
    MASTER: dict[int, int] = {}               # stage -> fp32 master copy (optional)
    full_bytes = []
    for si, st in enumerate(stages):
        _, pbytes = st.layout(desc.dtype)
        full_bytes.append(pbytes)
        if sharded:
            _, pbytes = st.shard_layout(desc.dtype, world)
        _, gbytes = st.layout(desc.grad_dtype, torch.float32, trainable_only=True)
        if sharded:
            _, sbytes_opt = st.shard_layout(desc.dtype, world, trainable_only=True)
        else:
            _, sbytes_opt = st.layout(desc.dtype, trainable_only=True)
        W.append(prog.add_object(ObjectSpec(f"{st.name}.weights", pbytes, "weight", True, stage=si,
                                            sharding="sharded" if sharded else "whole")))
        if not st.has_trainable:          # a frozen stage owns no gradients and no moments
            G.append(-1); M.append(-1); V.append(-1)
            continue
        if train:
            # gradients persist across calls when accumulation is driven from outside
            G.append(prog.add_object(ObjectSpec(f"{st.name}.gradients", gbytes, "gradient",
                                                persistent=desc.mode != "step", stage=si)))
        if step and desc.master_weights:
            if sharded:
                _, mbytes = st.shard_layout(torch.float32, world, trainable_only=True)
            else:
                _, mbytes = st.layout(torch.float32, trainable_only=True)
            MASTER[si] = prog.add_object(ObjectSpec(f"{st.name}.master", mbytes, "optimizer_state", True,
                                                    stage=si, sharding="sharded" if sharded else "whole"))
        if step:
            sh = "sharded" if sharded else "whole"
            M.append(prog.add_object(ObjectSpec(f"{st.name}.exp_avg", sbytes_opt, "optimizer_state", True, stage=si, sharding=sh)))
            V.append(prog.add_object(ObjectSpec(f"{st.name}.exp_avg_sq", sbytes_opt, "optimizer_state", True, stage=si, sharding=sh)))
    if only_optimizer:
        # the update alone: gradients accumulated by earlier forward_backward calls are state
        prog.metadata["n_microbatches"] = 0
        for si in reversed(range(S)):
            st = stages[si]
            if not st.has_trainable:
                continue
            pbytes = prog.objects[W[si]].bytes
            prog.add_task(TaskSpec(f"O.{st.name}", "optimizer", si, -1,
                                   [UseSpec(W[si], "mutate", "params"), UseSpec(G[si], "read", "grads"),
                                    UseSpec(M[si], "mutate", "m"), UseSpec(V[si], "mutate", "v")]
                                   + ([UseSpec(MASTER[si], "mutate", "master")] if si in MASTER else []),
                                   estimate_duration_ns(0.0, 8.0 * pbytes), 0,
                                   "adamw_dp" if sharded else "adamw",
                                   profile_key=f"opt:{pbytes}:{world}" + (":master" if si in MASTER else "")))
        prog.validate()
        return prog
    _, in_bytes = batch_layout(T, geo.slots, geo.extra_fields)
    IN = [prog.add_object(ObjectSpec(f"batch.{m}", in_bytes, "input", True, pinned_resident=True,
                                     microbatch=m)) for m in range(n_mb)]
    LOSS = prog.add_object(ObjectSpec("loss", 512, "output", True, pinned_resident=True))
    # a forward-only program also returns what the head computes per row (the log-probability
    # of each target token; the prediction vector of a regression head)
    ow = getattr(stages[-1], "output_width", 0)
    OUT = ([prog.add_object(ObjectSpec(f"outputs.{m}", -(-T * ow * 4 // ALIGN) * ALIGN, "output", True,
                                       pinned_resident=True, microbatch=m)) for m in range(n_mb)]
           if (not train and ow) else [])
    act_bytes = T * cfg.d_model * isz
    A = [[prog.add_object(ObjectSpec(f"{stages[si].name}.out.{m}", act_bytes, "activation",
                                     stage=si, microbatch=m)) for m in range(n_mb)]
         for si in range(S - 1)]
    DX = [prog.add_object(ObjectSpec(f"dx.{m}", act_bytes, "activation_gradient", microbatch=m))
          for m in range(n_mb)] if train else []
    SAVED: dict[tuple[int, int], int] = {}
    for si in range(1, S - 1):
        var = desc.variant(si)
        if train and var != "recompute":
            _, sbytes = saved_layout(stages[si], T, var, desc.dtype)
            for m in range(n_mb):
                SAVED[(si, m)] = prog.add_object(ObjectSpec(f"{stages[si].name}.saved.{m}", sbytes,
                                                            "saved", stage=si, microbatch=m))
    GG: dict[tuple[int, int], int] = {}       # (stage, group) -> that group's gradient object
    ACC: dict[int, int] = {}                  # stage -> fp32 shard-sized sum of the earlier groups
    acc_created: set[int] = set()

    def grad_obj(si: int) -> int:
        """The gradient object the current group of microbatches writes."""
        if groups <= 1:
            return G[si]
        gi = group_now[0]
        if (si, gi) not in GG:
            if gi == 0:
                GG[(si, gi)] = G[si]
            else:
                spec = prog.objects[G[si]]
                GG[(si, gi)] = prog.add_object(ObjectSpec(f"{stages[si].name}.gradients.g{gi}", spec.bytes,
                                                          "gradient", stage=si))
        return GG[(si, gi)]

    def grad_use(si: int, role: str) -> UseSpec:
        key_ = (si, group_now[0]) if groups > 1 else si
        if step_mode and key_ not in grads_started:
            grads_started.add(key_)
            return UseSpec(grad_obj(si), "create", role)
        return UseSpec(grad_obj(si), "mutate", role)
    grads_started: set = set()

    tag = ""
    if desc.lora is not None:
        tag += f":lora{desc.lora.rank}{'b' if desc.lora.train_base else ''}"
    if desc.expert_parallel and world > 1:
        tag += f":ep{world}"
    if desc.objective is not None and desc.objective.kind != "cross_entropy":
        tag += f":{desc.objective.kind}"

    def key(st: Stage, what: str, var: str = "") -> str:
        # layers of one class can differ in kind (DeltaNet or attention mixer): keep them apart
        kind = getattr(st, "mixer", "")
        return f"{cfg.family}:{st.kind}:{type(st).__name__}{':' + kind if kind else ''}:{what}:{var}:T{T}{tag}"

    fresh_gather: set[tuple[int, str]] = set()       # gathers whose first consumer is still to come

    groups = max(1, int(order.microbatch_groups)) if (sharded and order.walk == "breadth" and step_mode) else 1
    if groups > 1 and n_mb % groups:
        raise ValueError("microbatch_groups must divide the number of microbatches")
    if groups > 1 and desc.expert_parallel:
        raise ValueError("microbatch groups are not combined with expert parallelism (not tested together)")
    group_now = [0]

    def params_of(si: int, which: str) -> int:
        """The object a compute task reads its weights from; under sharded storage
        the first user in a pass is preceded by the all-gather task that builds it."""
        if not sharded:
            return W[si]
        tag = which if order.walk == "breadth" else "all"
        if groups > 1:
            tag = f"{tag}.g{group_now[0]}"
        if (si, tag) not in FULL:
            fresh_gather.add((si, tag))
            st = stages[si]
            obj = prog.add_object(ObjectSpec(f"{st.name}.weights.full.{tag}", full_bytes[si],
                                             "weight", stage=si))
            FULL[(si, tag)] = obj
            nbytes = full_bytes[si]
            prog.add_task(TaskSpec(f"AG.{st.name}.{tag}", "collective", si, -1,
                                   [UseSpec(W[si], "read", "shard"), UseSpec(obj, "create", "params")],
                                   exposed_collective_ns(nbytes, world), 0,
                                   "allgather", profile_key=f"allgather:{nbytes}:{world}"))
        return FULL[(si, tag)]

    def fwd(si: int, m: int) -> None:
        st = stages[si]
        var = desc.variant(si) if train else "recompute"
        uses = [UseSpec(params_of(si, "fwd"), "read", "params"), UseSpec(IN[m], "read", "batch"),
                UseSpec(A[si][m], "create", "y")]
        tag_ = "fwd" if order.walk == "breadth" else "all"
        if groups > 1:
            tag_ = f"{tag_}.g{group_now[0]}"
        if (si, tag_) in fresh_gather:
            fresh_gather.discard((si, tag_))
            if desc.fused_gather and getattr(st, "fused_gather_params", ()):
                # this task's GEMMs pull the peers' shards: the shard must outlive it
                uses.append(UseSpec(W[si], "read", "shard"))
        if si > 0:
            uses.append(UseSpec(A[si - 1][m], "read", "x"))
        if (si, m) in SAVED:
            uses.append(UseSpec(SAVED[(si, m)], "create", "saved"))
        fl = st.flops(T, geo.mean_seqlen)
        prog.add_task(TaskSpec(f"F.{st.name}.{m}", "forward", si, m, uses,
                               estimate_duration_ns(fl, 8.0 * act_bytes),
                               st.workspace_bytes(T, isz) // 2, var, flops=fl, tokens=T,
                               profile_key=key(st, "fwd", var)))

    def head(m: int) -> None:
        si, st = S - 1, stages[S - 1]
        uses = [UseSpec(params_of(si, "fwd"), "read", "params"), UseSpec(IN[m], "read", "batch"),
                UseSpec(A[si - 1][m], "read", "x"), UseSpec(LOSS, "mutate", "loss")]
        if cfg.tied_embeddings:
            # the output matrix is the embedding: read it here, and start (or add to) its gradient
            uses.append(UseSpec(params_of(0, "fwd"), "read", "tied_params"))
            if train and stages[0].has_trainable:
                uses.append(grad_use(0, "tied_grads"))
        if OUT:
            uses.append(UseSpec(OUT[m], "mutate", "outputs"))
        if train:
            uses.append(UseSpec(DX[m], "create", "dx"))
            if st.has_trainable:
                uses.append(grad_use(si, "grads"))
        fl = st.flops(T, geo.mean_seqlen) * (3.0 if train else 1.0)
        prog.add_task(TaskSpec(f"H.{st.name}.{m}", "head", si, m, uses,
                               estimate_duration_ns(fl, 8.0 * act_bytes),
                               st.workspace_bytes(T, isz), "train" if train else "eval",
                               flops=fl, tokens=T, profile_key=key(st, "head", "train" if train else "eval")))

    def bwd(si: int, m: int) -> None:
        st = stages[si]
        if not st.has_trainable and si == 0:
            return                      # a frozen embedding has nothing to compute backward
        var = desc.variant(si)
        uses = [UseSpec(IN[m], "read", "batch"),
                UseSpec(DX[m], "mutate" if si > 0 else "read", "dx")]
        if st.kind != "embedding":      # the embedding's backward is a scatter-add: no weights
            uses.append(UseSpec(params_of(si, "bwd"), "read", "params"))
        if si > 0:
            uses.append(UseSpec(A[si - 1][m], "read", "x"))
        if (si, m) in SAVED:
            uses.append(UseSpec(SAVED[(si, m)], "read", "saved"))
        if st.has_trainable:
            uses.append(grad_use(si, "grads"))
        fl = st.flops(T, geo.mean_seqlen) * (3.0 if var == "recompute" else 2.0)
        prog.add_task(TaskSpec(f"B.{st.name}.{m}", "backward", si, m, uses,
                               estimate_duration_ns(fl, 16.0 * act_bytes),
                               st.workspace_bytes(T, isz), var, flops=fl, tokens=T,
                               profile_key=key(st, "bwd", var)))

    def opt(si: int) -> None:
        st = stages[si]
        if not st.has_trainable:
            return
        pbytes = prog.objects[W[si]].bytes
        prog.add_task(TaskSpec(f"O.{st.name}", "optimizer", si, -1,
                               [UseSpec(W[si], "mutate", "params"), UseSpec(grad_obj(si), "read", "grads"),
                                UseSpec(M[si], "mutate", "m"), UseSpec(V[si], "mutate", "v")]
                               + ([UseSpec(MASTER[si], "mutate", "master")] if si in MASTER else [])
                               + ([UseSpec(ACC[si], "read", "acc")] if si in ACC else []),
                               estimate_duration_ns(0.0, 8.0 * pbytes),
                               # the unfused update holds a handful of fp32 temporaries per parameter
                               (6 * prog.objects[MASTER[si]].bytes) if si in MASTER else 0,
                               "adamw_dp" if sharded else "adamw",
                               profile_key=f"opt:{pbytes}:{world}" + (":master" if si in MASTER else "")
                               + (":acc" if si in ACC else "")))

    def accumulate(si: int) -> None:
        """Reduce-scatter this group's gradient of stage ``si`` into the fp32 shard accumulator."""
        st = stages[si]
        if not st.has_trainable:
            return
        if si not in ACC:
            _, abytes = st.shard_layout(torch.float32, world, trainable_only=True)
            ACC[si] = prog.add_object(ObjectSpec(f"{st.name}.gradient_sum", abytes, "gradient", stage=si,
                                                 sharding="sharded"))
        gbytes = prog.objects[grad_obj(si)].bytes
        mode = "mutate" if si in acc_created else "create"
        acc_created.add(si)
        prog.add_task(TaskSpec(f"RS.{st.name}.g{group_now[0]}", "collective", si, -1,
                               [UseSpec(grad_obj(si), "read", "grads"), UseSpec(ACC[si], mode, "acc")],
                               exposed_collective_ns(gbytes, world), 0, "rs_accumulate",
                               profile_key=f"rs_accumulate:{gbytes}:{world}"))

    body = list(range(S - 1))
    mbs = list(range(n_mb))
    step = desc.mode == "step"      # from here on: does this program contain the update?
    if order.walk == "breadth":
        per_group = n_mb // groups
        # the weight sets in the order the sweeps read them: a gather is emitted one set ahead of
        # its first reader, so that it runs on the communication stream under the tasks before it
        reads = [(si, "fwd") for si in body] + [(S - 1, "fwd")]
        if train:
            reads += [(si, "bwd") for si in reversed(body) if stages[si].kind != "embedding"]
        ahead = sharded and order.gather_ahead and not desc.fused_gather

        def gather_next(si: int, which: str, gi: int) -> None:
            """Emits the gather of the weight set read after ``(si, which)`` of group ``gi``."""
            if not ahead:
                return
            k = reads.index((si, which)) + 1 if (si, which) in reads else len(reads) + 1
            if k > len(reads):
                return
            nxt, g_next = (reads[k], gi) if k < len(reads) else (reads[0], gi + 1)
            if g_next >= groups:
                return
            keep, group_now[0] = group_now[0], g_next
            params_of(*nxt)
            group_now[0] = keep

        for gi in range(groups):
            group_now[0] = gi
            gm = mbs[gi * per_group:(gi + 1) * per_group]
            last = gi == groups - 1

            def finish(si: int) -> None:
                if not last:
                    accumulate(si)
                elif step and order.optimizer == "stage_interleaved":
                    opt(si)
            for si in body:
                params_of(si, "fwd")
                gather_next(si, "fwd", gi)
                for m in gm:
                    fwd(si, m)
            params_of(S - 1, "fwd")
            gather_next(S - 1, "fwd", gi)
            for m in gm:
                head(m)
            if train:
                # Under sharded storage a stage's gradients are consumed on the communication
                # stream (reduce-scatter into the sums, or the fused update), after a barrier that
                # waits for the slowest rank. Emitted right after the stage's last backward task,
                # the next stage's first backward task would create its gradients in the range
                # those still occupy and wait for the collective; emitted one task later, both
                # gradient buffers are live at once and the collective runs under the next tasks.
                owed = None
                if sharded:
                    owed = S - 1
                else:
                    finish(S - 1)
                for si in reversed(body):
                    gather_next(si, "bwd", gi)
                    for m in (list(reversed(gm)) if order.reverse_breadth else gm):
                        bwd(si, m)
                        if owed is not None:
                            finish(owed)
                            owed = None
                    if sharded:
                        owed = si
                    else:
                        finish(si)
                if owed is not None:
                    finish(owed)
    elif order.walk == "depth":
        for m in mbs:
            for si in body:
                fwd(si, m)
            head(m)
            if train:
                for si in reversed(body):
                    bwd(si, m)
        if step and order.optimizer == "stage_interleaved":
            for si in reversed(range(S)):
                opt(si)
    else:
        raise ValueError(f"unknown walk {order.walk!r}")
    if step and order.optimizer == "tail":
        for si in reversed(range(S)):
            opt(si)
    prog.validate()
    return prog


def build_step(cfg: DecoderConfig, geometry: BatchGeometry,
               ordering: StepDataOrdering | None = None, *, dtype=torch.bfloat16,
               grad_dtype=None, selection: dict[int, str] | None = None, world_size: int = 1,
               rank: int = 0, objective=None, lora=None, expert_parallel: bool = False,
               replicas: int = 1, min_shard_bytes: int = 0, head_block_rows: int = 0,
               master_weights: bool = False, frontend: str = "stages", fused_gather: bool = False,
               axis_chunk_rows: int = 0):
    """Forward + backward + optimizer of one global batch. Returns ``(Program, description)``.
    ``world_size > 1`` builds the data-parallel form: weights and AdamW moments are
    stored as 1/N shards, gathered before use and updated shard-locally."""
    desc = TrainingDescription(cfg, geometry, ordering or StepDataOrdering(), dtype,
                               grad_dtype or dtype, dict(selection or {}), "step", world_size,
                               rank, objective, lora, expert_parallel, replicas, min_shard_bytes,
                               head_block_rows, master_weights, frontend, fused_gather, axis_chunk_rows)
    return _build(desc), desc


def build_forward_backward(cfg, geometry, ordering=None, *, dtype=torch.bfloat16, grad_dtype=None,
                           selection=None, world_size=1, rank=0, objective=None, lora=None,
                           min_shard_bytes=0, head_block_rows=0, frontend="stages", axis_chunk_rows=0):
    """Gradient accumulation without the update (gradients are persistent state)."""
    desc = TrainingDescription(cfg, geometry, ordering or StepDataOrdering(), dtype,
                               grad_dtype or dtype, dict(selection or {}), "forward_backward",
                               world_size, rank, objective, lora, min_shard_bytes=min_shard_bytes,
                               head_block_rows=head_block_rows, frontend=frontend,
                               axis_chunk_rows=axis_chunk_rows)
    return _build(desc), desc


def build_forward(cfg, geometry, ordering=None, *, dtype=torch.bfloat16, world_size=1, rank=0,
                  objective=None, lora=None, min_shard_bytes=0, head_block_rows=0, frontend="stages",
                  axis_chunk_rows=0):
    """Evaluation: forward passes and the loss only."""
    desc = TrainingDescription(cfg, geometry, ordering or StepDataOrdering(), dtype, dtype, {},
                               "forward", world_size, rank, objective, lora,
                               min_shard_bytes=min_shard_bytes, head_block_rows=head_block_rows,
                               frontend=frontend, axis_chunk_rows=axis_chunk_rows)
    return _build(desc), desc


def build_optimizer(cfg, geometry, *, dtype=torch.bfloat16, grad_dtype=None, world_size=1, rank=0,
                    objective=None, lora=None, min_shard_bytes=0, head_block_rows=0, master_weights=False,
                    frontend="stages", axis_chunk_rows=0):
    """The optimizer update alone, over gradients that earlier ``forward_backward``
    invocations left in the spill pool (the ``optim_step`` operation)."""
    desc = TrainingDescription(cfg, geometry, StepDataOrdering(), dtype, grad_dtype or dtype, {},
                               "optimizer", world_size, rank, objective, lora,
                               min_shard_bytes=min_shard_bytes, head_block_rows=head_block_rows,
                               master_weights=master_weights, frontend=frontend,
                               axis_chunk_rows=axis_chunk_rows)
    return _build(desc), desc


def recompute_share_selections(cfg: DecoderConfig, shares=(100, 75, 50, 25, 0),
                               saved_variant: str = "save") -> list[dict[int, str]]:
    """One selection per recompute share: the recomputed layers sit at centred,
    evenly spaced positions in layer order (the reference's resolution rule,
    docs/architecture/graph-pair-selection.md:162-171,198)."""
    n = cfg.n_layers
    out = []
    for share in shares:
        k = round(n * share / 100)
        rec = {int((i + 0.5) * n / k) for i in range(k)} if k else set()
        out.append({li + 1: saved_variant for li in range(n) if li not in rec})
    return out


def mixed_selection(cfg: DecoderConfig, full_save_layers: int, base_variant: str = "save_attention",
                    full_variant: str = "save") -> dict[int, str]:
    """Every layer keeps ``base_variant``; ``full_save_layers`` of them, evenly spaced, keep the
    whole ``full_variant`` set instead. A finer resolution between "attention saved
    everywhere" and "everything saved everywhere" for budgets that afford a little more."""
    n = cfg.n_layers
    k = max(0, min(n, full_save_layers))
    full = {int((i + 0.5) * n / k) for i in range(k)} if k else set()
    return {li + 1: (full_variant if li in full else base_variant) for li in range(n)}
