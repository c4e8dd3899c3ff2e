"""Plan execution: the per-step hot path.

``Executor`` admits a ``Plan`` into a native ``Runtime``, keeps every persistent
tensor in the pinned spill pool between invocations, and on ``run`` stages the
batch, then walks the plan's tasks: ``before_task`` (native: stream waits for
fetched inputs and for the previous occupants of created ranges) -> the stage
function on the compute stream -> ``after_task`` (native: fence + publication
of the triggered fetch / evict / release batch to the worker thread). All
device tensors are views at the plan's fixed offsets; nothing is allocated for
planned objects while stepping.

Reference: packages/engine/src/shadowspill/execution/executor.py:35 (``Executor``),
``run`` :369, hot loop :507-516, dispatch.py:32.
"""
from __future__ import annotations

import math
import time
from dataclasses import dataclass, field

import numpy as np
import torch

from ..data.synthetic import HostMicrobatch
from ..frontend.capture import TrainingDescription, batch_layout, field_spec, saved_layout
from ..ir.plan import Plan
from ..models.decoder import BatchMeta, build_stages
from ..ops import functional as F
from ..runtime.core import Runtime

_TORCH_DT = {"int64": torch.int64, "int32": torch.int32, "float32": torch.float32}


@dataclass
class Hyperparameters:
    lr: float = 1e-4
    beta1: float = 0.9
    beta2: float = 0.95
    eps: float = 1e-8
    weight_decay: float = 0.0
    grad_scale: float = 1.0
    # "adamw" runs the fused kernels (bf16 state with stochastic rounding, fused with the gradient
    # reduce-scatter under data parallelism); "sgd" (momentum beta1) and "lion" run as plain
    # tensor operations with round-to-nearest stores
    rule: str = "adamw"
    # parameter groups: ``(patterns, lr_scale, weight_decay)`` tried in order against
    # "<stage>.<parameter>" (``fnmatch`` patterns); the first match scales the learning rate and,
    # unless its weight_decay is None, replaces the decay. The usual use: no decay on norm vectors.
    # (The reference binds per-group hyperparameters as ``optimizer_group.N.*``:
    # packages/engine/src/shadowspill/build/optimizer.py:49.)
    groups: tuple = ()
    # report the L2 norms of the final gradients and of the weights, taken just before the update
    # (single-worker runs: under sharded storage the summed gradient never exists in memory)
    observe_norms: bool = False

    def rates(self, name: str) -> tuple[float, float]:
        """``(learning rate, weight decay)`` of one parameter."""
        import fnmatch
        for patterns, lr_scale, decay in self.groups:
            if any(fnmatch.fnmatchcase(name, pat) for pat in patterns):
                return self.lr * float(lr_scale), (self.weight_decay if decay is None else float(decay))
        return self.lr, self.weight_decay


@dataclass
class InvocationResult:
    loss: float
    tokens: int
    execution_seconds: float
    device_seconds: float = 0.0
    h2d_bytes: int = 0
    d2h_bytes: int = 0
    task_seconds: list[float] = field(default_factory=list)
    task_start_seconds: list[float] = field(default_factory=list)   # from the step's first event
    trace: list[dict] = field(default_factory=list)
    transfer_begin_ns: list[int] = field(default_factory=list)      # device clock, per action
    transfer_end_ns: list[int] = field(default_factory=list)
    metrics: dict[str, float] = field(default_factory=dict)
    # forward-only programs: one float32 [T, width] array per microbatch (log p(target) per
    # position for language models, the prediction rows of a regression head)
    outputs: list = field(default_factory=list)


class TaskRunner:
    """Turns a program task plus the byte ranges of its objects into the stage
    call it stands for. Shared by the executor (ranges inside the device pool)
    and the profiler (ranges allocated ad hoc)."""

    def __init__(self, program, desc: TrainingDescription, hyper: Hyperparameters, seed: int,
                 stochastic_rounding: bool, collectives=None):
        self.program, self.desc, self.hyper, self.seed = program, desc, hyper, seed
        self.collectives = collectives
        self.world = desc.world_size
        self.sr = stochastic_rounding and desc.dtype == torch.bfloat16
        self.stages = desc.stages()
        meta = program.metadata
        self.T, self.n_mb, self.slots = meta["microbatch_tokens"], meta["n_microbatches"], meta["slots"]
        self.extra_fields = tuple(desc.geometry.extra_fields)
        self.batch_layout_, _ = batch_layout(self.T, self.slots, self.extra_fields)
        self.max_seqlen = [2] * self.n_mb
        self.norm_acc = None          # fp32[2]: sum of squares of gradients, of weights (observe_norms)
        self.uses = [program.sorted_uses(t) for t in range(len(program.tasks))]
        self.completed_updates = 0
        self.accumulated = 0
        self.grad_seen: set[int] = set()
        self.open_gathers: dict[int, list[int]] = {}     # stage -> full-weight buffers awaiting a fused gather
        self.param_offsets, off = {}, 0
        for si, st in enumerate(self.stages):
            for p in st.params:
                self.param_offsets[(si, p.name)] = off
                n = math.prod(p.global_shape) if p.expert_sharded else p.numel
                off += (n + 7) // 8 * 8

    def _batch_meta(self, flat: torch.Tensor, m: int) -> BatchMeta:
        parts = {}
        for name, (off, count, dt) in self.batch_layout_.items():
            tdt = _TORCH_DT[dt]
            parts[name] = flat[off:off + count * tdt.itemsize].view(tdt)
        extras = {}
        for spec in self.extra_fields:
            name, width = field_spec(spec)
            extras[name] = parts[name] if width == 1 else parts[name].view(self.T, width)
        return BatchMeta(parts["tokens"], parts["targets"], parts["weights"], parts["positions"],
                         parts["cu_seqlens"], self.max_seqlen[m], extras)

    def bind(self, task: int, flats: list[torch.Tensor]) -> dict[str, object]:
        """Role -> tensor views for one task over the flat byte tensors of its uses
        (in ``Program.sorted_uses`` order)."""
        t = self.program.tasks[task]
        st = self.stages[t.stage]
        out: dict[str, object] = {}
        for u, flat in zip(self.uses[task], flats):
            obj = self.program.objects[u.object]
            if u.role == "tied_params":
                out[u.role] = self.stages[0].views(flat, self.desc.dtype)
            elif u.role == "tied_grads":
                out[u.role] = self.stages[0].views(flat, self.desc.grad_dtype, torch.float32, True)
            elif u.role in ("params", "m", "v", "shard"):
                only = u.role in ("m", "v")       # moments exist for trainable parameters only
                if obj.sharding == "sharded":
                    out[u.role] = st.shard_views(flat, self.desc.dtype, self.world, only)
                else:
                    out[u.role] = st.views(flat, self.desc.dtype, trainable_only=only)
            elif u.role == "acc":
                out[u.role] = st.shard_views(flat, torch.float32, self.world, True)
            elif u.role == "master":
                if obj.sharding == "sharded":
                    out[u.role] = st.shard_views(flat, torch.float32, self.world, True)
                else:
                    out[u.role] = st.views(flat, torch.float32, trainable_only=True)
            elif u.role == "grads":
                out[u.role] = st.views(flat, self.desc.grad_dtype, torch.float32, True)
            elif u.role in ("x", "y", "dx"):
                out[u.role] = flat.view(self.desc.dtype).view(self.T, self.desc.cfg.d_model)
            elif u.role == "batch":
                out["batch_flat"] = flat
            elif u.role == "loss":
                out[u.role] = flat[:4].view(torch.float32)
            elif u.role == "outputs":
                w = st.output_width
                out[u.role] = flat[:self.T * w * 4].view(torch.float32).view(self.T, w)
            elif u.role == "saved":
                lay, _ = saved_layout(st, self.T, t.variant, self.desc.dtype)
                sv = {}
                for name, shape, dt, off in lay:
                    n = int(np.prod(shape)) * dt.itemsize
                    sv[name] = flat[off:off + n].view(dt).view(shape)
                out[u.role] = sv
            out[f"{u.role}.mode"] = u.mode
        return out

    # ------------------------------------------------------------------ task bodies
    def run_task(self, task: int, B: dict[str, object]) -> None:
        t = self.program.tasks[task]
        st = self.stages[t.stage]
        meta = self._batch_meta(B["batch_flat"], t.microbatch) if "batch_flat" in B else None
        if t.kind == "forward":
            if "saved" in B:
                keep = st.SAVE_SETS.get(t.variant, ())
                _, saved = st.forward(B["params"], B.get("x"), meta, keep, out=B["y"],
                                      saved_out=B["saved"])
                for name, dst in B["saved"].items():     # anything not produced in place
                    src = saved[name]
                    if src.data_ptr() != dst.data_ptr():
                        dst.copy_(src.reshape(dst.shape))
            else:
                st.forward(B["params"], B.get("x"), meta, (), out=B["y"])
        elif t.kind == "head":
            train = t.variant == "train"
            first = self._first(t.stage, B)
            tied = None
            if "tied_params" in B:
                if self.desc.mode == "step":
                    tied_first = B.get("tied_grads.mode") == "create"
                else:   # accumulation driven from outside: fresh on the first contribution
                    tied_first = self.accumulated == 0 and 0 not in self.grad_seen
                    self.grad_seen.add(0)
                tied = {"params": B["tied_params"], "grads": B.get("tied_grads"), "first": tied_first}
            st.loss_and_backward(B["params"], B.get("grads"), B["x"], meta, B["loss"], first,
                                 dx=B.get("dx"), train=train, grad_scale=1.0, tied=tied)
            if "outputs" in B:
                B["outputs"].copy_(st.outputs(B["params"], B["x"], meta, tied))
        elif t.kind == "backward":
            first = self._first(t.stage, B)
            saved = dict(B["saved"]) if "saved" in B else {}
            if "attn" in saved:
                saved["attn"] = saved["attn"]
            from ..ops import delta_rule
            with delta_rule.keeping_intermediates():     # a recomputed forward feeds its own backward
                st.backward(B.get("params"), B.get("grads") or {}, B.get("x"), B["dx"], meta, saved, first)
        elif t.kind == "optimizer":
            if t.variant == "adamw_dp":
                self._optimizer_sharded(t.stage, B)
            else:
                self._optimizer(t.stage, B)
        elif t.kind == "collective" and t.variant == "rs_accumulate":
            # one group's gradients, summed over ranks, folded into this rank's fp32 shard sums
            coll = self.collectives
            first = B.get("acc.mode") == "create"
            coll.barrier_begin()          # every rank's gradients of this group are complete
            for p in st.params:
                if not p.trainable:
                    continue
                g, acc = B["grads"][p.name].view(-1), B["acc"][p.name]
                if p.expert_sharded:      # the local bank's gradient is already the sum over ranks
                    dst = acc.view(-1)[:p.numel]
                    dst.copy_(g) if first else dst.add_(g.float())
                else:
                    coll.reduce_scatter_accumulate(g, acc, first=first,
                                                   whole=st.kept_whole(p, self.desc.dtype))
            coll.barrier_end()            # peers finished reading this rank's gradients
        elif t.kind == "collective" and t.variant == "allgather":
            coll = self.collectives
            coll.barrier_begin()          # every rank's shard has landed
            fuse = ()
            if (self.desc.fused_gather and hasattr(coll, "register_fused_gather")
                    and t.name.rsplit(".", 1)[-1] in ("fwd", "all")):
                fuse = getattr(st, "fused_gather_params", ())
            opened = []
            for p in st.params:
                if p.expert_sharded or st.kept_whole(p, self.desc.dtype):
                    # this rank's own experts, or a small tensor every rank stores whole: no gather
                    B["params"][p.name].view(-1).copy_(B["shard"][p.name][:p.numel])
                elif p.name in fuse and len(p.shape) == 2:
                    # the first GEMM that reads this matrix pulls the shards itself
                    coll.register_fused_gather(B["shard"][p.name], B["params"][p.name])
                    opened.append(B["params"][p.name].data_ptr())
                else:
                    coll.all_gather(B["shard"][p.name], B["params"][p.name].view(-1))
            if opened:
                # closed by close_gathers() after the stage's first forward task: peers read this
                # rank's shard until then
                self.open_gathers[t.stage] = opened
            else:
                coll.barrier_end()        # every rank is done reading this rank's shard
        else:
            raise RuntimeError(f"task kind {t.kind!r} has no executor")

    def close_gathers(self, stage: int) -> None:
        """After the first forward task of ``stage``: gather whatever no GEMM consumed, then wait
        (on the compute stream's own flag words) until every rank is done reading the shards."""
        opened = self.open_gathers.pop(stage, None)
        if not opened:
            return
        F.flush_gathers(set(opened))
        self.collectives.barrier_compute()

    def _first(self, stage: int, B) -> bool:
        if self.desc.mode == "step":
            return B.get("grads.mode") == "create"
        fresh = self.accumulated == 0 and stage not in self.grad_seen
        self.grad_seen.add(stage)
        return fresh

    def _optimizer_sharded(self, stage: int, B) -> None:
        """Gradient reduce-scatter fused with the AdamW update of the owned shards."""
        st, h, coll = self.stages[stage], self.hyper, self.collectives
        coll.barrier_begin()              # every rank's gradients for this stage are complete
        acc = B.get("acc")                # fp32 shard sums of the earlier microbatch groups
        for p in st.params:
            if not p.trainable:
                continue
            lr, wd = h.rates(f"{st.name}.{p.name}")
            if h.rule != "adamw" or "master" in B:
                from ..ops import reference
                hyper = dict(lr=lr, beta1=h.beta1, beta2=h.beta2, eps=h.eps, weight_decay=wd,
                             step=self.completed_updates + 1, grad_scale=h.grad_scale)
                # with master copies the rule runs on the fp32 shard, which is then rounded into
                # the model-dtype shard (both laid out alike)
                target = B["master"][p.name] if "master" in B else B["params"][p.name]
                if p.expert_sharded:
                    own = B["grads"][p.name].view(-1)
                    if acc is not None:
                        own = own.float() + acc[p.name].view(-1)[:p.numel]
                    reference.update_rule_(h.rule, target[:p.numel], own,
                                           B["m"][p.name][:p.numel], B["v"][p.name][:p.numel], **hyper)
                else:
                    coll.reduce_scatter_update(h.rule, B["grads"][p.name].view(-1), target,
                                               B["m"][p.name], B["v"][p.name],
                                               whole=st.kept_whole(p, self.desc.dtype),
                                               acc=None if acc is None else acc[p.name], **hyper)
                if "master" in B:
                    B["params"][p.name].copy_(target)
                continue
            if p.expert_sharded:
                # the local bank's gradient is already the sum over every rank's tokens
                # (expert parallelism routes all of them here): a plain local update
                own = B["grads"][p.name].view(-1)
                if acc is not None:
                    own = own.float() + acc[p.name].view(-1)[:p.numel]
                F.adamw_(B["params"][p.name][:p.numel], own,
                         B["m"][p.name][:p.numel], B["v"][p.name][:p.numel], lr=lr, beta1=h.beta1,
                         beta2=h.beta2, eps=h.eps, weight_decay=wd,
                         step=self.completed_updates + 1, grad_scale=h.grad_scale, seed=self.seed,
                         offset=self.param_offsets[(stage, p.name)] + p.expert_lo * (p.numel // p.shape[0]),
                         stochastic_param=self.sr, stochastic_state=self.sr)
                continue
            coll.reduce_scatter_adamw(
                B["grads"][p.name].view(-1), B["params"][p.name], B["m"][p.name], B["v"][p.name],
                offset=self.param_offsets[(stage, p.name)], lr=lr, beta1=h.beta1, beta2=h.beta2,
                eps=h.eps, weight_decay=wd, step=self.completed_updates + 1,
                grad_scale=h.grad_scale, seed=self.seed, stochastic_param=self.sr,
                stochastic_state=self.sr, whole=st.kept_whole(p, self.desc.dtype),
                **({} if acc is None else {"acc": acc[p.name]}))
        coll.barrier_end()                # peers finished reading this rank's gradients

    def norm_buffers(self, device) -> None:
        """Allocated once, outside any task: the norm observations allocate nothing while a step runs."""
        self.norm_acc = torch.zeros(2, dtype=torch.float32, device=device)
        self._norm_partials = torch.zeros(256, dtype=torch.float32, device=device)
        self._norm_tmp = torch.zeros((), dtype=torch.float32, device=device)

    def _observe(self, grad: torch.Tensor, param: torch.Tensor) -> None:
        """Adds the squares of one parameter's final gradient and of its weights to the step's sums
        (reference: packages/engine/src/shadowspill/training/observations.py:14, ``parameter_norms``)."""
        for slot, x in ((0, grad.reshape(-1)), (1, param.reshape(-1))):
            if x.is_cuda and x.dtype == torch.bfloat16:
                F.sumsq(x, self._norm_partials, self.norm_acc[slot:slot + 1], accumulate=True)
            elif x.is_cuda:                                    # the fp32 vectors: a dot product into a fixed scalar
                torch.dot(x, x, out=self._norm_tmp)
                self.norm_acc[slot].add_(self._norm_tmp)
            else:
                self.norm_acc[slot] += x.float().square().sum()

    def _optimizer(self, stage: int, B) -> None:
        st, h = self.stages[stage], self.hyper
        for p in st.params:
            if not p.trainable:
                continue
            lr, wd = h.rates(f"{st.name}.{p.name}")
            if self.norm_acc is not None:
                self._observe(B["grads"][p.name], B["params"][p.name])
            if "master" in B:
                # fp32 master copy: update it (unfused), then round it into the model-dtype weights
                from ..ops import reference
                master = B["master"][p.name].view(-1)
                reference.update_rule_(h.rule, master, B["grads"][p.name].view(-1),
                                       B["m"][p.name].view(-1), B["v"][p.name].view(-1), lr=lr,
                                       beta1=h.beta1, beta2=h.beta2, eps=h.eps, weight_decay=wd,
                                       step=self.completed_updates + 1, grad_scale=h.grad_scale)
                B["params"][p.name].view(-1).copy_(master)
                continue
            if h.rule != "adamw":
                from ..ops import reference
                reference.update_rule_(h.rule, B["params"][p.name].view(-1), B["grads"][p.name].view(-1),
                                       B["m"][p.name].view(-1), B["v"][p.name].view(-1), lr=lr,
                                       beta1=h.beta1, beta2=h.beta2, eps=h.eps, weight_decay=wd,
                                       step=self.completed_updates + 1, grad_scale=h.grad_scale)
                continue
            F.adamw_(B["params"][p.name].view(-1), B["grads"][p.name].view(-1),
                     B["m"][p.name].view(-1), B["v"][p.name].view(-1), lr=lr, beta1=h.beta1,
                     beta2=h.beta2, eps=h.eps, weight_decay=wd,
                     step=self.completed_updates + 1, grad_scale=h.grad_scale, seed=self.seed,
                     offset=self.param_offsets[(stage, p.name)], stochastic_param=self.sr,
                     stochastic_state=self.sr)


class Executor:
    def __init__(self, plan: Plan, desc: TrainingDescription, *, device: str = "cuda",
                 device_index: int = 0, seed: int = 0, hyper: Hyperparameters | None = None,
                 stochastic_rounding: bool = True, trace_capacity: int = 0,
                 mock_bps: float = 0.0, collectives: str = "auto",
                 extra_plans: dict[str, tuple[Plan, TrainingDescription]] | None = None,
                 file_pool: dict | None = None, annotate: bool = False, moe_chunks: int = 0):
        """``moe_chunks``: under expert parallelism, cut each routed layer's local experts into this
        many groups whose dispatch, GEMMs and combine are pipelined (0 or 1 = one group).
        ``annotate``: wrap every task in an NVTX range named after it (visible in Nsight
        Systems captures; no effect off the GPU).
        ``file_pool``: settings of the file-backed spill pool for plans whose homes were
        moved there (``planning.plan.move_homes_to_file``): ``directory`` or ``image``
        (+ ``create_image``, or ``adopt_image`` with a ``directory``: the image is read-only and
        holds the pool's first bytes) or ``remote`` ("host:port" of a memory daemon), optional
        ``chunk_bytes`` / ``queue_depth`` / ``io_threads``.
        ``collectives``: ``peer`` (own kernels over a symmetric device pool),
        ``dist`` (torch.distributed: NCCL or gloo) or ``auto`` (peer on GPUs).
        ``extra_plans``: further operations (``forward_backward``, ``optim_step``,
        ``forward``) admitted into the same runtime; they must have been planned
        with the same ``StateLayout`` so that persistent tensors share their homes."""
        self.plan, self.desc = plan, desc
        self.program = plan.program
        self.cuda = device == "cuda"
        self.annotate = bool(annotate) and self.cuda
        self.device_index = device_index
        self.torch_device = torch.device(f"cuda:{device_index}") if self.cuda else torch.device("cpu")
        self.hyper = hyper or Hyperparameters()
        if self.hyper.observe_norms and desc.world_size > 1:
            raise ValueError("norm observations are built for single-worker runs: under sharded storage the "
                             "gradient sum is consumed inside the fused update and never exists as a tensor")
        self.seed = seed
        # `world` / `rank`: the shard group this rank stores state with; with replicas the job has
        # world * replicas ranks and `global_rank` is this rank's index among all of them
        self.world, self.rank = desc.world_size, desc.shard_rank
        self.global_rank, self.total_ranks, self.replicas = desc.rank, desc.total_ranks, desc.replicas
        if desc.replicas > 1 and desc.world_size == 1:
            raise NotImplementedError("replicas need a shard group of at least two ranks")
        if desc.replicas > 1 and desc.expert_parallel:
            raise NotImplementedError("expert parallelism runs on one replica")
        extra_plans = dict(extra_plans or {})
        # With the allocation adapter installed, task temporaries are carved from a workspace slice
        # that sits right behind the planned ranges in the same device allocation.
        from ..runtime import allocator as _alloc
        self.allocator = _alloc.installed() if self.cuda else None
        self.workspace_bytes = 0
        if self.allocator is not None:
            ws = max([plan.summary.workspace_bytes] + [p.summary.workspace_bytes for p, _ in extra_plans.values()])
            self.workspace_bytes = -(-int(ws) // 4096) * 4096
        device_bytes = max([plan.device_bytes] + [p.device_bytes for p, _ in extra_plans.values()])
        self.planned_device_bytes = device_bytes
        device_bytes += self.workspace_bytes
        spill_bytes = max([plan.spill_bytes] + [p.spill_bytes for p, _ in extra_plans.values()])
        pool = coll = None
        if self.world > 1:
            from ..parallel import collectives as pc
            mode = ("peer" if device == "cuda" else "dist") if collectives == "auto" else collectives
            if mode == "peer":
                torch.cuda.set_device(device_index)
                pool = pc.allocate_symmetric_pool(device_bytes, self.torch_device)
                coll = pc.PeerCollectives(pool, ranks_per_replica=self.world)
            else:
                coll = pc.DistCollectives(ranks_per_replica=self.world)
        self.collectives = coll
        if self.world > 1:
            # refuse to start if the ranks would not issue the same collectives in the same order
            pc.check_collective_order({"main": plan.program,
                                       **{op: p.program for op, (p, _) in extra_plans.items()}})
        self.runner = TaskRunner(plan.program, desc, self.hyper, seed, stochastic_rounding, coll)
        if self.hyper.observe_norms:
            self.runner.norm_buffers(self.torch_device)
        self.stages = self.runner.stages
        self.ep_group = None
        if desc.expert_parallel and self.world > 1:
            if not self.cuda:
                raise NotImplementedError("expert parallelism needs CUDA devices")
            from ..parallel.expert_parallel import ExpertParallelGroup
            c = desc.cfg
            torch.cuda.set_device(device_index)
            # one symmetric workspace for every routed layer of the model (outside the plan's pool)
            self.ep_group = ExpertParallelGroup(self.runner.T, c.top_k, c.d_model, c.n_experts,
                                                device=self.torch_device)
            if moe_chunks > 1:
                self.ep_group.pipeline_chunks = int(moe_chunks)
            self._bind_expert_group(self.runner)
        if self.cuda:
            torch.cuda.set_device(device_index)
            from ..ops import _lib
            _lib.lib()   # fail loudly if the kernel library is missing
        file_bytes = max([plan.file_bytes] + [p.file_bytes for p, _ in extra_plans.values()])
        fp = dict(file_pool or {})
        if file_bytes > 0 and not (fp.get("directory") or fp.get("image") or fp.get("remote")):
            raise ValueError("the plan homes objects in a file pool: pass file_pool={'directory': ...} "
                             "(or 'image', or 'remote': 'host:port' of a memory daemon)")
        self.rt = Runtime(device_bytes, spill_bytes, "cuda" if self.cuda else "mock",
                          device_index, trace_capacity=trace_capacity, mock_bps=mock_bps,
                          device_pool=pool, file_bytes=file_bytes,
                          file_directory=str(fp.get("directory", "")), file_image=str(fp.get("image", "")),
                          file_create_image=bool(fp.get("create_image", False)),
                          file_adopt_image=bool(fp.get("adopt_image", False)),
                          file_chunk_bytes=int(fp.get("chunk_bytes", 0)),
                          file_queue_depth=int(fp.get("queue_depth", 0)),
                          file_io_threads=int(fp.get("io_threads", 0)),
                          remote_address=str(fp.get("remote", "")))
        # host mirrors of file-homed objects handed out by spill_view, written back before
        # the next step: {file offset: (tensor, writable)}
        self._mirrors: dict[int, tuple[torch.Tensor, bool]] = {}
        self.plan_id = self.rt.admit(plan)
        self.stream = torch.cuda.Stream(device=self.torch_device) if self.cuda else None
        # Collective tasks (weight all-gathers, the fused reduce-scatter + update) run on a stream of
        # their own, as the reference issues them on the transfer lane's route stream
        # (packages/engine/csrc/adapter/pytorch/storage/sharded.cpp:87-122), so they overlap the
        # compute tasks around them. SS_COMM_STREAM=0 keeps them on the compute stream.
        import os
        self.comm_stream = (torch.cuda.Stream(device=self.torch_device)
                            if (self.cuda and self.world > 1 and os.environ.get("SS_COMM_STREAM", "1") == "1")
                            else None)
        if self.allocator is not None:
            self.allocator.configure(self.rt.device_base + self.planned_device_bytes, self.workspace_bytes,
                                     self.stream.cuda_stream)
        self._views: dict[tuple[int, int], object] = {}
        self._uses = self.runner.uses
        self.T, self.n_mb, self.slots = self.runner.T, self.runner.n_mb, self.runner.slots
        self._batch_layout = self.runner.batch_layout_
        self._obj = {o.name: i for i, o in enumerate(self.program.objects)}
        self._loss_obj = self._obj.get("loss", -1)
        self.closed = False
        self.operation = {"step": "step", "forward_backward": "forward_backward",
                          "forward": "forward", "optimizer": "optim_step"}.get(desc.mode, desc.mode)
        self._primary = self._snapshot()
        self._bound = {self.operation: self._primary}
        for name, (xplan, xdesc) in extra_plans.items():
            self._bound[name] = self._bind_extra(xplan, xdesc, stochastic_rounding)

    # ------------------------------------------------------------------ several plans, one state
    _PLAN_FIELDS = ("plan", "desc", "program", "runner", "plan_id", "_views", "_uses", "T", "n_mb",
                    "slots", "_batch_layout", "_obj", "_loss_obj")

    def _snapshot(self) -> dict:
        return {k: getattr(self, k) for k in self._PLAN_FIELDS}

    def _bind_expert_group(self, runner: "TaskRunner") -> None:
        for st in runner.stages:
            if getattr(st, "ep_world", 1) > 1:
                st.ep_group = self.ep_group

    def _bind_extra(self, plan: Plan, desc: TrainingDescription, sr: bool) -> dict:
        runner = TaskRunner(plan.program, desc, self.hyper, self.seed, sr, self.collectives)
        if self.runner.norm_acc is not None:          # one set of observation buffers for every operation's plan
            runner.norm_acc, runner._norm_partials, runner._norm_tmp = (
                self.runner.norm_acc, self.runner._norm_partials, self.runner._norm_tmp)
        if self.ep_group is not None:
            self._bind_expert_group(runner)
        obj = {o.name: i for i, o in enumerate(plan.program.objects)}
        # persistent tensors of the same name must live at the same spill offset
        for name, i in obj.items():
            j = self._obj.get(name)
            if (j is not None and plan.program.objects[i].persistent
                    and self.program.objects[j].persistent
                    and (plan.spill_offsets[i] != self.plan.spill_offsets[j]
                         or plan.home_pool(i) != self.plan.home_pool(j)
                         or (plan.home_pool(i) == "file"
                             and plan.file_offsets[i] != self.plan.file_offsets[j]))):
                raise ValueError(f"plans disagree on the spill home of {name}")
        return {"plan": plan, "desc": desc, "program": plan.program, "runner": runner,
                "plan_id": self.rt.admit(plan), "_views": {}, "_uses": runner.uses, "T": runner.T,
                "n_mb": runner.n_mb, "slots": runner.slots, "_batch_layout": runner.batch_layout_,
                "_obj": obj, "_loss_obj": obj.get("loss", -1)}

    def _select(self, operation: str) -> None:
        """Makes ``operation``'s plan the current one (counters travel with the executor)."""
        if operation not in self._bound:
            raise KeyError(f"no plan admitted for operation {operation!r}; "
                           f"have {sorted(self._bound)}")
        done, acc = self.runner.completed_updates, self.runner.accumulated
        for k, v in self._bound[operation].items():
            setattr(self, k, v)
        self.runner.completed_updates, self.runner.accumulated = done, acc
        self.runner.hyper = self.hyper

    def operations(self) -> list[str]:
        return sorted(self._bound)

    def operation_name(self) -> str:
        """Name of the operation whose plan is currently selected."""
        for name, bound in self._bound.items():
            if bound["plan_id"] == self.plan_id:
                return name
        return self.operation

    # ------------------------------------------------------------------ state in the spill pool
    def spill_view(self, obj: int, writable: bool = True) -> torch.Tensor:
        """The object's home as host bytes. In the pinned pool this is a view. For an object
        homed in the file pool it is a host mirror read from the file; a writable mirror is
        written back by ``flush_homes`` (which every step calls first), so changes made
        through it reach the file before any fetch can read them."""
        nbytes = self.program.objects[obj].bytes
        if self.plan.home_pool(obj) == "file":
            off = self.plan.file_offsets[obj]
            hit = self._mirrors.get(off)
            if hit is not None and hit[0].numel() == nbytes:
                if writable and not hit[1]:
                    self._mirrors[off] = (hit[0], True)
                return hit[0]
            mirror = self.rt.file_read(off, nbytes)
            self._mirrors[off] = (mirror, writable)
            return mirror
        off = self.plan.spill_offsets[obj]
        if off < 0:
            raise KeyError(f"{self.program.objects[obj].name} has no spill home")
        return self.rt.spill[off:off + nbytes]

    def release_mirrors(self) -> None:
        """Forgets read-only mirrors (their memory goes once the caller lets go of its views)."""
        for off in [o for o, (_, writable) in self._mirrors.items() if not writable]:
            del self._mirrors[off]

    def flush_homes(self) -> int:
        """Writes every writable mirror back to the file pool and drops all mirrors;
        returns the bytes written."""
        total = 0
        for off, (mirror, writable) in sorted(self._mirrors.items()):
            if writable:
                self.rt.file_write(off, mirror)
                total += mirror.numel()
        self._mirrors.clear()
        return total

    def initialize(self, seed: int | None = None, on_device: bool | None = None) -> None:
        """Random initialisation of the spill homes (seed-only, so the result does
        not depend on plan, budget or sharding); moments start at zero.
        ``on_device`` draws each stage on the GPU and copies it down, which is what
        makes multi-billion-parameter models initialise in seconds; the CPU
        generator is the default off-GPU and gives the same values everywhere."""
        on_device = self.cuda if on_device is None else on_device
        seed = self.seed if seed is None else seed
        gen = (torch.Generator(device=self.torch_device) if on_device else torch.Generator())
        gen.manual_seed(seed)
        for si, st in enumerate(self.stages):
            w = self.spill_view(self._obj[f"{st.name}.weights"])
            _, full_bytes = st.layout(self.desc.dtype)
            dev = self.torch_device if on_device else torch.device("cpu")
            if self.world == 1 and not on_device:
                w.zero_()
                st.init_(st.views(w, self.desc.dtype), gen)
            else:
                # every rank draws the whole stage from the same seed, then keeps its slices
                if on_device and self.rt.device.numel() >= full_bytes:
                    # between steps the planned device pool holds nothing: stage in it
                    # instead of asking the (capped) torch allocator for a whole stage
                    flat = self.rt.device[:full_bytes].zero_()
                else:
                    flat = torch.zeros(full_bytes, dtype=torch.uint8, device=dev)
                full = st.views(flat, self.desc.dtype)
                st.init_(full, gen)
                if self.world == 1:
                    w.copy_(flat)
                else:
                    w.zero_()
                    shards = st.shard_views(w, self.desc.dtype, self.world)
                    for p in st.params:
                        src, dst = full[p.name].reshape(-1), shards[p.name]
                        if p.expert_sharded or st.kept_whole(p, self.desc.dtype):
                            dst[:src.numel()].copy_(src)
                            continue
                        lo = self.rank * dst.numel()
                        hi = min(src.numel(), lo + dst.numel())
                        if hi > lo:
                            dst[:hi - lo].copy_(src[lo:hi])
                if on_device:
                    torch.cuda.synchronize(self.torch_device)
                del flat
            for suffix in ("exp_avg", "exp_avg_sq", "gradients"):
                name = f"{st.name}.{suffix}"
                if name in self._obj and self.plan.home_pool(self._obj[name]):
                    self.spill_view(self._obj[name]).zero_()
            self._sync_master(st)
            if self._mirrors:
                self.flush_homes()      # file-homed state: one stage in host memory at a time
        self.runner.completed_updates = 0
        self.runner.accumulated = 0

    def _sync_master(self, st) -> None:
        """fp32 master copy of a stage := its current weights (after initialisation or a load)."""
        name = f"{st.name}.master"
        if name not in self._obj:
            return
        w = self.spill_view(self._obj[f"{st.name}.weights"], False)
        mflat = self.spill_view(self._obj[name])
        if self.world > 1:
            src = st.shard_views(w, self.desc.dtype, self.world)
            dst = st.shard_views(mflat, torch.float32, self.world, True)
        else:
            src = st.views(w, self.desc.dtype)
            dst = st.views(mflat, torch.float32, trainable_only=True)
        for k, d in dst.items():
            d.copy_(src[k].reshape(d.shape))

    def named_tensors(self, writable: bool = True):
        """Yields ``(name, tensor view in the spill pool)`` for every persistent
        model tensor: parameters, then ``exp_avg.*`` / ``exp_avg_sq.*``."""
        for si, st in enumerate(self.stages):
            for kind, prefix in (("weights", ""), ("exp_avg", "exp_avg."), ("exp_avg_sq", "exp_avg_sq."),
                                 ("master", "master.")):
                name = f"{st.name}.{kind}"
                if name not in self._obj:
                    continue
                flat = self.spill_view(self._obj[name], writable)
                only = kind != "weights"      # moments and masters exist for trainable parameters only
                dt = torch.float32 if kind == "master" else self.desc.dtype
                if self.world > 1:
                    views = st.shard_views(flat, dt, self.world, only)
                else:
                    views = st.views(flat, dt, trainable_only=only)
                for p in st.params:
                    if p.name in views:
                        yield f"{prefix}{st.name}.{p.name}", views[p.name]

    def state_dict(self) -> dict[str, torch.Tensor]:
        return {k: v.clone() for k, v in self.named_tensors(writable=False)}

    def load_state_dict(self, state: dict[str, torch.Tensor], strict: bool = True) -> None:
        seen = set()
        for k, v in self.named_tensors():
            if k in state:
                v.copy_(state[k].to(v.dtype).reshape(v.shape))
                seen.add(k)
            elif strict:
                raise KeyError(f"missing tensor {k}")
        extra = set(state) - seen
        if strict and extra:
            raise KeyError(f"unexpected tensors {sorted(extra)[:4]}")
        if not any(k.startswith("master.") for k in state):
            for st in self.stages:          # weights came without masters: derive them
                self._sync_master(st)

    def load_full_state_dict(self, state: dict[str, torch.Tensor], strict: bool = True) -> None:
        """Loads WHOLE parameters (``{"<stage>.<param>": tensor}``, for example a converted
        Hugging Face checkpoint) into this rank's homes: with sharded storage every rank keeps
        its 1/N slice of each tensor, with expert parallelism its own rows of each bank.
        Moments are left as they are. Parameters the state does not name keep their values
        unless ``strict``."""
        if self.world == 1:
            if strict:
                for st in self.stages:
                    for p in st.params:
                        if f"{st.name}.{p.name}" not in state:
                            raise KeyError(f"missing tensor {st.name}.{p.name}")
            self.load_state_dict(state, strict=False)
            return
        for st in self.stages:
            name = f"{st.name}.weights"
            if name not in self._obj:
                continue
            shards = st.shard_views(self.spill_view(self._obj[name]), self.desc.dtype, self.world)
            for p in st.params:
                key = f"{st.name}.{p.name}"
                if key not in state:
                    if strict:
                        raise KeyError(f"missing tensor {key}")
                    continue
                src, dst = state[key], shards[p.name]
                if p.expert_sharded:
                    want = tuple(p.global_shape)
                    if tuple(src.shape) != want:
                        raise ValueError(f"{key}: shape {tuple(src.shape)} != {want}")
                    rows = src[p.expert_lo:p.expert_lo + p.shape[0]].reshape(-1)
                    dst[:rows.numel()].copy_(rows.to(dst.dtype))
                    continue
                if src.numel() != p.numel:
                    raise ValueError(f"{key}: {src.numel()} elements, expected {p.numel}")
                flat = src.reshape(-1)
                lo = 0 if st.kept_whole(p, self.desc.dtype) else self.rank * dst.numel()
                hi = min(flat.numel(), lo + dst.numel())
                dst.zero_()
                if hi > lo:
                    dst[:hi - lo].copy_(flat[lo:hi].to(dst.dtype))
            self._sync_master(st)

    # ------------------------------------------------------------------ inputs
    def stage_inputs(self, batch: list[HostMicrobatch]) -> int:
        """Writes the packed microbatches into their spill homes; returns bytes staged."""
        if len(batch) != self.n_mb:
            raise ValueError(f"plan expects {self.n_mb} microbatches, got {len(batch)}")
        total = 0
        for m, mb in enumerate(batch):
            if mb.tokens.shape[0] != self.T:
                raise ValueError(f"microbatch {m}: {mb.tokens.shape[0]} tokens, plan expects {self.T}")
            if mb.cu_seqlens.shape[0] > self.slots + 1:
                raise ValueError(f"microbatch {m}: too many sequences for {self.slots} slots")
            dst = self.spill_view(self._obj[f"batch.{m}"]).numpy()
            for name, (off, count, dt) in self._batch_layout.items():
                src = getattr(mb, name) if hasattr(mb, name) else mb.extras[name]
                view = dst[off:off + count * np.dtype(dt).itemsize].view(dt)
                if name == "cu_seqlens":
                    view[:src.shape[0]] = src
                    view[src.shape[0]:] = src[-1]
                else:
                    view[:] = np.asarray(src).reshape(-1)
                total += view.nbytes
            self.runner.max_seqlen[m] = int(mb.max_seqlen)
        return total

    # ------------------------------------------------------------------ views
    def _device_view(self, ptr: int, nbytes: int) -> torch.Tensor:
        # An alias with its own autograd version counter (not a view of the pool tensor):
        # in-place writes to one object must not invalidate tensors autograd saved from
        # another object that merely lives in the same pool.
        off = ptr - self.rt.device_base
        pool = self.rt.device
        return torch.empty(0, dtype=torch.uint8, device=pool.device).set_(
            pool.untyped_storage(), pool.storage_offset() + off, (nbytes,))

    def _bind(self, task: int, ptrs: list[int]) -> dict[str, object]:
        """Views for one task, cached: the plan fixes every offset."""
        key = (task, hash(tuple(ptrs)))
        hit = self._views.get(key)
        if hit is None:
            flats = [self._device_view(ptr, self.program.objects[u.object].bytes)
                     for u, ptr in zip(self._uses[task], ptrs)]
            hit = self._views[key] = self.runner.bind(task, flats)
        return hit

    @property
    def completed_updates(self) -> int:
        return self.runner.completed_updates

    @completed_updates.setter
    def completed_updates(self, value: int) -> None:
        self.runner.completed_updates = value

    @property
    def accumulated(self) -> int:
        return self.runner.accumulated

    # ------------------------------------------------------------------ run
    def run(self, batch: list[HostMicrobatch] | None = None, *, operation: str | None = None,
            trace: bool = False, time_tasks: bool = False) -> InvocationResult:
        if self.closed:
            raise RuntimeError("executor is closed")
        t0 = time.perf_counter()
        self._select(operation or self.operation)
        try:
            return self._run(batch, trace, time_tasks, t0)
        finally:
            self._select_primary()

    def _select_primary(self) -> None:
        done, acc = self.runner.completed_updates, self.runner.accumulated
        for k, v in self._primary.items():
            setattr(self, k, v)
        self.runner.completed_updates, self.runner.accumulated = done, acc

    def _run(self, batch, trace: bool, time_tasks: bool, t0: float) -> InvocationResult:
        if self.total_ranks > 1:
            # host-side work first, then agreement: a rank whose batch is bad (or which raised for
            # any other reason) stops every rank before the first collective is enqueued
            from ..parallel import control

            def prepare():
                control.check_invocation(self.operation_name(), self.runner.accumulated)
                return self.stage_inputs(batch) if self.n_mb and batch is not None else 0
            h2d = control.coordinated(prepare)
        else:
            h2d = self.stage_inputs(batch) if self.n_mb and batch is not None else 0
        if self._loss_obj >= 0:
            self.spill_view(self._loss_obj).zero_()
        self.runner.grad_seen = set()
        if trace:
            self.rt.trace_begin()
        n_tasks = len(self.program.tasks)
        events = None
        if self.cuda:
            start_ev, end_ev = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            if time_tasks:
                events = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
                          for _ in range(n_tasks)]
            ctx = torch.cuda.stream(self.stream)
            ctx.__enter__()
            start_ev.record(self.stream)
        task_seconds = [0.0] * n_tasks
        try:
            if self._mirrors:
                self.flush_homes()
            self.rt.step_begin(self.plan_id, self.stream.cuda_stream if self.cuda else None)
            pending: dict[int, torch.cuda.Event] = {}     # object -> end of the side-stream task using it
            tasks = self.program.tasks
            for task in range(n_tasks):
                t = tasks[task]
                side = self.comm_stream is not None and (t.kind == "collective" or t.variant == "adamw_dp")
                run_stream = self.comm_stream if side else self.stream
                if side:
                    if t.kind != "collective" or t.variant == "rs_accumulate":
                        # reads what compute tasks produced (gradients): order after them. A weight
                        # gather depends on fetches and freed ranges only, which the runtime orders.
                        ready = torch.cuda.Event()
                        ready.record(self.stream)
                        self.comm_stream.wait_event(ready)
                    ptrs = self.rt.before_task(self.plan_id, task, len(self._uses[task]),
                                               stream=self.comm_stream.cuda_stream)
                else:
                    if pending:
                        for u in self._uses[task]:
                            ev = pending.pop(u.object, None)
                            if ev is not None:
                                self.stream.wait_event(ev)
                    ptrs = self.rt.before_task(self.plan_id, task, len(self._uses[task]))
                B = self._bind(task, ptrs)
                if self.allocator is not None:
                    self.allocator.begin_task(t.name, 2 if (t.allocations and not side) else 0,
                                              t.allocations if not side else None)
                if events:
                    events[task][0].record(run_stream)
                elif not self.cuda and time_tasks:
                    tt = time.perf_counter()
                if self.annotate:
                    torch.cuda.nvtx.range_push(t.name)
                if side:
                    with torch.cuda.stream(self.comm_stream):
                        self.runner.run_task(task, B)
                else:
                    self.runner.run_task(task, B)
                    if self.runner.open_gathers and t.stage in self.runner.open_gathers:
                        self.runner.close_gathers(t.stage)     # inside the task: its fence covers the barrier
                if self.annotate:
                    torch.cuda.nvtx.range_pop()
                if events:
                    events[task][1].record(run_stream)
                elif not self.cuda and time_tasks:
                    task_seconds[task] = time.perf_counter() - tt
                if self.allocator is not None:
                    self.allocator.end_task()
                    self.allocator.raise_if_failed()     # OutOfMemoryError / contract violation naming the task
                if side:
                    self.rt.after_task(self.plan_id, task, stream=self.comm_stream.cuda_stream)
                    done = torch.cuda.Event()
                    done.record(self.comm_stream)
                    for u in self._uses[task]:
                        pending[u.object] = done
                else:
                    self.rt.after_task(self.plan_id, task)
            for ev in set(pending.values()):          # the step ends when the side stream has ended
                self.stream.wait_event(ev)
            if self.cuda:
                end_ev.record(self.stream)
            self.rt.step_end(self.plan_id)
        except BaseException as exc:
            # a task raised inside the step: the pool's contents are undefined from here on, so the
            # runtime goes terminal (as after any latched failure) and the plan becomes closable
            if self.allocator is not None:
                try:
                    self.allocator.end_task()
                except RuntimeError:
                    pass                       # the scope was closed before the error was raised
            self.rt.step_abandon(self.plan_id, f"{type(exc).__name__} in a task: {exc}")
            raise
        finally:
            if self.cuda:
                ctx.__exit__(None, None, None)
        loss = (float(self.spill_view(self._loss_obj)[:4].view(torch.float32)[0])   # device -> host
                if self._loss_obj >= 0 else 0.0)
        device_seconds = 0.0
        task_starts: list[float] = []
        if self.cuda:
            device_seconds = start_ev.elapsed_time(end_ev) * 1e-3
            if events:
                task_seconds = [a.elapsed_time(b) * 1e-3 for a, b in events]
                task_starts = [start_ev.elapsed_time(a) * 1e-3 for a, _ in events]
        if self.desc.mode in ("step", "optimizer"):
            self.runner.completed_updates += 1
            self.runner.accumulated = 0
        elif self.desc.mode == "forward_backward":
            self.runner.accumulated += 1
        metrics = {}
        if self.runner.norm_acc is not None and self.desc.mode in ("step", "optimizer"):
            g2, p2 = (float(v) for v in self.runner.norm_acc.tolist())
            metrics["grad_norm"] = (g2 ** 0.5) * abs(self.hyper.grad_scale)
            metrics["param_norm"] = p2 ** 0.5
            self.runner.norm_acc.zero_()
        aux = [st.aux_sum for st in self.stages if getattr(st, "aux_sum", None) is not None]
        if aux:
            metrics["moe_balance"] = float(sum(float(a.item()) for a in aux))
            for a in aux:
                a.zero_()
        tr = self.rt.trace_end() if trace else []
        tb, te = (self.rt.transfer_times(self.plan_id, len(self.plan.schedule.actions))
                  if trace else ([], []))
        outputs, d2h = [], 4
        for m in range(self.n_mb):
            o = self._obj.get(f"outputs.{m}")
            if o is None:
                break
            w = self.stages[-1].output_width
            outputs.append(self.spill_view(o, False)[:self.T * w * 4].view(torch.float32)
                           .view(self.T, w).numpy().copy())
            d2h += outputs[-1].nbytes
        return InvocationResult(loss, self.T * self.n_mb, time.perf_counter() - t0, device_seconds,
                                h2d, d2h, task_seconds if time_tasks else [], task_starts, tr, tb, te,
                                metrics, outputs)

    def discard_gradients(self) -> None:
        self.runner.accumulated = 0

    def close(self) -> None:
        if self.closed:
            return
        self.closed = True
        if self.cuda:
            torch.cuda.synchronize(self.torch_device)
        try:
            if self._mirrors and self.rt.failure() is None:
                self.flush_homes()          # a kept pool image must hold the latest state
            for b in self._bound.values():
                b["_views"].clear()
                self.rt.close_plan(b["plan_id"])
            if self.allocator is not None:
                try:
                    self.allocator.configure(0, 0)
                except RuntimeError:
                    pass                      # a caller still holds a tensor from the slice
        finally:
            self.rt.close()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()
