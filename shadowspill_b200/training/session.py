"""In-process training composition: build -> profile -> calibrate -> plan -> execute.

``TrainingSession`` is what one worker process runs for one rank: it resolves a
``TrainingSetup`` into a model configuration and batch geometry, builds the
candidate programs (walk orders x save/recompute selections), profiles their
distinct tasks on the device, calibrates the host link, plans every candidate
under the memory budget and keeps the fastest, then admits that plan into an
``Executor``. ``step`` takes the global batch as host arrays and returns the
host-side result. The service layer wraps exactly this object per worker.

Reference: packages/engine/src/shadowspill/training/preparation/phases/operations.py
(build :39, profile :92, communicate :129, plan :199) and
training/worker/runtime.py:195 (``PreparedWorker.open``).
"""
from __future__ import annotations

import json
import time
from pathlib import Path
from dataclasses import dataclass, field

import torch

from ..communication.info import CommunicationInfo
from ..data.synthetic import HostMicrobatch
from ..execution.executor import Executor, Hyperparameters, InvocationResult
from ..frontend.capture import (BatchGeometry, StepDataOrdering, build_forward,
                                build_forward_backward, build_optimizer, build_step,
                                recompute_share_selections)
from ..models.config import DecoderConfig, preset
from ..planning.plan import (MemoryBudgets, PlanningError, SearchOptions, StateLayout,
                             plan_program, sweep_programs)
from ..profiling.measure import Profiles, apply_profiles, measure_program
from ..runtime.core import Runtime

GIB = 1 << 30


@dataclass
class TrainingSetup:
    model: str | DecoderConfig = "llama3-8b"
    device_gib: float = 24.0
    spill_gib: float = 128.0
    tokens_per_step: int = 65536          # per worker
    microbatch_tokens: int = 8192
    slots: int = 0                        # 0 = derived from the microbatch size
    mean_seqlen: float = 2048.0
    lr: float = 1e-4
    beta1: float = 0.9
    beta2: float = 0.95
    eps: float = 1e-8
    weight_decay: float = 0.0
    # parameter groups, first match wins: {"match": ["*norm*"], "lr_scale": 1.0, "weight_decay": 0.0}
    # (patterns against "<stage>.<parameter>"; weight_decay None or absent = the run's own)
    parameter_groups: tuple = ()
    observe_norms: bool = False          # report grad_norm / param_norm of every update (single-worker runs)
    # added to the planned duration of every task that runs on the communication stream (collectives,
    # the sharded update): what such a task costs the compute lane beyond the modelled share, as a
    # traced step shows it (qualification/gap_report.py prints the measured figure)
    collective_overhead_us: float = 0.0
    # adamw | sgd (momentum beta1) | lion, or the captured update of any elementwise
    # torch.optim optimizer (frontend/optimizer_capture.py: capture_optimizer_update)
    optimizer_rule: object = "adamw"
    seed: int = 0
    dtype: str = "bfloat16"
    stochastic_rounding: bool = True
    device: str = "cuda"
    device_index: int = 0
    rank: int = 0
    world_size: int = 1
    walks: tuple[str, ...] = ("breadth",)   # breadth | depth | breadth/<microbatch groups>
    recompute_shares: tuple[int, ...] = (100,)
    saved_variant: str = "save_attention"
    # explicit "<recompute share>:<saved variant>" candidates (e.g. "50:save") or "mix:<K>"
    # (attention saved on every layer, K layers saved whole); when given they replace the
    # recompute_shares x saved_variant grid
    candidate_selections: tuple[str, ...] = ()
    profile: bool = True
    calibrate: bool = True
    # scale burst-measured task profiles to sustained clocks with both lanes streaming
    calibrate_overlap: bool = True
    search: SearchOptions = field(default_factory=SearchOptions)
    trace_capacity: int = 0
    collectives: str = "auto"             # peer | dist | auto
    # prepared bundle (training.ssp): read when it matches this setup, written after planning
    bundle: str = ""
    # training choices beyond the architecture (JSON records, see models/lora.py, models/objectives.py)
    lora: dict | None = None
    objective: dict | None = None
    expert_parallel: bool = False        # routed layers keep 1/world of the experts per rank
    ranks_per_replica: int = 0           # 0 = one replica; else state is sharded inside groups of this size
    min_shard_bytes: int = 0             # sharded storage keeps smaller tensors whole on every rank
    head_chunks: int = 0                 # evaluate the output projection in this many row chunks (0 = default)
    moe_chunks: int = 0                  # expert parallelism: pipeline each routed layer in this many expert groups
    master_weights: bool = False         # fp32 master copies of trainable parameters (unfused update path)
    # "graph": torch.export -> stage partition -> AOT save/recompute graph pairs for the models the
    # graph frontend covers (frontend/graph_stage.py); "stages": the hand-written stage classes
    frontend: str = "stages"
    # "planned": install the allocation adapter (runtime/allocator.py) before the first CUDA use:
    # task temporaries then come out of a workspace slice of the device pool under a checked
    # per-task contract. "caching": torch's caching allocator, capped to the planned workspace.
    allocator: str = "caching"
    # sharded data parallelism on GPUs with the peer collectives: fuse the forward weight gather
    # into the consuming GEMM
    fused_gather: bool = False
    # graph frontend: row chunk of the token-local operators inside a layer stage (0 = off); what
    # lets one long sequence fit: the wide projection outputs then exist one chunk at a time
    axis_chunk_rows: int = 0
    # gated delta rule: run each call in this many groups of key heads (1 = all at once); the chunk
    # intermediates then exist for one group at a time
    delta_head_groups: int = 1
    # profile the tasks on sequences of exactly this many tokens (0 = the packed log-normal mix):
    # the cost of the sequence mixers depends on it, so long-context runs set it
    profile_sequence_tokens: int = 0
    # preparation as separate processes (training/phases.py): a session stops after the named
    # phase ("build" | "profile" | "communicate" | "plan") having written that phase's result
    # into phase_directory; later phases read the earlier results from there instead of measuring
    stop_after: str = ""
    phase_directory: str = ""
    pretrained: str = ""                 # directory of Hugging Face safetensors to start from
    # content-addressed store of task profiles shared between runs ("" = none)
    store: str = ""
    store_mode: str = "read_write"
    operations: tuple[str, ...] = ("step",)   # also: forward_backward, optim_step, forward
    # spilled state in pinned host memory ("host") or in a direct-I/O file ("file"): then
    # spill_gib is the file's size and only batches and the loss word stay pinned
    # ... or in the memory of an ss_memory_daemon on another machine ("remote", spill_address)
    profiler_annotations: bool = False    # NVTX range per task
    spill_pool: str = "host"
    spill_address: str = ""               # "remote": host:port of the daemon
    spill_directory: str = ""             # existing directory for the unlinked scratch file
    spill_image: str = ""                 # or a named file that is kept when the run closes
    spill_create_image: bool = False
    spill_chunk_bytes: int = 2 << 20
    spill_queue_depth: int = 16


_DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32}


def _selection_label(selection: dict) -> str:
    if not selection:
        return "recompute"
    kinds: dict[str, int] = {}
    for v in selection.values():
        kinds[v] = kinds.get(v, 0) + 1
    return ", ".join(f"{k} x{n}" for k, n in sorted(kinds.items()))


class TrainingSession:
    def __init__(self, setup: TrainingSetup, log=None):
        self.setup = setup
        self.log = log or (lambda msg: None)
        self.cfg = setup.model if isinstance(setup.model, DecoderConfig) else preset(setup.model)
        self.dtype = _DTYPES[setup.dtype]
        if setup.allocator == "planned" and setup.device == "cuda":
            from ..runtime import allocator as _alloc
            _alloc.install()
        elif setup.allocator not in ("planned", "caching"):
            raise ValueError("allocator is 'planned' or 'caching'")
        cuda = setup.device == "cuda"
        if setup.tokens_per_step % setup.microbatch_tokens:
            raise ValueError("tokens_per_step must be a multiple of microbatch_tokens")
        self.slots = setup.slots or max(16, setup.microbatch_tokens // 32 + 1)
        if self.cfg.family == "regression":
            if self.dtype != torch.float32:
                raise ValueError("the regression family trains in float32")
            self.slots = max(self.slots, setup.microbatch_tokens + 1)   # every row is its own datum
        self.geometry = BatchGeometry(setup.microbatch_tokens,
                                      setup.tokens_per_step // setup.microbatch_tokens,
                                      self.slots, setup.mean_seqlen)
        self.budgets = MemoryBudgets.from_gib(setup.device_gib, setup.spill_gib)
        self.timings: dict[str, float] = {}
        world, rank = setup.world_size, setup.rank
        self.executor = None
        if setup.delta_head_groups != 1:
            from ..ops import delta_rule
            delta_rule.set_head_groups(setup.delta_head_groups)
        if setup.stop_after not in ("", "build", "profile", "communicate", "plan"):
            raise ValueError("stop_after is one of build, profile, communicate, plan")
        phase_dir = Path(setup.phase_directory) if setup.phase_directory else None
        if setup.stop_after and phase_dir is None:
            raise ValueError("stop_after needs phase_directory")
        if phase_dir is not None:
            phase_dir.mkdir(parents=True, exist_ok=True)

        def phase_result(name: str):
            f = phase_dir / f"{name}.json" if phase_dir is not None else None
            return json.loads(f.read_text()) if (f is not None and f.exists()) else None
        if setup.candidate_selections:
            selections = []
            for item in setup.candidate_selections:
                share, _, variant = item.partition(":")
                if share == "mix":        # "mix:K[:variant]": save_attention everywhere, K layers keep more
                    from ..frontend.capture import mixed_selection
                    count, _, full = variant.partition(":")
                    selections.append(mixed_selection(self.cfg, int(count), full_variant=full or "save"))
                    continue
                selections += recompute_share_selections(self.cfg, (int(share),),
                                                         variant or setup.saved_variant)
        else:
            selections = recompute_share_selections(self.cfg, setup.recompute_shares,
                                                    setup.saved_variant)
        variants = [(walk, sel) for walk in setup.walks for sel in selections]

        from ..models.lora import LoRAConfig
        from ..models.objectives import Objective
        self.lora = LoRAConfig.from_json(setup.lora)
        self.objective = Objective.from_json(setup.objective) if setup.objective else None
        graph_covers = False
        if setup.frontend == "graph":
            from ..frontend.graph_stage import supports
            graph_covers = supports(self.cfg, self.lora, (world, rank) if setup.expert_parallel else None,
                                    self.objective)
        if (self.lora is not None or setup.expert_parallel) and not graph_covers:
            # these layers run through the autograd-derived stage, which only recomputes
            selections = [{}]
            variants = [(walk, {}) for walk in setup.walks]
        choices = dict(objective=self.objective, lora=self.lora, frontend=setup.frontend,
                       axis_chunk_rows=setup.axis_chunk_rows if setup.frontend == "graph" else 0)
        shard_world = setup.ranks_per_replica or world
        if world % shard_world:
            raise ValueError("world_size must be a multiple of ranks_per_replica")
        replicas = world // shard_world
        if replicas > 1 and shard_world < 2:
            raise ValueError("replicas repeat a shard group of at least two ranks")

        head_rows = -(-setup.microbatch_tokens // setup.head_chunks) if setup.head_chunks > 0 else 0

        def with_replicas(built):
            built[1].replicas = replicas          # programs depend on the shard count only
            if setup.collective_overhead_us > 0:
                from ..frontend.capture import add_collective_overhead
                add_collective_overhead(built[0], setup.collective_overhead_us)
            if setup.optimizer_rule != "adamw":
                # the unfused rules cost (and allocate) differently: keep their profiles apart
                for t in built[0].tasks:
                    if t.kind == "optimizer" and t.profile_key:
                        t.profile_key += f":{setup.optimizer_rule}"
            return built

        def build(index: int):
            walk, sel = variants[index]
            # "breadth/4": the microbatches in four forward + backward sweeps (sharded storage)
            walk, _, in_groups = walk.partition("/")
            order = StepDataOrdering(walk=walk, optimizer="stage_interleaved" if walk == "breadth" else "tail",
                                     microbatch_groups=int(in_groups or 1))
            return with_replicas(build_step(self.cfg, self.geometry, order, dtype=self.dtype,
                                            selection=sel, world_size=shard_world, rank=rank,
                                            expert_parallel=setup.expert_parallel,
                                            min_shard_bytes=setup.min_shard_bytes,
                                            head_block_rows=head_rows,
                                            master_weights=setup.master_weights,
                                            fused_gather=setup.fused_gather and world > 1, **choices))

        def build_extra(op: str):
            kw = dict(dtype=self.dtype, world_size=shard_world, rank=rank,
                      min_shard_bytes=setup.min_shard_bytes, head_block_rows=head_rows, **choices)
            if op == "forward_backward":
                return with_replicas(build_forward_backward(self.cfg, self.geometry, StepDataOrdering(), **kw))
            if op == "optim_step":
                return with_replicas(build_optimizer(self.cfg, self.geometry,
                                                     master_weights=setup.master_weights, **kw))
            if op == "forward":
                return with_replicas(build_forward(self.cfg, self.geometry, StepDataOrdering(), **kw))
            raise ValueError(f"unknown operation {op!r}")

        extra_ops = [op for op in setup.operations if op != "step"]
        self.profiles = Profiles()
        self.communication = CommunicationInfo(world_size=world)
        chosen, plan_json, extra_json = 0, None, {}
        from .preparation import load_bundle, save_bundle, setup_identity
        identity = setup_identity(setup, self.cfg)
        loaded = load_bundle(setup.bundle, identity) if (rank == 0 and setup.bundle) else None
        self.prepared_from_bundle = loaded is not None
        self.sweep = None
        # ---- host link calibration: every rank of the job measures its lanes at the same time,
        # because they share the host's memory system; the plan is made for the slowest rank
        from_bundle = loaded is not None
        # a preparation phase other than "communicate" is one process, whatever the job's size
        solo = setup.stop_after in ("build", "profile", "plan")
        if world > 1 and not solo:
            import torch.distributed as dist
            flag = [from_bundle]
            dist.broadcast_object_list(flag, src=0)
            from_bundle = flag[0]
        calibrated = None
        file_spill = setup.spill_pool in ("file", "remote")
        remote = setup.spill_address if setup.spill_pool == "remote" else ""
        if setup.spill_pool not in ("host", "file", "remote"):
            raise ValueError("spill_pool is 'host', 'file' or 'remote'")
        if setup.spill_pool == "file" and not (setup.spill_directory or setup.spill_image):
            raise ValueError("a file spill pool needs spill_directory or spill_image")
        if setup.spill_pool == "remote" and not remote:
            raise ValueError("a remote spill pool needs spill_address (host:port of a memory daemon)")
        measured_comm = phase_result("communication") if setup.stop_after != "communicate" else None
        if measured_comm is not None:
            calibrated = CommunicationInfo.from_json(measured_comm["communication"])
            self.log(f"communication: from {phase_dir / 'communication.json'}")
        if setup.stop_after in ("build", "profile"):
            pass                                   # these phases do not touch the lanes
        elif setup.calibrate and cuda and not from_bundle and measured_comm is None:
            t0 = time.perf_counter()
            probe = 256 << 20
            if world > 1:
                dist.barrier()
            if file_spill:
                # rates of the staged lanes (device <-> file), every rank's file on the drive at once;
                # a probe well beyond a drive's write cache, or the plan is built on its burst rate
                probe = 1 << 30
                import os
                scratch = "" if remote else (setup.spill_directory
                                             or os.path.dirname(os.path.abspath(setup.spill_image)))
                with Runtime(2 * probe, 4096, "cuda", setup.device_index, file_bytes=2 * probe,
                             file_directory=scratch, remote_address=remote,
                             file_chunk_bytes=setup.spill_chunk_bytes,
                             file_queue_depth=setup.spill_queue_depth) as rt:
                    r = rt.calibrate_file(probe, 2)
            else:
                with Runtime(2 * probe, 2 * probe, "cuda", setup.device_index) as rt:
                    r = rt.calibrate(probe, 3)
            rates = torch.tensor([r.fetch_solo_bps, r.fetch_concurrent_bps, r.evict_solo_bps,
                                  r.evict_concurrent_bps], dtype=torch.float64, device="cuda")
            lat = torch.tensor([r.fetch_latency_ns, r.evict_latency_ns], dtype=torch.float64, device="cuda")
            if world > 1:
                dist.all_reduce(rates, op=dist.ReduceOp.MIN)
                dist.all_reduce(lat, op=dist.ReduceOp.MAX)
            rates, lat = rates.tolist(), lat.tolist()
            calibrated = CommunicationInfo(rates[0], rates[1], rates[2], rates[3], int(lat[0]), int(lat[1]),
                                           world_size=world,
                                           source="calibrated" if world == 1 else f"calibrated with {world} ranks streaming")
            self.timings["communication"] = time.perf_counter() - t0
            self.log(f"{'staged lanes' if file_spill else 'host link'}: fetch {rates[0] / 1e9:.1f} ({rates[1] / 1e9:.1f} two-way) GB/s, "
                     f"evict {rates[2] / 1e9:.1f} ({rates[3] / 1e9:.1f}) GB/s")
        if setup.stop_after == "communicate":
            scale = 1.0
            if setup.profile and setup.calibrate_overlap and cuda:
                from ..communication.measure import measure_overlap
                scale = min(1.3, max(1.0, measure_overlap(setup.device_index).duration_scale))
            if rank == 0:
                comm = calibrated or CommunicationInfo(world_size=world)
                (phase_dir / "communication.json").write_text(json.dumps(
                    {"communication": comm.to_json(), "duration_scale": scale, "timings": self.timings}))
            return
        if loaded is not None:
            from ..ir.plan import Plan
            chosen, plan_json, extra_json = loaded["chosen"], loaded["plan"], loaded["extra_plans"]
            self.plan = Plan.from_json(plan_json)
            self.desc = build(chosen)[1]
            self.extra_plans = {op: (Plan.from_json(j), build_extra(op)[1])
                                for op, j in extra_json.items()}
            if loaded.get("communication"):
                self.communication = CommunicationInfo.from_json(loaded["communication"])
            if loaded.get("profiles"):
                self.profiles = Profiles.from_json(loaded["profiles"])
            self.log(f"prepared bundle {setup.bundle}: build, profile and plan skipped")
        elif rank == 0:
            # ---- build candidates
            t0 = time.perf_counter()
            candidates = [build(i) for i in range(len(variants))]
            extras = {op: build_extra(op) for op in extra_ops}
            layout = StateLayout.build([p for p, _ in candidates] + [p for p, _ in extras.values()])
            self.timings["build"] = time.perf_counter() - t0
            digests = {"candidates": [p.digest() for p, _ in candidates],
                       "operations": {op: p.digest() for op, (p, _) in extras.items()}}
            built = phase_result("build")
            if setup.stop_after == "build":
                (phase_dir / "build.json").write_text(json.dumps(
                    {**digests, "identity": identity, "timings": self.timings,
                     "tasks": [len(p.tasks) for p, _ in candidates],
                     "objects": [len(p.objects) for p, _ in candidates]}))
                return
            if built is not None and {k: built[k] for k in digests} != digests:
                raise RuntimeError("the programs built in this process differ from the ones the build phase "
                                   "recorded: the phases were not given the same setup")
            # ---- profile distinct tasks once
            t0 = time.perf_counter()
            scale = 1.0
            measured_profiles = phase_result("profiles") if setup.stop_after != "profile" else None
            if measured_profiles is not None:
                self.profiles = Profiles.from_json(measured_profiles["profiles"])
                self.log(f"profiles: {len(self.profiles.tasks)} tasks from {phase_dir / 'profiles.json'}")
            if measured_comm is not None:
                scale = float(measured_comm.get("duration_scale", 1.0))
            elif setup.profile and setup.calibrate_overlap and cuda and setup.stop_after != "profile":
                from ..communication.measure import measure_overlap
                ov = measure_overlap(setup.device_index)
                scale = min(1.3, max(1.0, ov.duration_scale))
                self.overlap = ov
                self.log(f"overlap: burst {ov.burst_tflops:.0f}, sustained {ov.sustained_tflops:.0f}, "
                         f"streaming {ov.streaming_tflops:.0f} TFLOP/s -> task times x{scale:.3f}")
            if setup.profile:
                dev = f"cuda:{setup.device_index}" if cuda else "cpu"
                store = ident = None
                if setup.store and measured_profiles is None:
                    from ..store import ContentStore, kernel_library_digest
                    store = ContentStore(setup.store, setup.store_mode)
                    ident = {"device": torch.cuda.get_device_name(setup.device_index) if cuda else "cpu",
                             "kernels": kernel_library_digest(), "dtype": setup.dtype,
                             "sequence_tokens": setup.profile_sequence_tokens}
                for prog, desc in candidates + list(extras.values()):
                    missing = {t.profile_key for t in prog.tasks} - set(self.profiles.tasks)
                    if store is not None:
                        from ..profiling.measure import TaskProfile
                        for key in sorted(missing):
                            hit = store.get("task_profile", {**ident, "task": key})
                            if hit is not None:
                                self.profiles.tasks[key] = TaskProfile(**hit)
                        missing -= set(self.profiles.tasks)
                    if missing and measured_profiles is not None:
                        raise KeyError(f"the profile phase did not measure {sorted(missing)[:3]}")
                    if missing:
                        got = measure_program(prog, desc, dev, keys=missing, rule=setup.optimizer_rule,
                                              fixed_len=setup.profile_sequence_tokens)
                        self.profiles.tasks.update(got.tasks)
                        self.profiles.device = got.device
                        if store is not None:
                            from dataclasses import asdict as _asdict
                            for key, prof in got.tasks.items():
                                store.put("task_profile", {**ident, "task": key}, _asdict(prof))
                    apply_profiles(prog, self.profiles, duration_scale=scale)
                if cuda and measured_profiles is None and setup.stop_after != "profile":
                    if setup.allocator == "planned":
                        from ..runtime import allocator as _alloc
                        _alloc.installed().trim()
                    else:
                        torch.cuda.empty_cache()
            self.timings["profile"] = time.perf_counter() - t0
            if setup.stop_after == "profile":      # with profiling off: an empty record, estimates stay
                (phase_dir / "profiles.json").write_text(json.dumps(
                    {"profiles": self.profiles.to_json(), "timings": self.timings}))
                return
            if setup.profile and setup.store:
                self.log(f"profile store: {store.hits} hits, {store.writes} new entries")
            # ---- host link calibration (done by every rank at once, see below)
            if calibrated is not None:
                self.communication = calibrated
            # ---- plan every candidate, keep the fastest
            t0 = time.perf_counter()
            sweep = sweep_programs([p for p, _ in candidates], self.budgets, self.communication,
                                   setup.search, state_layout=layout)
            self.extra_plans = {op: (plan_program(p, self.budgets, self.communication,
                                                  setup.search, layout), d)
                                for op, (p, d) in extras.items()}
            extra_json = {op: pl.to_json() for op, (pl, _) in self.extra_plans.items()}
            self.sweep = sweep
            self._candidates = [(p, f"{d.ordering.label()} [{_selection_label(d.selection)}]")
                                for p, d in candidates]
            self.plan = sweep.best
            chosen = next(i for i, (p, _) in enumerate(candidates) if p is self.plan.program)
            self.desc = candidates[chosen][1]
            self.timings["plan"] = time.perf_counter() - t0
            plan_json = self.plan.to_json()
            if setup.bundle:
                save_bundle(setup.bundle, identity, chosen, plan_json, extra_json,
                            self.profiles.to_json(), self.communication.to_json(), self.timings)
                self.log(f"prepared bundle written to {setup.bundle}")
        if setup.stop_after == "plan":
            if not setup.bundle:
                raise ValueError("the plan phase writes its result into TrainingSetup.bundle")
            return
        if world > 1 and not solo:
            # one plan for the whole job: identical offsets on every rank are what makes the
            # device pool symmetric, and identical task order keeps collectives matched
            import torch.distributed as dist
            box = [chosen, plan_json, extra_json]
            dist.broadcast_object_list(box, src=0)
            if rank != 0:
                from ..ir.plan import Plan
                chosen, plan_json, extra_json = box
                self.plan = Plan.from_json(plan_json)
                self.desc = build(chosen)[1]
                self.extra_plans = {op: (Plan.from_json(j), build_extra(op)[1])
                                    for op, j in extra_json.items()}
        file_pool = None
        if file_spill:
            from ..planning.plan import move_homes_to_file
            move_homes_to_file(self.plan)
            for xplan, _ in self.extra_plans.values():
                move_homes_to_file(xplan)
            image = setup.spill_image
            if image and world > 1:
                image = f"{image}.rank{rank}"
            file_pool = {"directory": setup.spill_directory, "image": image, "remote": remote,
                         "create_image": setup.spill_create_image,
                         "chunk_bytes": setup.spill_chunk_bytes, "queue_depth": setup.spill_queue_depth}
            self.log(f"spill pool: {self.plan.file_bytes / 2**30:.2f} GiB "
                     f"{'at ' + remote if remote else 'file'}, "
                     f"{self.plan.spill_bytes / 2**20:.1f} MiB pinned")
        self.log(f"plan: {self.plan.summary.ordering} {self.plan.summary.selection} "
                 f"simulated {self.plan.summary.duration_seconds * 1e3:.1f} ms")
        # ---- executor (caps the torch allocator to the planned workspace)
        t0 = time.perf_counter()
        if cuda and setup.allocator != "planned":
            total = torch.cuda.get_device_properties(setup.device_index).total_memory
            cap = max([self.plan.summary.workspace_bytes] +
                      [p.summary.workspace_bytes for p, _ in self.extra_plans.values()]) + (256 << 20)
            torch.cuda.set_per_process_memory_fraction(min(1.0, cap / total), setup.device_index)
        from ..ops.reference import RULES
        if setup.optimizer_rule not in RULES and not hasattr(setup.optimizer_rule, "apply"):
            raise ValueError(f"unknown optimizer rule {setup.optimizer_rule!r}; known: {RULES}")
        groups = tuple((tuple(g.get("match", ())), float(g.get("lr_scale", 1.0)), g.get("weight_decay"))
                       for g in (dict(x) for x in setup.parameter_groups))
        hyper = Hyperparameters(setup.lr, setup.beta1, setup.beta2, setup.eps, setup.weight_decay,
                                rule=setup.optimizer_rule, groups=groups, observe_norms=bool(setup.observe_norms))
        self.executor = Executor(self.plan, self.desc, device=setup.device,
                                 device_index=setup.device_index, seed=setup.seed, hyper=hyper,
                                 stochastic_rounding=setup.stochastic_rounding,
                                 trace_capacity=setup.trace_capacity,
                                 collectives=setup.collectives, extra_plans=self.extra_plans,
                                 file_pool=file_pool, annotate=setup.profiler_annotations,
                                 moe_chunks=setup.moe_chunks)
        if not (file_spill and setup.spill_image and not setup.spill_create_image):
            self.executor.initialize()      # an opened image already holds the state
        if setup.pretrained:
            # expert-parallel stages hold local banks: name the whole banks from a plain build
            from ..models.decoder import build_stages as _plain
            naming = (_plain(self.cfg, self.objective, self.lora) if setup.expert_parallel
                      else self.executor.stages)
            # one stage's tensors at a time (memory-mapped reads): the checkpoint never has to fit in
            # host memory beside the spill pool. Adapters and anything else the checkpoint does not name
            # keep their initial values; with several ranks each keeps its slice of every tensor
            from ..checkpoint.hf import stream_hf
            for _, part in stream_hf(self.cfg, setup.pretrained, naming):
                if part:
                    self.executor.load_full_state_dict(part, strict=False)
            self.log(f"weights from {setup.pretrained}")
        self.timings["open"] = time.perf_counter() - t0
        if cuda:
            if setup.allocator == "planned":
                self.executor.allocator.reset_peak()
            else:
                torch.cuda.reset_peak_memory_stats(setup.device_index)

    # ------------------------------------------------------------------ operations
    def step(self, batch: list[HostMicrobatch], **kw) -> InvocationResult:
        return self.executor.run(batch, **kw)

    def run(self, operation: str, batch: list[HostMicrobatch] | None = None, **kw) -> InvocationResult:
        return self.executor.run(batch, operation=operation, **kw)

    def save(self, directory: str, metadata: dict | None = None):
        from ..checkpoint import save_checkpoint
        return save_checkpoint(self.executor, directory, metadata=metadata)

    def restore(self, directory: str) -> dict:
        from ..checkpoint import load_checkpoint
        return load_checkpoint(self.executor, directory)

    def peak_device_bytes(self) -> int:
        """Peak device memory of this worker. Under the allocation adapter that is reported from the
        pool itself: planned ranges + the workspace slice (its peak use) + driver blocks held outside
        tasks. Otherwise: the planned ranges plus the torch allocator's peak reservation."""
        if self.setup.device != "cuda":
            return self.plan.device_bytes
        adapter = getattr(self.executor, "allocator", None)
        if adapter is not None:
            st = adapter.stats()
            return self.plan.device_bytes + st["peak"] + st["driver_bytes"]
        return self.plan.device_bytes + torch.cuda.max_memory_reserved(self.setup.device_index)

    def write_plan_report(self, directory: str) -> None:
        from ..reporting.write import write_report
        write_report(self.plan, directory)

    def planning_inputs(self):
        """What planning consumed, for offline sweeps over other budgets and link rates
        (``planning.offline.PlanningInputs``): the candidate programs with their measured costs,
        the calibrated link, the budgets and the search options. Needs a session that prepared
        itself (one opened from a bundle never built its candidates)."""
        from ..planning.offline import PlanningInputs
        if not getattr(self, "_candidates", None):
            raise ValueError("this session was opened from a prepared bundle: it holds one plan, not the candidates")
        return PlanningInputs([p for p, _ in self._candidates], self.communication, self.budgets,
                              [label for _, label in self._candidates], self.setup.search)

    def traced_step(self, batch: list[HostMicrobatch], directory: str | None = None):
        """Runs one real training step with per-task device timing and the runtime trace
        on, and returns ``(result, StepDiagnostics)``; with ``directory`` also writes the
        runtime report there. Needs ``TrainingSetup.trace_capacity > 0``."""
        from ..diagnostics.step import diagnose_step
        if self.setup.trace_capacity <= 0:
            raise ValueError("traced_step needs TrainingSetup.trace_capacity > 0")
        result = self.executor.run(batch, trace=True, time_tasks=True)
        diag = diagnose_step(self.plan, result, runtime_stats=self.executor.rt.stats())
        if directory:
            from ..reporting.runtime import write_runtime_report
            write_runtime_report(self.plan, diag, directory)
        return result, diag

    def close(self) -> None:
        if self.executor is None:                 # a session stopped after a preparation phase
            return
        self.executor.close()
        if self.setup.device == "cuda" and self.setup.allocator != "planned":
            torch.cuda.set_per_process_memory_fraction(1.0, self.setup.device_index)
