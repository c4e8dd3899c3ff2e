"""Profile phase: time every distinct task of a program in isolation.

Tasks that share a ``profile_key`` (same stage type, form, variant and token
count) share one measurement. Each is run on freshly allocated byte ranges with
valid synthetic inputs: conditioning runs first, then samples until the median
absolute deviation is within tolerance (or a cap is hit), timed with CUDA events
on the launching stream. The torch allocator's peak over the run is the task's
workspace. ``apply_profiles`` writes durations and workspaces into a program.

Reference: packages/engine/src/shadowspill/profiling/measure.py:31
(``measure_program``), profiling/timing.py:80-126 (stability rule),
profiling/apply.py:14.
"""
from __future__ import annotations

import statistics
import time
from dataclasses import asdict, dataclass, field

import numpy as np
import torch

from ..data.synthetic import make_batch
from ..execution.executor import Hyperparameters, TaskRunner
from ..frontend.capture import TrainingDescription
from ..ir.program import Program


@dataclass
class TaskProfile:
    key: str
    seconds: float
    workspace_bytes: int
    samples: int
    spread: float            # MAD / median
    allocations: list = field(default_factory=list)   # request sizes under the allocation adapter
    # the same task when it adds to an existing gradient instead of creating it (later microbatches)
    allocations_accumulate: list = field(default_factory=list)


@dataclass
class Profiles:
    tasks: dict[str, TaskProfile] = field(default_factory=dict)
    device: str = ""

    def to_json(self) -> dict:
        return {"device": self.device, "tasks": {k: asdict(v) for k, v in self.tasks.items()}}

    @staticmethod
    def from_json(d: dict) -> "Profiles":
        return Profiles({k: TaskProfile(**v) for k, v in d["tasks"].items()}, d.get("device", ""))


def _fill_inputs(runner: TaskRunner, task: int, flats: list[torch.Tensor], host_batch) -> None:
    prog = runner.program
    t = prog.tasks[task]
    for u, flat in zip(runner.uses[task], flats):
        obj = prog.objects[u.object]
        if u.role == "batch":
            mb = host_batch[max(t.microbatch, 0)]
            buf = np.zeros(obj.bytes, dtype=np.uint8)
            for name, (off, count, dt) in runner.batch_layout_.items():
                if hasattr(mb, name):
                    src = getattr(mb, name)
                else:      # objective inputs: zeros keep ratios at one and every branch finite
                    src = mb.extras.get(name, np.zeros(count, dtype=dt))
                view = buf[off:off + count * np.dtype(dt).itemsize].view(dt)
                view[:src.shape[0]] = src
                if name == "cu_seqlens":
                    view[src.shape[0]:] = src[-1]
            flat.copy_(torch.from_numpy(buf))
            runner.max_seqlen[max(t.microbatch, 0)] = int(mb.max_seqlen)
        elif u.role in ("params", "x", "dx", "saved", "grads", "m", "v"):
            # small random values of the model dtype keep every kernel on its normal path
            dt = runner.desc.dtype
            n = obj.bytes // dt.itemsize
            vals = torch.randn(min(n, 1 << 22), device=flat.device, dtype=torch.float32) * 0.02
            view = flat[:n * dt.itemsize].view(dt)
            reps = (n + vals.numel() - 1) // vals.numel()
            view.copy_(vals.to(dt).repeat(reps)[:n])
            if u.role == "v":
                view.abs_()
        else:
            flat.zero_()


def measure_program(program: Program, desc: TrainingDescription, device: str = "cuda",
                    min_samples: int = 3, max_samples: int = 8, tolerance: float = 0.03,
                    keys: set[str] | None = None, rule: str = "adamw", fixed_len: int = 0) -> Profiles:
    """Times one representative task per ``profile_key`` with the ordinary torch allocator.
    ``rule``: the run's update rule (the unfused rules allocate temporaries the fused one does not).
    ``fixed_len``: profile on sequences of exactly this length (long-context runs) instead of the
    packed log-normal mix."""
    dev = torch.device(device)
    cuda = dev.type == "cuda"
    runner = TaskRunner(program, desc, Hyperparameters(lr=0.0, rule=rule), seed=0, stochastic_rounding=True)
    meta = program.metadata
    cfg = desc.cfg
    host_batch = make_batch(0, vocab=cfg.vocab_size, tokens_per_step=runner.T * runner.n_mb,
                            microbatch_tokens=runner.T, slots=runner.slots,
                            max_len=min(8192, runner.T), fixed_len=min(fixed_len, runner.T) or None,
                            median=min(1200.0, runner.T / 4), min_len=min(32, runner.T // 4))
    profiles = Profiles(device=torch.cuda.get_device_name(dev) if cuda else "cpu")
    seen: dict[str, int] = {}
    for ti, t in enumerate(program.tasks):
        if t.kind == "collective" or t.variant == "adamw_dp":
            continue      # needs every rank; keeps its modelled cost until calibrated
        if t.profile_key and t.profile_key not in seen and (keys is None or t.profile_key in keys):
            seen[t.profile_key] = ti
    for key, ti in seen.items():
        flats = [torch.empty(program.objects[u.object].bytes, dtype=torch.uint8, device=dev)
                 for u in runner.uses[ti]]
        _fill_inputs(runner, ti, flats, host_batch)
        B = runner.bind(ti, flats)
        samples: list[float] = []
        from ..runtime import allocator as _alloc
        adapter = _alloc.installed() if cuda else None
        contract: list[int] = []
        contract_acc: list[int] = []
        if adapter is not None:
            # the allocation contract: three warmed runs must ask for the same tensors in the same
            # order (packages/engine/src/shadowspill/profiling/measure.py:31 does the same)
            runner.grad_seen = set()
            runner.run_task(ti, B)                 # warm-up outside the record
            runs = []
            for _ in range(3):
                runner.grad_seen = set()
                with adapter.task(program.tasks[ti].name, _alloc.RECORD) as seq:
                    runner.run_task(ti, B)
                runs.append(list(seq))
            torch.cuda.synchronize(dev)
            if not (runs[0] == runs[1] == runs[2]):
                raise RuntimeError(f"task {program.tasks[ti].name} allocates differently from run to run: "
                                   f"{[len(r) for r in runs]} requests; it has no stable allocation contract")
            contract = runs[0]
            workspace = adapter.stats()["task_peak"]
            own = B.get("grads.mode") or B.get("tied_grads.mode")
            if own in ("create", "mutate"):
                # the same task runs with the gradient created (first microbatch) and added to
                # (later ones); the two forms may allocate differently, so each has its contract
                other = "mutate" if own == "create" else "create"
                alt = dict(B)
                for role in ("grads", "tied_grads"):
                    if f"{role}.mode" in alt:
                        alt[f"{role}.mode"] = other
                runner.grad_seen = set(range(len(runner.stages))) if other == "mutate" else set()
                with adapter.task(program.tasks[ti].name, _alloc.RECORD) as seq:
                    runner.run_task(ti, alt)
                flipped = list(seq)
                workspace = max(workspace, adapter.stats()["task_peak"])
                torch.cuda.synchronize(dev)
                contract, contract_acc = (contract, flipped) if own == "create" else (flipped, contract)
        elif cuda:
            torch.cuda.synchronize(dev)
            torch.cuda.reset_peak_memory_stats(dev)
            base = torch.cuda.memory_allocated(dev)
            runner.grad_seen = set()
            runner.run_task(ti, B)                 # conditioning
            torch.cuda.synchronize(dev)
            workspace = torch.cuda.max_memory_allocated(dev) - base
        else:
            runner.grad_seen = set()
            runner.run_task(ti, B)                 # conditioning
            workspace = program.tasks[ti].workspace_bytes
        while len(samples) < max_samples:
            runner.grad_seen = set()
            if cuda:
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                runner.run_task(ti, B)
                b.record()
                torch.cuda.synchronize(dev)
                samples.append(a.elapsed_time(b) * 1e-3)
            else:
                t0 = time.perf_counter()
                runner.run_task(ti, B)
                samples.append(time.perf_counter() - t0)
            if len(samples) >= min_samples:
                med = statistics.median(samples)
                mad = statistics.median(abs(s - med) for s in samples)
                if med > 0 and mad / med <= tolerance:
                    break
        med = statistics.median(samples)
        mad = statistics.median(abs(s - med) for s in samples)
        profiles.tasks[key] = TaskProfile(key, med, int(workspace), len(samples),
                                          mad / med if med > 0 else 0.0, contract, contract_acc)
        del flats, B
        if cuda and adapter is not None:
            adapter.trim()
        elif cuda:
            torch.cuda.empty_cache()
    return profiles


def apply_profiles(program: Program, profiles: Profiles, workspace_margin: float = 1.05,
                   duration_scale: float = 1.0) -> Program:
    """Writes measured durations and workspaces into ``program`` (in place)."""
    missing = []
    for t in program.tasks:
        p = profiles.tasks.get(t.profile_key)
        if p is None:
            if not (t.kind == "collective" or t.variant == "adamw_dp"):
                missing.append(t.profile_key)
            continue
        t.duration_ns = max(1, int(p.seconds * duration_scale * 1e9))
        # stages whose backward is derived by autograd allocate many large temporaries in
        # data-dependent order: leave the caching allocator room for fragmentation
        margin = (max(workspace_margin, 1.25) if ("HybridLayerStage" in t.profile_key or "Graph" in t.profile_key)
                  else workspace_margin)
        if ":ep" in t.profile_key:
            # profiled on one rank with its local experts; in the job the rows a rank receives
            # depend on every rank's routing
            margin = max(margin, 1.75)
        t.workspace_bytes = int(p.workspace_bytes * margin)
        accumulates = any(u.role in ("grads", "tied_grads") and u.mode == "mutate" for u in t.uses)
        t.allocations = list(p.allocations_accumulate if (accumulates and p.allocations_accumulate)
                             else p.allocations)
    if missing:
        raise KeyError(f"no profile for {sorted(set(missing))[:4]}")
    program.metadata["profiled_on"] = profiles.device
    return program
