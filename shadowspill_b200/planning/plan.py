"""``plan_program``: program + budgets + link facts -> executable ``Plan``.

Runs the native search (reduce / emit / simulate / repair / place), then gives
every object that touches the spill pool a home there, recovers the reuse
dependencies of the fixed device layout, and fills the plan summary the reports
show. ``sweep_programs`` plans a family of candidate programs (orderings,
save/recompute selections, microbatch geometries) and keeps the fastest.

Reference: packages/engine/src/shadowspill/planning/plan.py:26 (``plan_program``),
planning/sweep.py:21, planning/memory_search/algorithm.py:284 (``SearchOptions``).
"""
from __future__ import annotations

import concurrent.futures
import ctypes as C
from dataclasses import dataclass, field

from .. import native
from ..communication.info import CommunicationInfo
from ..ir.plan import MemoryAction, MemorySchedule, Plan, PlanSummary
from ..ir.program import Program
from ..simulator.api import (SimulationConfig, place_lifetimes, recover_layout_reuse,
                             stays_from_native)

GIB = 1 << 30
EXTERNAL_HEADROOM = 512 << 20   # bytes of the device budget left to the driver and libraries


class PlanningError(RuntimeError):
    pass


@dataclass
class SearchOptions:
    workers: int = 0
    strategies: tuple[str, ...] = native.STRATEGIES
    fetch_rules: tuple[str, ...] = native.FETCH_RULES
    max_repairs: int = 16
    minimum_object_bytes_evict_eligible: int = 1 << 20
    capacity_refinement_step: int = 256 << 20
    deterministic: bool = False
    trace: bool = False
    alignment: int = 512
    # the plain O(cuts x gaps) reducer instead of the indexed one (same decisions; for comparison)
    linear_reduce: bool = False
    # small never-cut objects get static homes in a slice behind the main layout
    resident_slice: bool = True

    def to_native(self) -> native.SearchOptions:
        sm = sum(1 << native.STRATEGIES.index(s) for s in self.strategies)
        rm = sum(1 << native.FETCH_RULES.index(r) for r in self.fetch_rules)
        return native.SearchOptions(self.workers, sm, rm, self.max_repairs,
                                    self.minimum_object_bytes_evict_eligible,
                                    self.capacity_refinement_step, int(self.deterministic),
                                    int(self.trace), int(self.linear_reduce), int(not self.resident_slice))


@dataclass
class MemoryBudgets:
    device_bytes: int
    spill_bytes: int
    headroom_bytes: int = EXTERNAL_HEADROOM
    fixed_device_bytes: int = 0     # resident allocations outside the plan (status words, streams)

    @property
    def capacity(self) -> int:
        return self.device_bytes - self.headroom_bytes - self.fixed_device_bytes

    @staticmethod
    def from_gib(device_gib: float, spill_gib: float) -> "MemoryBudgets":
        return MemoryBudgets(int(device_gib * GIB), int(spill_gib * GIB))


@dataclass
class StateLayout:
    """Spill homes shared by every plan of one run: persistent tensors keep the
    same offset whichever operation's plan is executing."""
    offsets: dict[str, int] = field(default_factory=dict)
    reserved: int = 0

    @staticmethod
    def build(programs: list[Program]) -> "StateLayout":
        lay = StateLayout()
        for prog in programs:
            for o in prog.objects:
                if o.persistent and o.kind in ("weight", "optimizer_state", "gradient") \
                        and o.name not in lay.offsets:
                    lay.offsets[o.name] = lay.reserved
                    lay.reserved += -(-o.bytes // 4096) * 4096
        return lay


def plan_program(program: Program, budgets: MemoryBudgets,
                 communication: CommunicationInfo | None = None,
                 options: SearchOptions | None = None,
                 state_layout: StateLayout | None = None) -> Plan:
    communication = communication or CommunicationInfo()
    options = options or SearchOptions()
    program.validate()
    if budgets.capacity <= 0:
        raise PlanningError("device budget does not cover the external headroom")
    lib = native.core()
    prog, keep = program.to_native()
    cfg = SimulationConfig(budgets.capacity, communication, options.alignment).to_native()
    opt = options.to_native()
    handle = native.vp()
    native.check(lib.ss_plan_search(C.byref(prog), C.byref(cfg), C.byref(opt), C.byref(handle)),
                 "ss_plan_search")
    try:
        s = lib.ss_search_summary_of(handle).contents
        trace = lib.ss_search_trace(handle).decode() if options.trace else ""
        if s.status != native.OK:
            need = max((t.workspace_bytes for t in program.tasks), default=0)
            raise PlanningError(
                f"no schedule fits {budgets.capacity / GIB:.2f} GiB of plan capacity "
                f"({s.candidates_evaluated} candidates; largest task workspace "
                f"{need / GIB:.2f} GiB)\n{trace}")
        na, ni, nt = s.n_actions, s.n_intervals, len(program.tasks)
        acts = lib.ss_search_actions(handle)
        actions = [MemoryAction(("fetch", "evict", "release")[acts[i].kind], acts[i].object,
                                acts[i].trigger_task) for i in range(na)]
        stays = stays_from_native(lib.ss_search_intervals(handle), ni)
        ts = [lib.ss_search_task_start(handle)[i] for i in range(nt)]
        te = [lib.ss_search_task_end(handle)[i] for i in range(nt)]
        as_ = [lib.ss_search_action_start(handle)[i] for i in range(na)]
        ae = [lib.ss_search_action_end(handle)[i] for i in range(na)]
        summary = PlanSummary(
            duration_seconds=s.sim.makespan_ns * 1e-9, compute_seconds=s.sim.compute_ns * 1e-9,
            input_wait_seconds=s.sim.input_wait_ns * 1e-9,
            capacity_wait_seconds=s.sim.capacity_wait_ns * 1e-9,
            execution_peak_bytes=s.sim.peak_bytes, layout_span_bytes=s.layout_span,
            fetch_bytes=s.sim.fetch_bytes, evict_bytes=s.sim.evict_bytes,
            strategy=native.STRATEGIES[s.best_strategy],
            fetch_rule=native.FETCH_RULES[s.best_fetch_rule],
            candidates_evaluated=s.candidates_evaluated,
            candidates_feasible=s.candidates_feasible, repairs_applied=s.repairs_applied,
            logical_capacity_bytes=s.logical_capacity)
    finally:
        lib.ss_search_result_destroy(handle)
        del keep
    # ---- reuse dependencies of the device layout
    sb = [-(-st.bytes // options.alignment) * options.alignment for st in stays]
    pb, pi = recover_layout_reuse(sb, [st.start_ns for st in stays], [st.end_ns for st in stays],
                                  [st.offset for st in stays])
    # ---- spill homes: persistent objects first, then evicted transients by lifetime
    spill_offsets = [-1] * len(program.objects)
    cursor = state_layout.reserved if state_layout else 0
    for i, o in enumerate(program.objects):
        if o.persistent:
            if state_layout and o.name in state_layout.offsets:
                spill_offsets[i] = state_layout.offsets[o.name]
                continue
            spill_offsets[i] = cursor
            cursor += -(-o.bytes // 4096) * 4096
    persistent_end = cursor
    first_evict, last_fetch = {}, {}
    for ai, a in enumerate(actions):
        if program.objects[a.object].persistent:
            continue
        if a.kind == "evict":
            first_evict.setdefault(a.object, as_[ai])
        elif a.kind == "fetch":
            last_fetch[a.object] = ae[ai]
    spilled = sorted(first_evict)
    if spilled:
        horizon = max(te) if te else 0
        offs, span = place_lifetimes(
            [-(-program.objects[o].bytes // 4096) * 4096 for o in spilled],
            [first_evict[o] for o in spilled],
            [max(last_fetch.get(o, horizon), first_evict[o] + 1) for o in spilled], 4096)
        for o, off in zip(spilled, offs):
            spill_offsets[o] = persistent_end + off
        cursor = persistent_end + span
    if cursor > budgets.spill_bytes:
        raise PlanningError(f"spill pool needs {cursor / GIB:.2f} GiB, budget is "
                            f"{budgets.spill_bytes / GIB:.2f} GiB")
    summary.spill_peak_bytes = cursor
    summary.workspace_bytes = max((t.workspace_bytes for t in program.tasks), default=0)
    summary.fixed_device_bytes = budgets.fixed_device_bytes
    summary.tokens = int(program.metadata.get("tokens", 0))
    summary.ordering = str(program.metadata.get("ordering", ""))
    summary.selection = str(program.metadata.get("selection", ""))
    if summary.duration_seconds > 0:
        summary.tokens_per_second = summary.tokens / summary.duration_seconds
    plan = Plan(program, MemorySchedule(actions), stays, spill_offsets, pb, pi, ts, te, as_, ae,
                device_bytes=max(summary.layout_span_bytes, options.alignment),
                spill_bytes=max(cursor, 4096),
                budgets={"device_bytes": budgets.device_bytes, "spill_bytes": budgets.spill_bytes,
                         "headroom_bytes": budgets.headroom_bytes,
                         "capacity_bytes": budgets.capacity},
                summary=summary, communication=communication.to_json())
    if options.trace:
        plan.communication["search_trace"] = trace
    return plan


def reduce_emit(program: Program, capacity: int, communication: CommunicationInfo | None = None,
                options: SearchOptions | None = None, strategy: str = "stall",
                fetch_rule: str = "latest-safe", tight: bool = False):
    """One Reduce + Emit pass of the native planner at ``capacity`` (no simulation, repair or
    placement): ``(cuts, actions)`` with cuts as ``(object, use index)`` in cut order and actions as
    ``(kind, object, trigger task)`` with kind 0 fetch / 1 evict / 2 release, or ``None`` when the
    capacity cannot be met. For comparison with ``qualification/pressurefit_oracle.py``."""
    communication = communication or CommunicationInfo()
    options = options or SearchOptions()
    lib = native.core()
    prog, keep = program.to_native()
    cfg = SimulationConfig(capacity, communication, options.alignment).to_native()
    opt = options.to_native()
    n_uses = sum(len(t.uses) for t in program.tasks)
    max_cuts, max_actions = n_uses + 1, 2 * n_uses + 2 * len(program.objects) + 2
    co, cu = (C.c_int32 * max_cuts)(), (C.c_int32 * max_cuts)()
    acts = (native.Action * max_actions)()
    nc, na = C.c_int32(0), C.c_int32(0)
    rc = lib.ss_plan_reduce_emit(C.byref(prog), C.byref(cfg), C.byref(opt), int(capacity),
                                 native.STRATEGIES.index(strategy), native.FETCH_RULES.index(fetch_rule),
                                 int(tight), co, cu, max_cuts, C.byref(nc), acts, max_actions, C.byref(na))
    del keep
    if rc == native.INFEASIBLE:
        return None
    native.check(rc, "ss_plan_reduce_emit")
    return ([(co[i], cu[i]) for i in range(nc.value)],
            [(acts[i].kind, acts[i].object, acts[i].trigger_task) for i in range(na.value)])


def host_kept(name: str, nbytes: int) -> bool:
    """Objects the host reads or writes every step stay in pinned memory when the spill pool
    is a file: packed batches, the loss word and anything too small to be worth a disk I/O."""
    return name.startswith("batch.") or name == "loss" or nbytes < 4096


def move_homes_to_file(plan: Plan, keep_host=host_kept) -> Plan:
    """Re-homes a plan for a file-backed spill pool (in place; returns the plan).

    Every spilled object keeps its offset but in the file; the few objects ``keep_host``
    names are packed into a small pinned pool instead (sorted by persistence and name, so
    that plans of several operations over the same state agree on them). The schedule is
    untouched: which pool an object's home is in only changes the lanes its transfers use
    (reference: packages/engine/src/shadowspill/ssd.py:38-110, where the SSD pool takes the
    place of the pinned spill pool)."""
    objs = plan.program.objects
    file_offsets = [-1] * len(objs)
    kept = []
    for i, o in enumerate(objs):
        off = plan.spill_offsets[i]
        if off < 0:
            continue
        if keep_host(o.name, o.bytes):
            kept.append(i)
        else:
            file_offsets[i] = off
    plan.file_bytes = max(plan.spill_bytes, 4096)
    cursor = 0
    for i in sorted(kept, key=lambda i: (not objs[i].persistent, objs[i].name)):
        plan.spill_offsets[i] = cursor
        cursor += -(-objs[i].bytes // 4096) * 4096
    for i, off in enumerate(file_offsets):
        if off >= 0:
            plan.spill_offsets[i] = -1
    plan.file_offsets = file_offsets
    plan.spill_bytes = max(cursor, 4096)
    plan.budgets["file_bytes"] = plan.file_bytes
    return plan


@dataclass
class SweepResult:
    best: Plan
    plans: list[Plan | None]
    errors: list[str]

    def table(self) -> list[dict]:
        rows = []
        for p, e in zip(self.plans, self.errors):
            if p is None:
                rows.append({"feasible": False, "error": e.splitlines()[0] if e else ""})
            else:
                s = p.summary
                rows.append({"feasible": True, "ordering": s.ordering, "selection": s.selection,
                             "seconds": s.duration_seconds, "tokens_per_second": s.tokens_per_second,
                             "fetch_bytes": s.fetch_bytes, "evict_bytes": s.evict_bytes})
        return rows


def sweep_programs(programs: list[Program], budgets: MemoryBudgets,
                   communication: CommunicationInfo | None = None,
                   options: SearchOptions | None = None, threads: int = 4,
                   state_layout: StateLayout | None = None) -> SweepResult:
    """Plan every candidate program and keep the one with the shortest simulated step."""
    plans: list[Plan | None] = [None] * len(programs)
    errors = [""] * len(programs)

    def one(i: int) -> None:
        try:
            plans[i] = plan_program(programs[i], budgets, communication, options, state_layout)
        except PlanningError as exc:
            errors[i] = str(exc)

    with concurrent.futures.ThreadPoolExecutor(max_workers=max(1, threads)) as pool:
        list(pool.map(one, range(len(programs))))
    feasible = [p for p in plans if p is not None]
    if not feasible:
        raise PlanningError("no candidate program fits the budgets:\n" + "\n".join(errors))
    best = min(feasible, key=lambda p: p.summary.duration_seconds)
    return SweepResult(best, plans, errors)
