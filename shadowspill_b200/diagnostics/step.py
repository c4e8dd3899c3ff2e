"""Evidence from one traced step: measured task times joined to the plan's
simulated timeline, idle time between tasks split by cause, and transfer rates
seen by the lanes.

The join and the summary fields follow the reference's step diagnostics
(packages/engine/src/shadowspill/diagnostics/step.py;
docs/python/advanced/step-diagnostics.md:118-175): profiled / simulated / real
task seconds, inter-task idle divided into readiness waits and exposed frontend
overhead, makespan, entry delay, terminal tail, optimizer span and a per-phase
comparison. Device times come from CUDA events recorded around every task on
the compute stream; host times come from the runtime's trace ring.
"""
from __future__ import annotations

from collections import defaultdict
from dataclasses import asdict, dataclass, field
from typing import Any

from ..ir.plan import Plan


@dataclass
class TaskRow:
    index: int
    name: str
    kind: str
    stage: int
    microbatch: int
    profiled_s: float
    simulated_start_s: float
    simulated_s: float
    real_start_s: float
    real_s: float
    gap_before_s: float            # device idle between the previous task's end and this start
    simulated_gap_s: float
    waited_inputs: int = 0         # fetches this task had to wait on (stream waits inserted)
    waited_reuse: int = 0          # range predecessors it had to wait on


@dataclass
class TransferRow:
    action: int
    kind: str
    object: str
    bytes: int
    simulated_start_s: float
    simulated_s: float
    issue_host_s: float            # host clock at enqueue, relative to step begin
    real_start_s: float            # device clock, relative to the step's first event
    real_s: float
    gbps: float


@dataclass
class StepDiagnostics:
    tokens: int
    makespan_s: float
    simulated_makespan_s: float
    task_seconds_real: float
    task_seconds_simulated: float
    task_seconds_profiled: float
    idle_seconds_real: float
    idle_seconds_simulated: float
    input_readiness_wait_seconds: float
    allocation_reuse_wait_seconds: float
    frontend_overhead_seconds: float
    entry_delay_seconds: float
    terminal_tail_seconds: float
    optimizer_span_seconds: float
    cycle_seconds: float
    tokens_per_second: float
    trace_complete: bool
    phases: dict[str, dict[str, float]] = field(default_factory=dict)
    runtime: dict[str, Any] = field(default_factory=dict)
    tasks: list[TaskRow] = field(default_factory=list)
    transfers: list[TransferRow] = field(default_factory=list)

    def to_json(self, rows: bool = True) -> dict[str, Any]:
        d = asdict(self)
        if not rows:
            d.pop("tasks")
            d.pop("transfers")
        return d

    def worst_tasks(self, n: int = 10) -> list[TaskRow]:
        """Tasks whose real time exceeds the profile by the largest margin."""
        return sorted(self.tasks, key=lambda r: r.real_s - r.profiled_s, reverse=True)[:n]


def diagnose_step(plan: Plan, result, task_start_seconds: list[float] | None = None,
                  runtime_stats: dict[str, Any] | None = None) -> StepDiagnostics:
    """``result`` is an ``InvocationResult`` from ``Executor.run(..., trace=True,
    time_tasks=True)``; ``task_start_seconds`` defaults to ``result.task_start_seconds``."""
    prog = plan.program
    n = len(prog.tasks)
    real = list(result.task_seconds) or [0.0] * n
    starts = list(task_start_seconds if task_start_seconds is not None
                  else getattr(result, "task_start_seconds", []) or [])
    if len(starts) != n:                      # no per-task clock: lay tasks end to end
        starts, t = [], 0.0
        for d in real:
            starts.append(t)
            t += d
    makespan = result.device_seconds or (starts[-1] + real[-1] if n else 0.0)
    # ---- trace: per-task wait counts, per-action issue/done host times
    waits_in, waits_reuse = defaultdict(int), defaultdict(int)
    issue = {}
    t_begin = t_end = None
    for ev in result.trace:
        k = ev["kind"]
        if k == "step_begin":
            t_begin = ev["host_ns"]
        elif k == "step_end":
            t_end = ev["host_ns"]
        elif k == "input_wait":
            waits_in[ev["id"]] += 1
        elif k == "reuse_wait":
            waits_reuse[ev["id"]] += 1
        elif k in ("fetch_issue", "evict_issue"):
            issue[ev["id"]] = ev["host_ns"]
    trace_complete = bool(result.trace) and t_begin is not None and t_end is not None
    base = t_begin or 0
    # ---- task rows
    rows: list[TaskRow] = []
    # the executor runs collectives and the sharded update on a communication stream: a task's gap
    # is measured against the previous task of ITS lane (the simulation has one lane)
    sharded = any(t.kind == "collective" for t in prog.tasks)
    side = [t.kind == "collective" or (sharded and t.kind == "optimizer") for t in prog.tasks]
    prev_real_end = {False: 0.0, True: 0.0}
    prev_sim_end = 0
    for i, t in enumerate(prog.tasks):
        s_ns, e_ns = plan.task_start_ns[i], plan.task_end_ns[i]
        lane = side[i]
        rows.append(TaskRow(i, t.name, t.kind, t.stage, t.microbatch, t.duration_ns * 1e-9,
                            s_ns * 1e-9, (e_ns - s_ns) * 1e-9, starts[i], real[i],
                            max(0.0, starts[i] - prev_real_end[lane]), (s_ns - prev_sim_end) * 1e-9,
                            waits_in.get(i, 0), waits_reuse.get(i, 0)))
        prev_real_end[lane] = max(prev_real_end[lane], starts[i] + real[i])
        prev_sim_end = e_ns
    # ---- idle attribution: a gap before a task that had to wait on a fetch is readiness
    # wait, on a reused range allocation wait, otherwise the frontend was late
    lane_rows = [r for r in rows if not side[r.index]]          # idle = the compute lane's idle
    first = lane_rows[0].index if lane_rows else -1
    lane_rows = [r for r in lane_rows if r.index != first]
    w_in = sum(r.gap_before_s for r in lane_rows if r.waited_inputs)
    w_reuse = sum(r.gap_before_s for r in lane_rows if not r.waited_inputs and r.waited_reuse)
    idle_real = sum(r.gap_before_s for r in lane_rows)
    frontend = idle_real - w_in - w_reuse
    # ---- phases
    phases: dict[str, dict[str, float]] = {}
    for r in rows:
        p = phases.setdefault(r.kind, {"tasks": 0, "profiled_s": 0.0, "simulated_s": 0.0,
                                       "real_s": 0.0, "gap_s": 0.0})
        p["tasks"] += 1
        p["profiled_s"] += r.profiled_s
        p["simulated_s"] += r.simulated_s
        p["real_s"] += r.real_s
        p["gap_s"] += r.gap_before_s
    opt = [r for r in rows if r.kind == "optimizer"]
    opt_span = (opt[-1].real_start_s + opt[-1].real_s - opt[0].real_start_s) if opt else 0.0
    # ---- transfers
    transfers: list[TransferRow] = []
    tb = list(getattr(result, "transfer_begin_ns", []) or [])
    te = list(getattr(result, "transfer_end_ns", []) or [])
    for a, act in enumerate(plan.schedule.actions):
        if act.kind == "release" or a not in issue:
            continue
        o = prog.objects[act.object]
        have = a < len(tb) and tb[a] >= 0 and te[a] >= tb[a]
        start = tb[a] * 1e-9 if have else 0.0
        dur = (te[a] - tb[a]) * 1e-9 if have else 0.0
        transfers.append(TransferRow(a, act.kind, o.name, o.bytes, plan.action_start_ns[a] * 1e-9,
                                     (plan.action_end_ns[a] - plan.action_start_ns[a]) * 1e-9,
                                     (issue[a] - base) * 1e-9, start, dur,
                                     o.bytes / dur * 1e-9 if dur > 0 else 0.0))
    sim_total = max(plan.task_end_ns, default=0) * 1e-9
    last_end = (starts[-1] + real[-1]) if n else 0.0
    cycle = (t_end - t_begin) * 1e-9 if trace_complete else result.execution_seconds
    return StepDiagnostics(
        tokens=result.tokens, makespan_s=makespan, simulated_makespan_s=sim_total,
        task_seconds_real=sum(real), task_seconds_simulated=sum(r.simulated_s for r in rows),
        task_seconds_profiled=sum(r.profiled_s for r in rows),
        idle_seconds_real=idle_real, idle_seconds_simulated=sum(r.simulated_gap_s for r in rows[1:]),
        input_readiness_wait_seconds=w_in, allocation_reuse_wait_seconds=w_reuse,
        frontend_overhead_seconds=frontend,
        entry_delay_seconds=starts[0] if n else 0.0,
        terminal_tail_seconds=max(0.0, makespan - last_end),
        optimizer_span_seconds=opt_span, cycle_seconds=cycle,
        tokens_per_second=result.tokens / makespan if makespan > 0 else 0.0,
        trace_complete=trace_complete, phases=phases, runtime=dict(runtime_stats or {}),
        tasks=rows, transfers=transfers)
