"""Explain a memory search: what each candidate did, and the pressure profile it worked on.

    python -m shadowspill_b200.planning.trace --model llama3-8b --device-gib 24 --spill-gib 128 \\
        [--microbatch 8192 --microbatches 8] [--svg pressure.svg] [--json trace.json]

The native search records one line per decision when tracing is on (``SearchOptions(trace=True)``):
reductions with their capacity and number of cuts, simulations that could not finish and the
boundary that starved, boundary-pressure and fetch repairs, placements with their span. This tool
plans one program that way, parses the lines into per-candidate trajectories, and prints them; it
also computes the task-boundary pressure of the program before any cut and of the winning plan
(from its stays), and can draw both against the capacity as an SVG.

Reference: tools/pressurefit_trace (collect / explain / pressure: per-candidate trajectories and
boundary pressure, rendered as charts and videos there).
"""
from __future__ import annotations

import argparse
import json
import re
import sys

import torch

from ..communication.info import CommunicationInfo
from ..frontend.capture import BatchGeometry, StepDataOrdering, build_step, mixed_selection
from ..ir.plan import Plan
from ..ir.program import Program
from ..models.config import preset
from .plan import MemoryBudgets, SearchOptions, plan_program

GIB = 1 << 30
_STRATEGIES, _RULES = ("stall", "traffic"), ("demand", "latest-safe", "packed-fifo", "packed-fit")


def parse_trace(text: str) -> list[dict]:
    """Per candidate: its strategy and rule and the ordered list of events the search logged."""
    out: list[dict] = []
    for line in text.splitlines():
        m = re.match(r"candidate strategy=(\d+) rule=(\d+)", line)
        if m:
            out.append({"strategy": _STRATEGIES[int(m.group(1))], "fetch_rule": _RULES[int(m.group(2))],
                        "events": []})
            continue
        if not out:
            continue
        ev = out[-1]["events"]
        if m := re.match(r"reduce: capacity (\d+) cuts (\d+) of (\d+) gaps", line):
            ev.append({"kind": "reduce", "capacity": int(m.group(1)), "cuts": int(m.group(2)), "gaps": int(m.group(3))})
        elif m := re.match(r"reduce: infeasible at task (\d+) pressure (-?\d+) capacity (\d+)", line):
            ev.append({"kind": "reduce_infeasible", "task": int(m.group(1)), "pressure": int(m.group(2)),
                       "capacity": int(m.group(3))})
        elif m := re.match(r"simulate: no progress \(status (\d+), task (-?\d+), t=(\d+)\)", line):
            ev.append({"kind": "simulate_stalled", "task": int(m.group(2)), "at_ns": int(m.group(3))})
        elif m := re.match(r"repair: boundary pressure \+(\d+) at task (\d+)", line):
            ev.append({"kind": "boundary_pressure", "bytes": int(m.group(1)), "task": int(m.group(2))})
        elif m := re.match(r"repair: (\d+) accepted, makespan (\d+)", line):
            ev.append({"kind": "fetch_repair", "accepted": int(m.group(1)), "makespan_ns": int(m.group(2))})
        elif m := re.match(r"place: span (\d+) slice (\d+) workspace (\d+) capacity (\d+) makespan (\d+)", line):
            ev.append({"kind": "place", "span": int(m.group(1)), "slice": int(m.group(2)),
                       "workspace": int(m.group(3)), "capacity": int(m.group(4)), "makespan_ns": int(m.group(5)),
                       "fits": int(m.group(1)) + int(m.group(2)) + int(m.group(3)) <= int(m.group(4))})
    for c in out:
        places = [e for e in c["events"] if e["kind"] == "place" and e["fits"]]
        c["placed"] = bool(places)
        c["makespan_ns"] = places[-1]["makespan_ns"] if places else None
    return out


def uncut_pressure(program: Program) -> list[int]:
    """Bytes that would be resident at each task if every object stayed from its first to its
    last use, plus the task's workspace."""
    nt = len(program.tasks)
    first, last = {}, {}
    for ti, t in enumerate(program.tasks):
        for u in t.uses:
            first.setdefault(u.object, ti)
            last[u.object] = ti
    p = [t.workspace_bytes for t in program.tasks]
    for o, a in first.items():
        for t in range(a, last[o] + 1):
            p[t] += program.objects[o].bytes
    return p[:nt]


def planned_pressure(plan: Plan) -> list[int]:
    """Bytes the plan keeps resident while each task runs (its stays), plus the task's workspace."""
    p = [t.workspace_bytes for t in plan.program.tasks]
    for s in plan.stays:
        for ti, (a, b) in enumerate(zip(plan.task_start_ns, plan.task_end_ns)):
            if s.start_ns < b and a < s.end_ns or (a == b and s.start_ns <= a < s.end_ns):
                p[ti] += s.bytes
    return p


def explain(trajectories: list[dict]) -> str:
    lines = []
    for c in trajectories:
        head = f"{c['strategy']:8s} {c['fetch_rule']:12s}"
        if not c["placed"]:
            lines.append(f"{head} no placed plan ({len(c['events'])} events)")
        else:
            lines.append(f"{head} makespan {c['makespan_ns'] / 1e6:9.2f} ms")
        for e in c["events"]:
            if e["kind"] == "reduce":
                lines.append(f"    reduce to {e['capacity'] / GIB:.2f} GiB: {e['cuts']} of {e['gaps']} gaps cut")
            elif e["kind"] == "reduce_infeasible":
                lines.append(f"    cannot reduce: task {e['task']} needs {e['pressure'] / GIB:.2f} GiB "
                             f"of {e['capacity'] / GIB:.2f}")
            elif e["kind"] == "simulate_stalled":
                lines.append(f"    simulation starved at task {e['task']}")
            elif e["kind"] == "boundary_pressure":
                lines.append(f"    boundary-pressure repair: +{e['bytes'] / (1 << 20):.0f} MiB at task {e['task']}")
            elif e["kind"] == "fetch_repair" and e["accepted"]:
                lines.append(f"    {e['accepted']} fetch move(s) kept, makespan {e['makespan_ns'] / 1e6:.2f} ms")
            elif e["kind"] == "place":
                lines.append(f"    layout {e['span'] / GIB:.2f} GiB + slice {e['slice'] / (1 << 20):.1f} MiB + workspace "
                             f"{e['workspace'] / GIB:.2f} GiB: {'fits' if e['fits'] else 'overruns'}")
    return "\n".join(lines)


def pressure_svg(uncut: list[int], planned: list[int], capacity: int, width: int = 1100, height: int = 320) -> str:
    top = max(max(uncut, default=1), capacity, 1) * 1.05
    n = max(len(uncut), 2)

    def path(values):
        pts = [f"{i * (width - 60) / (n - 1) + 50:.1f},{height - 30 - v / top * (height - 50):.1f}"
               for i, v in enumerate(values)]
        return "M" + " L".join(pts)
    cap_y = height - 30 - capacity / top * (height - 50)
    return (f'<svg xmlns="http://www.w3.org/2000/svg" width="{width}" height="{height}" font-family="sans-serif" font-size="11">'
            f'<rect width="100%" height="100%" fill="white"/>'
            f'<path d="{path(uncut)}" fill="none" stroke="#bbb" stroke-width="1.2"/>'
            f'<path d="{path(planned)}" fill="none" stroke="#1f6fb5" stroke-width="1.4"/>'
            f'<line x1="50" x2="{width - 10}" y1="{cap_y:.1f}" y2="{cap_y:.1f}" stroke="#c33" stroke-dasharray="5,3"/>'
            f'<text x="54" y="{cap_y - 4:.1f}" fill="#c33">capacity {capacity / GIB:.1f} GiB</text>'
            f'<text x="54" y="14" fill="#888">grey: every object resident first to last use ({max(uncut) / GIB:.1f} GiB peak); '
            f'blue: the plan ({max(planned) / GIB:.1f} GiB peak); x: task index</text></svg>')


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", default="llama3-8b")
    ap.add_argument("--device-gib", type=float, default=24.0)
    ap.add_argument("--spill-gib", type=float, default=128.0)
    ap.add_argument("--microbatch", type=int, default=8192)
    ap.add_argument("--microbatches", type=int, default=8)
    ap.add_argument("--full-save-layers", type=int, default=0, help="layers that keep the whole save set")
    ap.add_argument("--fetch-gbs", type=float, default=55.0)
    ap.add_argument("--evict-gbs", type=float, default=55.0)
    ap.add_argument("--svg", default="")
    ap.add_argument("--json", default="")
    a = ap.parse_args(argv)
    cfg = preset(a.model)
    geo = BatchGeometry(a.microbatch, a.microbatches, a.microbatch // 32 + 1, 1200)
    program, _ = build_step(cfg, geo, StepDataOrdering(), dtype=torch.bfloat16,
                            selection={} if cfg.is_moe else mixed_selection(cfg, a.full_save_layers))
    comm = CommunicationInfo(fetch_solo_bps=a.fetch_gbs * 1e9, fetch_concurrent_bps=a.fetch_gbs * 0.9e9,
                             evict_solo_bps=a.evict_gbs * 1e9, evict_concurrent_bps=a.evict_gbs * 0.9e9)
    budgets = MemoryBudgets(int(a.device_gib * GIB), int(a.spill_gib * GIB))
    plan = plan_program(program, budgets, comm, SearchOptions(trace=True, workers=1))
    trajectories = parse_trace(plan.communication.get("search_trace", ""))
    print(explain(trajectories))
    s = plan.summary
    print(f"winner: {s.strategy} / {s.fetch_rule}: {s.duration_seconds * 1e3:.1f} ms simulated, "
          f"{s.fetch_bytes / 1e9:.1f} GB fetched, {s.evict_bytes / 1e9:.1f} GB evicted")
    uncut, planned = uncut_pressure(program), planned_pressure(plan)
    if a.svg:
        open(a.svg, "w").write(pressure_svg(uncut, planned, budgets.capacity))
    if a.json:
        json.dump({"candidates": trajectories, "uncut_pressure": uncut, "planned_pressure": planned,
                   "capacity": budgets.capacity}, open(a.json, "w"))
    return 0


if __name__ == "__main__":
    sys.exit(main())
