"""Plan report: ``index.html``, ``summary.json``, ``tasks.csv``, ``transfers.csv``,
``timeline.json`` and an SVG timeline, all static files readable offline.

The file set and the summary fields follow the reference's ``write_report``
(packages/engine/src/shadowspill/reporting/write.py:54,
docs/python/advanced/plan-report.md:57-75).
"""
from __future__ import annotations

import csv
import html
import json
from dataclasses import asdict
from pathlib import Path

from ..ir.plan import Plan

GIB = 1 << 30
_COLORS = {"forward": "#4c78a8", "backward": "#f58518", "head": "#54a24b", "optimizer": "#b279a2",
           "fetch": "#72b7b2", "evict": "#e45756", "control": "#9d9d9d", "collective": "#eeca3b"}


def _timeline_svg(plan: Plan, width: int = 1400) -> str:
    total = max(max(plan.task_end_ns, default=1), max(plan.action_end_ns, default=1), 1)
    sx = (width - 120) / total
    rows = [("compute", 20), ("fetch", 60), ("evict", 100)]
    out = [f'<svg xmlns="http://www.w3.org/2000/svg" width="{width}" height="150" '
           'font-family="monospace" font-size="11">']
    for name, y in rows:
        out.append(f'<text x="4" y="{y + 18}">{name}</text>')
    for t, s, e in zip(plan.program.tasks, plan.task_start_ns, plan.task_end_ns):
        out.append(f'<rect x="{100 + s * sx:.1f}" y="20" width="{max((e - s) * sx, 0.5):.1f}" '
                   f'height="28" fill="{_COLORS.get(t.kind, "#999")}"><title>{html.escape(t.name)} '
                   f'{(e - s) / 1e6:.2f} ms</title></rect>')
    for a, s, e in zip(plan.schedule.actions, plan.action_start_ns, plan.action_end_ns):
        if a.kind == "release":
            continue
        y = 60 if a.kind == "fetch" else 100
        name = plan.program.objects[a.object].name
        out.append(f'<rect x="{100 + s * sx:.1f}" y="{y}" width="{max((e - s) * sx, 0.5):.1f}" '
                   f'height="28" fill="{_COLORS[a.kind]}"><title>{a.kind} {html.escape(name)} '
                   f'{(e - s) / 1e6:.2f} ms</title></rect>')
    out.append("</svg>")
    return "\n".join(out)


def occupancy_series(plan: Plan) -> list[tuple[int, int]]:
    """(time_ns, device bytes held by planned stays) at every change point."""
    events = []
    for s in plan.stays:
        events.append((s.start_ns, s.bytes))
        events.append((s.end_ns, -s.bytes))
    events.sort()
    out, level = [], 0
    for t, d in events:
        level += d
        out.append((t, level))
    return out


def write_report(plan: Plan, directory: str | Path) -> Path:
    d = Path(directory)
    d.mkdir(parents=True, exist_ok=True)
    summary = asdict(plan.summary)
    summary["device_pool_bytes"] = plan.device_bytes
    summary["spill_pool_bytes"] = plan.spill_bytes
    summary["budgets"] = plan.budgets
    (d / "summary.json").write_text(json.dumps(summary, indent=1))
    with open(d / "tasks.csv", "w", newline="") as f:
        w = csv.writer(f)
        w.writerow(["index", "name", "kind", "stage", "microbatch", "variant", "profiled_ms",
                    "start_ms", "end_ms", "wait_ms", "workspace_bytes"])
        prev_end = 0
        for i, (t, s, e) in enumerate(zip(plan.program.tasks, plan.task_start_ns, plan.task_end_ns)):
            w.writerow([i, t.name, t.kind, t.stage, t.microbatch, t.variant, t.duration_ns / 1e6,
                        s / 1e6, e / 1e6, (s - prev_end) / 1e6, t.workspace_bytes])
            prev_end = e
    with open(d / "transfers.csv", "w", newline="") as f:
        w = csv.writer(f)
        w.writerow(["index", "kind", "object", "bytes", "trigger_task", "start_ms", "end_ms"])
        for i, (a, s, e) in enumerate(zip(plan.schedule.actions, plan.action_start_ns,
                                          plan.action_end_ns)):
            o = plan.program.objects[a.object]
            w.writerow([i, a.kind, o.name, o.bytes, a.trigger_task, s / 1e6, e / 1e6])
    (d / "timeline.json").write_text(json.dumps({
        "tasks": [{"name": t.name, "kind": t.kind, "start_ns": s, "end_ns": e}
                  for t, s, e in zip(plan.program.tasks, plan.task_start_ns, plan.task_end_ns)],
        "transfers": [{"kind": a.kind, "object": plan.program.objects[a.object].name,
                       "start_ns": s, "end_ns": e}
                      for a, s, e in zip(plan.schedule.actions, plan.action_start_ns,
                                         plan.action_end_ns) if a.kind != "release"],
        "occupancy": occupancy_series(plan)}))
    svg = _timeline_svg(plan)
    (d / "timeline.svg").write_text(svg)
    s = plan.summary
    rows = [("simulated step", f"{s.duration_seconds * 1e3:.1f} ms"),
            ("tokens / s (scheduled tokens)", f"{s.tokens_per_second:,.0f}"),
            ("compute", f"{s.compute_seconds * 1e3:.1f} ms"),
            ("waiting for inputs", f"{s.input_wait_seconds * 1e3:.1f} ms"),
            ("waiting for memory", f"{s.capacity_wait_seconds * 1e3:.1f} ms"),
            ("device pool (fixed layout)", f"{plan.device_bytes / GIB:.2f} GiB"),
            ("task workspace", f"{s.workspace_bytes / GIB:.2f} GiB"),
            ("spill pool", f"{plan.spill_bytes / GIB:.2f} GiB"),
            ("fetched / evicted per step", f"{s.fetch_bytes / GIB:.2f} / {s.evict_bytes / GIB:.2f} GiB"),
            ("walk / selection", f"{s.ordering} / {s.selection}"),
            ("search", f"{s.strategy} x {s.fetch_rule}; {s.candidates_feasible} of "
                       f"{s.candidates_evaluated} candidates feasible; {s.repairs_applied} repairs")]
    body = "".join(f"<tr><th align=left>{html.escape(k)}</th><td>{html.escape(v)}</td></tr>" for k, v in rows)
    (d / "index.html").write_text(
        "<!doctype html><meta charset=utf-8><title>plan report</title>"
        "<style>body{font-family:sans-serif;margin:2em}td,th{padding:2px 12px}</style>"
        f"<h1>Plan report</h1><table>{body}</table><h2>Timeline</h2>{svg}"
        "<p>Files: summary.json, tasks.csv, transfers.csv, timeline.json, timeline.svg</p>")
    return d / "index.html"
