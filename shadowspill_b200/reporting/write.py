"""Plan report: ``index.html``, ``summary.json``, ``tasks.csv``, ``transfers.csv``,
``timeline.json``, ``occupancy.html`` and an SVG timeline, all static files readable offline.

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


def _occupancy_page(plan: Plan, width: int = 1400, height: int = 360) -> str:
    """Static page: device bytes held by planned stays over simulated time, against the
    pool size and the budget, with the ten largest stays alive at the peak."""
    series = occupancy_series(plan)
    total_ns = max([t for t, _ in series] + [1])
    cap = max([plan.device_bytes, plan.summary.logical_capacity_bytes or 0] + [v for _, v in series] + [1])
    sx, sy = (width - 80) / total_ns, (height - 40) / cap
    pts, level = [f"60,{height - 20}"], 0
    for t, v in series:
        x = 60 + t * sx
        pts.append(f"{x:.1f},{height - 20 - level * sy:.1f}")
        pts.append(f"{x:.1f},{height - 20 - v * sy:.1f}")
        level = v
    peak_t, peak = max(series, key=lambda p: p[1]) if series else (0, 0)
    alive = sorted((s for s in plan.stays if s.start_ns <= peak_t < s.end_ns), key=lambda s: -s.bytes)[:10]
    rows = "".join(f"<tr><td>{html.escape(plan.program.objects[s.object].name)}</td>"
                   f"<td>{s.bytes / (1 << 20):.1f} MiB</td><td>{s.offset}</td>"
                   f"<td>{s.start_ns / 1e6:.2f} - {s.end_ns / 1e6:.2f} ms</td></tr>" for s in alive)
    line = lambda v, color, label: (
        f'<line x1="60" x2="{width - 20}" y1="{height - 20 - v * sy:.1f}" y2="{height - 20 - v * sy:.1f}" '
        f'stroke="{color}" stroke-dasharray="6 4"/><text x="64" y="{height - 24 - v * sy:.1f}" '
        f'fill="{color}">{label} {v / GIB:.2f} GiB</text>')
    svg = (f'<svg xmlns="http://www.w3.org/2000/svg" width="{width}" height="{height}" '
           'font-family="monospace" font-size="11">'
           f'<polyline fill="none" stroke="#4c78a8" stroke-width="1.5" points="{" ".join(pts)}"/>'
           + line(plan.device_bytes, "#e45756", "device pool")
           + f'<text x="60" y="{height - 4}">0 ms</text>'
           f'<text x="{width - 90}" y="{height - 4}">{total_ns / 1e6:.0f} ms</text></svg>')
    return ("<!doctype html><meta charset=utf-8><title>occupancy</title>"
            "<style>body{font-family:sans-serif;margin:2em}td,th{padding:2px 12px;text-align:left}</style>"
            f"<h1>Device occupancy</h1><p>peak {peak / GIB:.2f} GiB at {peak_t / 1e6:.1f} ms; "
            f"pool {plan.device_bytes / GIB:.2f} GiB</p>{svg}"
            "<h2>Largest stays alive at the peak</h2><table><tr><th>object</th><th>size</th>"
            f"<th>offset</th><th>interval</th></tr>{rows}</table>")


def write_report(plan: Plan, directory: str | Path) -> Path:
    d = Path(directory)
    d.mkdir(parents=True, exist_ok=True)
    summary = asdict(plan.summary)
    summary["device_pool_bytes"] = plan.device_bytes
    summary["spill_pool_bytes"] = plan.spill_bytes       # pinned host memory
    summary["file_pool_bytes"] = plan.file_bytes         # file-backed (or remote) pool, 0 = none
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
        w.writerow(["index", "kind", "object", "bytes", "trigger_task", "start_ms", "end_ms", "home_pool"])
        for i, (a, s, e) in enumerate(zip(plan.schedule.actions, plan.action_start_ns,
                                          plan.action_end_ns)):
            o = plan.program.objects[a.object]
            w.writerow([i, a.kind, o.name, o.bytes, a.trigger_task, s / 1e6, e / 1e6,
                        plan.home_pool(a.object)])
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
    (d / "occupancy.html").write_text(_occupancy_page(plan))
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
        "<p>Files: summary.json, tasks.csv, transfers.csv, timeline.json, timeline.svg, "
        "<a href=occupancy.html>occupancy.html</a></p>")
    return d / "index.html"
