"""Runtime report: what a traced step really did next to what the plan said it
would do. Writes ``runtime.html`` (summary, per-phase table, the worst tasks and
a two-row timeline per lane: simulated above, measured below), ``runtime.json``,
``runtime_tasks.csv`` and ``runtime_transfers.csv``; all static files.

The reference serves the same page from a traced step
(packages/client/src/shadowspill_client/traces.py:91 ``download_report("runtime.html")``;
fields in docs/python/advanced/step-diagnostics.md:118-175).
"""
from __future__ import annotations

import csv
import html
import json
from dataclasses import asdict, fields
from pathlib import Path

from ..diagnostics.step import StepDiagnostics, TaskRow, TransferRow
from ..ir.plan import Plan
from .write import _COLORS


def _lanes_svg(diag: StepDiagnostics, width: int = 1400) -> str:
    total = max(diag.makespan_s, diag.simulated_makespan_s,
                max((t.real_start_s + t.real_s for t in diag.transfers), default=0.0), 1e-9)
    sx = (width - 150) / total
    lanes = [("compute plan", 10), ("compute real", 34), ("fetch plan", 68), ("fetch real", 92),
             ("evict plan", 126), ("evict real", 150)]
    out = [f'<svg xmlns="http://www.w3.org/2000/svg" width="{width}" height="185" '
           'font-family="monospace" font-size="11">']
    for name, y in lanes:
        out.append(f'<text x="4" y="{y + 14}">{name}</text>')

    def rect(y, start, dur, color, title):
        out.append(f'<rect x="{130 + start * sx:.1f}" y="{y}" width="{max(dur * sx, 0.4):.1f}" '
                   f'height="20" fill="{color}"><title>{html.escape(title)}</title></rect>')

    for r in diag.tasks:
        c = _COLORS.get(r.kind, "#999")
        rect(10, r.simulated_start_s, r.simulated_s, c, f"{r.name} plan {r.simulated_s * 1e3:.2f} ms")
        rect(34, r.real_start_s, r.real_s, c, f"{r.name} real {r.real_s * 1e3:.2f} ms")
    for t in diag.transfers:
        y = 68 if t.kind == "fetch" else 126
        c = _COLORS.get(t.kind, "#999")
        rect(y, t.simulated_start_s, t.simulated_s, c, f"{t.kind} {t.object} plan {t.simulated_s * 1e3:.2f} ms")
        if t.real_s > 0:
            rect(y + 24, t.real_start_s, t.real_s, c,
                 f"{t.kind} {t.object} real {t.real_s * 1e3:.2f} ms ({t.gbps:.1f} GB/s)")
    out.append("</svg>")
    return "\n".join(out)


def _table(header, rows) -> str:
    h = "".join(f"<th>{html.escape(str(c))}</th>" for c in header)
    b = "".join("<tr>" + "".join(f"<td>{html.escape(str(c))}</td>" for c in r) + "</tr>" for r in rows)
    return f"<table><tr>{h}</tr>{b}</table>"


def _write_rows(path: Path, cls, rows) -> None:
    names = [f.name for f in fields(cls)]
    with open(path, "w", newline="") as f:
        w = csv.writer(f)
        w.writerow(names)
        for r in rows:
            w.writerow([getattr(r, n) for n in names])


def write_runtime_report(plan: Plan, diag: StepDiagnostics, directory: str | Path) -> Path:
    d = Path(directory)
    d.mkdir(parents=True, exist_ok=True)
    (d / "runtime.json").write_text(json.dumps(diag.to_json(rows=False), indent=1))
    _write_rows(d / "runtime_tasks.csv", TaskRow, diag.tasks)
    _write_rows(d / "runtime_transfers.csv", TransferRow, diag.transfers)
    ms = lambda s: f"{s * 1e3:.1f} ms"
    summary = [
        ("measured step (device)", ms(diag.makespan_s)),
        ("simulated step", ms(diag.simulated_makespan_s)),
        ("tokens / s (supplied tokens / traced time)", f"{diag.tokens_per_second:,.0f}"),
        ("task time: real / simulated / profiled",
         f"{ms(diag.task_seconds_real)} / {ms(diag.task_seconds_simulated)} / {ms(diag.task_seconds_profiled)}"),
        ("idle between tasks: real / simulated", f"{ms(diag.idle_seconds_real)} / {ms(diag.idle_seconds_simulated)}"),
        ("  waiting for inputs", ms(diag.input_readiness_wait_seconds)),
        ("  waiting for a reused range", ms(diag.allocation_reuse_wait_seconds)),
        ("  exposed frontend overhead", ms(diag.frontend_overhead_seconds)),
        ("entry delay / terminal tail", f"{ms(diag.entry_delay_seconds)} / {ms(diag.terminal_tail_seconds)}"),
        ("optimizer span", ms(diag.optimizer_span_seconds)),
        ("host cycle", ms(diag.cycle_seconds)),
        ("trace complete", str(diag.trace_complete)),
    ]
    phase_rows = [(k, int(p["tasks"]), ms(p["profiled_s"]), ms(p["simulated_s"]), ms(p["real_s"]),
                   f'{(p["real_s"] / p["profiled_s"] if p["profiled_s"] else 0):.3f}', ms(p["gap_s"]))
                  for k, p in sorted(diag.phases.items())]
    worst = [(r.index, r.name, ms(r.profiled_s), ms(r.real_s), ms(r.gap_before_s), r.waited_inputs,
              r.waited_reuse) for r in diag.worst_tasks(15)]
    lanes = {}
    for t in diag.transfers:
        a = lanes.setdefault(t.kind, [0, 0.0, 0.0])
        a[0] += t.bytes
        a[1] += t.real_s
        a[2] += t.simulated_s
    lane_rows = [(k, f"{v[0] / 1e9:.2f} GB", ms(v[1]), ms(v[2]),
                  f"{(v[0] / v[1] * 1e-9 if v[1] else 0):.1f} GB/s") for k, v in sorted(lanes.items())]
    body = "".join(f"<tr><th align=left>{html.escape(k)}</th><td>{html.escape(v)}</td></tr>"
                   for k, v in summary)
    runtime_rows = [(k, v) for k, v in diag.runtime.items()]
    (d / "runtime.html").write_text(
        "<!doctype html><meta charset=utf-8><title>runtime report</title>"
        "<style>body{font-family:sans-serif;margin:2em}td,th{padding:2px 12px;text-align:left}"
        "table{border-collapse:collapse;margin-bottom:1.5em}</style>"
        f"<h1>Runtime report</h1><table>{body}</table>"
        f"<h2>Timeline (plan above, measured below)</h2>{_lanes_svg(diag)}"
        "<h2>Phases</h2>"
        + _table(["phase", "tasks", "profiled", "simulated", "real", "real / profiled", "idle before"],
                 phase_rows)
        + "<h2>Transfer lanes</h2>"
        + _table(["lane", "bytes", "busy (real)", "busy (simulated)", "rate while busy"], lane_rows)
        + "<h2>Tasks furthest over their profile</h2>"
        + _table(["#", "task", "profiled", "real", "idle before", "input waits", "reuse waits"], worst)
        + ("<h2>Runtime counters</h2>" + _table(["counter", "value"], runtime_rows) if runtime_rows else "")
        + "<p>Files: runtime.json, runtime_tasks.csv, runtime_transfers.csv</p>")
    return d / "runtime.html"
