"""Offline planning: what would this job do with another memory budget or another host link?

``PlanningInputs`` holds what planning needs and nothing else: the candidate programs with their
measured task durations and workspaces already applied, the calibrated link rates, the budgets
and the search options. ``TrainingSession.planning_inputs()`` exports them after a preparation
(``measurements.zip``); ``PlanningInputs.load`` reads them on any machine (no GPU, no CUDA
libraries, no service), and ``sweep`` plans every candidate for every combination of device
budget, spill budget and transfer-rate scale. All timings are predictions for the machine the
measurements came from. ``OfflineSweep.write_report`` writes an HTML index that links to the full
plan report (timeline, occupancy, task and transfer tables) of every feasible cell.

Reference: ``PlanningInputs.load(...).sweep(device_gib=[...], transfer_scale=[...])`` of the
reference's offline planning workflow (examples/demos/offline_sweep.py:1-17).
"""
from __future__ import annotations

import html
import itertools
from dataclasses import asdict, dataclass, field, replace
from pathlib import Path

from ..artifacts.archive import load_archive, save_archive
from ..communication.info import CommunicationInfo
from ..ir.program import Program
from .plan import GIB, MemoryBudgets, PlanningError, SearchOptions, SweepResult, sweep_programs

KIND = "planning_inputs"


@dataclass
class SweepCell:
    device_gib: float
    spill_gib: float
    transfer_scale: float
    result: SweepResult | None
    error: str = ""

    @property
    def seconds(self) -> float | None:
        return None if self.result is None else self.result.best.summary.duration_seconds


@dataclass
class OfflineSweep:
    cells: list[SweepCell]
    labels: list[str]
    tokens: int = 0

    def table(self) -> list[dict]:
        rows = []
        for c in self.cells:
            row = {"device_gib": c.device_gib, "spill_gib": c.spill_gib, "transfer_scale": c.transfer_scale,
                   "feasible": c.result is not None}
            if c.result is not None:
                s = c.result.best.summary
                chosen = next(i for i, p in enumerate(c.result.plans) if p is c.result.best)
                row.update(seconds=s.duration_seconds, tokens_per_second=s.tokens_per_second,
                           candidate=self.labels[chosen] if chosen < len(self.labels) else str(chosen),
                           fetch_gb=s.fetch_bytes / 1e9, evict_gb=s.evict_bytes / 1e9)
            else:
                row["error"] = c.error.splitlines()[0] if c.error else ""
            rows.append(row)
        return rows

    def write_report(self, path: str | Path) -> Path:
        """``path`` (an ``.html`` file) plus a directory of the same stem with one plan report per
        feasible cell."""
        from ..reporting.write import write_report
        path = Path(path)
        root = path.with_suffix("")
        root.mkdir(parents=True, exist_ok=True)
        lines = ["<!doctype html><meta charset='utf-8'><title>Offline planning sweep</title>",
                 "<style>body{font-family:sans-serif}td,th{padding:4px 10px;text-align:right;border-bottom:1px solid #ddd}"
                 "</style>", "<h1>Offline planning sweep</h1>",
                 "<p>Predictions for the machine the measurements were taken on.</p>",
                 "<table><tr><th>device GiB</th><th>spill GiB</th><th>transfer rate x</th><th>step ms</th>"
                 "<th>tokens/s</th><th>candidate</th><th>fetch GB</th><th>evict GB</th><th>report</th></tr>"]
        for c, row in zip(self.cells, self.table()):
            head = f"<tr><td>{c.device_gib:g}</td><td>{c.spill_gib:g}</td><td>{c.transfer_scale:g}</td>"
            if c.result is None:
                lines.append(head + f"<td colspan=6 style='text-align:left'>does not fit: {html.escape(row['error'])}</td></tr>")
                continue
            name = f"d{c.device_gib:g}_s{c.spill_gib:g}_x{c.transfer_scale:g}".replace(".", "p")
            write_report(c.result.best, root / name)
            lines.append(head + f"<td>{row['seconds'] * 1e3:,.1f}</td><td>{row['tokens_per_second']:,.0f}</td>"
                         f"<td style='text-align:left'>{html.escape(str(row['candidate']))}</td>"
                         f"<td>{row['fetch_gb']:.1f}</td><td>{row['evict_gb']:.1f}</td>"
                         f"<td><a href='{root.name}/{name}/index.html'>plan</a></td></tr>")
        lines.append("</table>")
        path.write_text("\n".join(lines))
        return path


@dataclass
class PlanningInputs:
    programs: list[Program]
    communication: CommunicationInfo
    budgets: MemoryBudgets
    labels: list[str] = field(default_factory=list)
    search: SearchOptions = field(default_factory=SearchOptions)

    # ------------------------------------------------------------------ files
    def save(self, path: str | Path) -> Path:
        meta = {"programs": [p.to_json() for p in self.programs], "communication": self.communication.to_json(),
                "budgets": asdict(self.budgets), "labels": list(self.labels), "search": asdict(self.search)}
        return save_archive(path, KIND, meta)

    @staticmethod
    def load(path: str | Path) -> "PlanningInputs":
        meta, _ = load_archive(path, KIND)
        search = dict(meta.get("search") or {})
        for k in ("strategies", "fetch_rules"):
            if k in search and search[k] is not None:
                search[k] = tuple(search[k])
        return PlanningInputs([Program.from_json(p) for p in meta["programs"]],
                              CommunicationInfo.from_json(meta["communication"]),
                              MemoryBudgets(**meta["budgets"]), list(meta.get("labels") or []),
                              SearchOptions(**search))

    # ------------------------------------------------------------------ planning
    def scaled_link(self, scale: float) -> CommunicationInfo:
        c = self.communication
        return replace(c, fetch_solo_bps=c.fetch_solo_bps * scale, fetch_concurrent_bps=c.fetch_concurrent_bps * scale,
                       evict_solo_bps=c.evict_solo_bps * scale, evict_concurrent_bps=c.evict_concurrent_bps * scale,
                       source=f"{c.source} x{scale:g}")

    def sweep(self, device_gib=None, spill_gib=None, transfer_scale=(1.0,), threads: int = 4) -> OfflineSweep:
        """Every combination of the given device budgets, spill budgets and link-rate scales (each
        defaults to the measured run's own value)."""
        devices = list(device_gib) if device_gib is not None else [self.budgets.device_bytes / GIB]
        spills = list(spill_gib) if spill_gib is not None else [self.budgets.spill_bytes / GIB]
        cells = []
        tokens = int(self.programs[0].metadata.get("tokens", 0)) if self.programs else 0
        for d, s, x in itertools.product(devices, spills, list(transfer_scale)):
            if d <= 0 or s <= 0 or x <= 0:
                raise ValueError("budgets and transfer scales must be positive")
            budgets = replace(self.budgets, device_bytes=int(d * GIB), spill_bytes=int(s * GIB))
            try:
                cells.append(SweepCell(d, s, x, sweep_programs(self.programs, budgets, self.scaled_link(x),
                                                               self.search, threads=threads)))
            except PlanningError as exc:
                cells.append(SweepCell(d, s, x, None, str(exc)))
        return OfflineSweep(cells, list(self.labels), tokens)
