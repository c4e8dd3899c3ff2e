"""Where a measured step differs from its simulation: lanes, kinds, waits and interference.

    python -m shadowspill_b200.qualification.gap_report REPORT_DIR [--json OUT]

``REPORT_DIR`` is what a traced step writes (``TrainingSession.traced_step(batch, directory)``,
``bench.py --report DIR``): it holds ``runtime_tasks.csv`` with one row per task (profiled,
simulated and measured start and duration). The planner's timeline has one lane; the executor
has two (compute stream and communication stream), so a task-by-task difference says little.
This report separates them:

  lanes          busy time and gaps of the compute lane (forward, backward, head, unsharded
                 update) and of the communication lane (collectives, sharded update)
  kinds          per task kind: count, measured, profiled, ratio
  waits          every gap on the compute lane, attributed to the communication task that ended
                 when the gap did (the compute task waited for it), else to the runtime's own
                 record (input fetch, range reuse), else to the host being late
  interference   compute tasks that ran beside a communication task against those that ran
                 alone: measured over profiled for each group. A ratio well above the other
                 group's means the two streams slow each other down

Reference: qualification/gap_report.py of the reference repository (measured-vs-simulated
breakdown of a traced step).
"""
from __future__ import annotations

import argparse
import csv
import json
import sys
from collections import defaultdict
from dataclasses import asdict, dataclass, field
from pathlib import Path

EDGE = 50e-6          # two events closer than this are the same moment (event timing resolution)


@dataclass
class Row:
    index: int
    name: str
    kind: str
    profiled_s: float
    simulated_s: float
    start_s: float
    real_s: float
    waited_inputs: int = 0
    waited_reuse: int = 0

    @property
    def end_s(self) -> float:
        return self.start_s + self.real_s


@dataclass
class GapReport:
    makespan_s: float
    simulated_s: float
    lanes: dict = field(default_factory=dict)
    kinds: dict = field(default_factory=dict)
    waits: dict = field(default_factory=dict)
    longest_gaps: list = field(default_factory=list)
    interference: dict = field(default_factory=dict)
    exposure: dict = field(default_factory=dict)

    def to_json(self) -> dict:
        return asdict(self)

    def text(self) -> str:
        ms = lambda s: f"{s * 1e3:9.1f}"
        out = [f"step: measured {self.makespan_s * 1e3:.1f} ms, simulated {self.simulated_s * 1e3:.1f} ms "
               f"({(self.makespan_s / self.simulated_s - 1) * 100 if self.simulated_s else 0:+.1f} %)", "",
               f"{'lane':<15}{'tasks':>7}{'busy ms':>11}{'gaps ms':>11}{'profiled ms':>13}"]
        for lane, v in self.lanes.items():
            out.append(f"{lane:<15}{v['tasks']:>7}{ms(v['busy_s']):>11}{ms(v['gap_s']):>11}{ms(v['profiled_s']):>13}")
        out += ["", f"{'kind':<15}{'tasks':>7}{'measured ms':>13}{'profiled ms':>13}{'ratio':>8}"]
        for kind, v in self.kinds.items():
            ratio = v["real_s"] / v["profiled_s"] if v["profiled_s"] else 0.0
            out.append(f"{kind:<15}{v['tasks']:>7}{ms(v['real_s']):>13}{ms(v['profiled_s']):>13}{ratio:>8.2f}")
        out += ["", "gaps on the compute lane, by what the next task waited for:"]
        for why, v in sorted(self.waits.items(), key=lambda kv: -kv[1]["seconds"]):
            out.append(f"  {why:<34}{v['count']:>6} gaps{ms(v['seconds']):>11} ms")
        if self.longest_gaps:
            out.append("  longest: " + ", ".join(f"{g['before']} {g['seconds'] * 1e3:.1f} ms ({g['why']})"
                                                 for g in self.longest_gaps[:5]))
        i = self.interference
        if i:
            out += ["", "compute tasks beside a communication task vs alone (measured / profiled):",
                    f"  beside: {i['beside']['tasks']:>5} tasks, ratio {i['beside']['ratio']:.2f}, "
                    f"{i['beside']['excess_s'] * 1e3:.1f} ms over profile",
                    f"  alone:  {i['alone']['tasks']:>5} tasks, ratio {i['alone']['ratio']:.2f}, "
                    f"{i['alone']['excess_s'] * 1e3:.1f} ms over profile"]
        e = self.exposure
        if e:
            out += ["", f"communication-stream tasks cost the compute lane {e['seconds'] * 1e3:.1f} ms "
                        f"({e['per_task_us']:.0f} us each over {e['tasks']} tasks; planned with {e['planned_per_task_us']:.0f} us each)",
                    f"  to plan with the measured figure: collective_overhead_us = {e['suggested_overhead_us']:.0f}"]
        return "\n".join(out)


def lane_of(row: Row, sharded: bool) -> str:
    if row.kind == "collective" or (sharded and row.kind == "optimizer"):
        return "communication"
    return "compute"


def build(rows: list[Row], simulated_s: float = 0.0) -> GapReport:
    if not rows:
        return GapReport(0.0, simulated_s)
    sharded = any(r.kind == "collective" for r in rows)
    lanes = {"compute": [r for r in rows if lane_of(r, sharded) == "compute"],
             "communication": [r for r in rows if lane_of(r, sharded) == "communication"]}
    makespan = max(r.end_s for r in rows)
    rep = GapReport(makespan, simulated_s or sum(r.simulated_s for r in rows))
    side = sorted(lanes["communication"], key=lambda r: r.end_s)
    for lane, members in lanes.items():
        if not members:
            continue
        members = sorted(members, key=lambda r: r.start_s)
        gap, prev = 0.0, 0.0
        for r in members:
            gap += max(0.0, r.start_s - prev)
            prev = max(prev, r.end_s)
        rep.lanes[lane] = {"tasks": len(members), "busy_s": sum(r.real_s for r in members), "gap_s": gap,
                           "profiled_s": sum(r.profiled_s for r in members)}
    for r in rows:
        k = rep.kinds.setdefault(r.kind, {"tasks": 0, "real_s": 0.0, "profiled_s": 0.0})
        k["tasks"] += 1
        k["real_s"] += r.real_s
        k["profiled_s"] += r.profiled_s
    # ---- compute-lane gaps and what ended them
    compute = sorted(lanes["compute"], key=lambda r: r.start_s)
    waits = defaultdict(lambda: {"count": 0, "seconds": 0.0})
    gaps = []
    prev_end = 0.0
    for r in compute:
        g = r.start_s - prev_end
        prev_end = max(prev_end, r.end_s)
        if g <= EDGE:
            continue
        blocker = next((s for s in side if abs(s.end_s - r.start_s) <= EDGE), None)
        if blocker is not None:
            why = f"end of a {blocker.name.split('.')[0]} task (communication lane)"
        elif r.waited_inputs:
            why = "input fetch"
        elif r.waited_reuse:
            why = "range reuse"
        elif r is compute[0]:
            why = "entry of the step"
        else:
            why = "host (frontend late)"
        waits[why]["count"] += 1
        waits[why]["seconds"] += g
        gaps.append({"before": r.name, "seconds": g, "why": why})
    rep.waits = dict(waits)
    rep.longest_gaps = sorted(gaps, key=lambda g: -g["seconds"])[:10]
    # ---- interference: compute tasks overlapped by a communication task for at least a tenth of their time
    if side:
        groups = {"beside": [], "alone": []}
        for r in compute:
            if r.real_s <= 0 or r.profiled_s <= 0:
                continue
            over = sum(max(0.0, min(r.end_s, s.end_s) - max(r.start_s, s.start_s)) for s in side)
            groups["beside" if over >= 0.1 * r.real_s else "alone"].append(r)
        for name, members in groups.items():
            real, prof = sum(r.real_s for r in members), sum(r.profiled_s for r in members)
            rep.interference[name] = {"tasks": len(members), "ratio": real / prof if prof else 0.0,
                                      "excess_s": real - prof}
        # what the communication lane cost the compute lane: the gaps it caused, plus the slowdown of the
        # compute tasks beside it relative to how the tasks that ran alone compare with their profiles
        gaps = sum(v["seconds"] for why, v in rep.waits.items() if "communication lane" in why)
        base = rep.interference["alone"]["ratio"] or 1.0
        beside = groups["beside"]
        slowed = sum(r.real_s for r in beside) - base * sum(r.profiled_s for r in beside)
        cost = gaps + max(0.0, slowed)
        planned = sum(s_.profiled_s for s_ in side)
        rep.exposure = {"seconds": cost, "tasks": len(side), "per_task_us": cost / len(side) * 1e6,
                        "planned_per_task_us": planned / len(side) * 1e6,
                        "suggested_overhead_us": max(0.0, (cost - planned) / len(side) * 1e6)}
    return rep


def read_tasks_csv(path: str | Path) -> list[Row]:
    rows = []
    with open(path, newline="") as f:
        for d in csv.DictReader(f):
            rows.append(Row(int(d["index"]), d["name"], d["kind"], float(d["profiled_s"]), float(d["simulated_s"]),
                            float(d["real_start_s"]), float(d["real_s"]), int(d.get("waited_inputs") or 0),
                            int(d.get("waited_reuse") or 0)))
    return rows


def from_diagnostics(diag) -> GapReport:
    """From a ``diagnostics.step.StepDiagnostics`` (no files involved)."""
    rows = [Row(t.index, t.name, t.kind, t.profiled_s, t.simulated_s, t.real_start_s, t.real_s,
                t.waited_inputs, t.waited_reuse) for t in diag.tasks]
    return build(rows, diag.simulated_makespan_s)


def from_directory(directory: str | Path) -> GapReport:
    directory = Path(directory)
    rows = read_tasks_csv(directory / "runtime_tasks.csv")
    simulated = 0.0
    summary = directory / "runtime.json"
    if summary.exists():
        simulated = float(json.loads(summary.read_text()).get("simulated_makespan_s", 0.0))
    return build(rows, simulated)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("directory", help="runtime report directory of a traced step")
    ap.add_argument("--json", default="", help="also write the report as JSON to this path")
    a = ap.parse_args(argv)
    rep = from_directory(a.directory)
    print(rep.text())
    if a.json:
        Path(a.json).write_text(json.dumps(rep.to_json(), indent=1))
    return 0


if __name__ == "__main__":
    sys.exit(main())
