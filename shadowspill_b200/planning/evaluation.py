"""Planner evaluation over a corpus of programs.

    python -m shadowspill_b200.planning.evaluation [--models llama3-8b,qwen35-9b,...] [--json OUT]

The corpus is the cross product of catalog models, batch geometries, walk orders and save/recompute
resolutions (the programs a preparation would hand to the planner). Every program is planned under
each residency strategy and fetch rule at the given budgets and host-link rates; the table answers
the questions one asks when changing the planner: which candidate wins where, how far apart the
candidates are, how long the search takes, and whether two planner builds (for instance the indexed
and the scanning reducer) agree. No GPU is involved: durations are the builder's analytic estimates
unless a profiles file is given.

Reference: tools/planning (corpus + evaluation: a 168-program corpus evaluated across search
configurations, tools/planning/evaluation/configs/*.json).
"""
from __future__ import annotations

import argparse
import json
import statistics
import sys
import time
from dataclasses import asdict, dataclass

import torch

from ..communication.info import CommunicationInfo
from ..frontend.capture import (BatchGeometry, StepDataOrdering, build_step, mixed_selection,
                                recompute_share_selections)
from ..models.config import preset
from ..profiling.measure import Profiles, apply_profiles
from .plan import MemoryBudgets, PlanningError, SearchOptions, plan_program

GIB = 1 << 30


@dataclass
class Case:
    model: str
    microbatch_tokens: int
    microbatches: int
    walk: str
    selection: str                   # name of the resolution
    program: object

    @property
    def name(self) -> str:
        return f"{self.model}/T{self.microbatch_tokens}x{self.microbatches}/{self.walk}/{self.selection}"


def corpus(models, geometries=((8192, 8), (4096, 16), (16384, 4)), walks=("breadth", "depth"),
           shares=(100, 50, 0), saved_variants=("save_attention", "save")) -> list[Case]:
    """models x geometries x walks x (recompute shares x saved variants, plus one mixed resolution)."""
    cases = []
    for name in models:
        cfg = preset(name)
        for T, n_mb in geometries:
            geo = BatchGeometry(microbatch_tokens=T, n_microbatches=n_mb, slots=T // 32 + 1, mean_seqlen=1200)
            selections: dict[str, dict[int, str]] = {}
            for variant in saved_variants:
                for share, sel in zip(shares, recompute_share_selections(cfg, shares, variant)):
                    selections["recompute" if share == 100 else f"{100 - share}%{variant}"] = sel
            selections[f"mixed:{cfg.n_layers // 4}"] = mixed_selection(cfg, cfg.n_layers // 4)
            for walk in walks:
                order = StepDataOrdering(walk=walk, optimizer="stage_interleaved" if walk == "breadth" else "tail")
                for sel_name, sel in selections.items():
                    if cfg.is_moe and sel:       # routed layers recompute only
                        continue
                    prog, _ = build_step(cfg, geo, order, dtype=torch.bfloat16, selection=sel)
                    cases.append(Case(name, T, n_mb, walk, sel_name, prog))
    return cases


def evaluate(cases: list[Case], budgets: MemoryBudgets, communication: CommunicationInfo,
             configurations: dict[str, SearchOptions], profiles: Profiles | None = None) -> list[dict]:
    """One row per (case, configuration): feasibility, simulated step, traffic, search time."""
    rows = []
    for case in cases:
        if profiles is not None:
            try:
                apply_profiles(case.program, profiles)
            except KeyError:
                pass                                  # a task the profiles do not cover keeps its estimate
        for label, options in configurations.items():
            t0 = time.perf_counter()
            try:
                plan = plan_program(case.program, budgets, communication, options)
                s = plan.summary
                rows.append({"case": case.name, "configuration": label, "feasible": True,
                             "simulated_ms": round(s.duration_seconds * 1e3, 2),
                             "compute_ms": round(s.compute_seconds * 1e3, 2),
                             "input_wait_ms": round(s.input_wait_seconds * 1e3, 2),
                             "fetch_gb": round(s.fetch_bytes / 1e9, 2), "evict_gb": round(s.evict_bytes / 1e9, 2),
                             "strategy": s.strategy, "fetch_rule": s.fetch_rule, "repairs": s.repairs_applied,
                             "layout_gib": round(s.layout_span_bytes / GIB, 2),
                             "search_ms": round((time.perf_counter() - t0) * 1e3, 1),
                             "actions": len(plan.schedule.actions)})
            except PlanningError as exc:
                rows.append({"case": case.name, "configuration": label, "feasible": False,
                             "error": str(exc).splitlines()[0],
                             "search_ms": round((time.perf_counter() - t0) * 1e3, 1)})
    return rows


def summarize(rows: list[dict]) -> dict:
    """Per configuration: how many cases plan, median search time, and how often it has the
    shortest simulated step among the configurations that plan the same case."""
    by_case: dict[str, list[dict]] = {}
    for r in rows:
        by_case.setdefault(r["case"], []).append(r)
    out: dict[str, dict] = {}
    for r in rows:
        c = out.setdefault(r["configuration"], {"cases": 0, "feasible": 0, "wins": 0, "search_ms": []})
        c["cases"] += 1
        c["search_ms"].append(r["search_ms"])
        if r["feasible"]:
            c["feasible"] += 1
            best = min(x["simulated_ms"] for x in by_case[r["case"]] if x["feasible"])
            c["wins"] += r["simulated_ms"] <= best * 1.0005
    for c in out.values():
        c["median_search_ms"] = round(statistics.median(c.pop("search_ms")), 1)
    return out


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--models", default="llama3-8b,qwen35-9b,olmoe-7b-a1b")
    ap.add_argument("--device-gib", type=float, default=24.0)
    ap.add_argument("--spill-gib", type=float, default=128.0)
    ap.add_argument("--fetch-gbs", type=float, default=55.0)
    ap.add_argument("--evict-gbs", type=float, default=55.0)
    ap.add_argument("--profiles", default="", help="profiles JSON written by a preparation (optional)")
    ap.add_argument("--compare-reducers", action="store_true",
                    help="also plan with the scanning reducer and report disagreements")
    ap.add_argument("--json", default="", help="write every row here")
    a = ap.parse_args(argv)
    comm = CommunicationInfo(fetch_solo_bps=a.fetch_gbs * 1e9, fetch_concurrent_bps=a.fetch_gbs * 0.9e9,
                             evict_solo_bps=a.evict_gbs * 1e9, evict_concurrent_bps=a.evict_gbs * 0.9e9)
    budgets = MemoryBudgets(int(a.device_gib * GIB), int(a.spill_gib * GIB))
    configurations = {"all": SearchOptions(),
                      "stall": SearchOptions(strategies=("stall",)),
                      "traffic": SearchOptions(strategies=("traffic",)),
                      "demand-only": SearchOptions(fetch_rules=("demand",))}
    if a.compare_reducers:
        configurations["all-scanning-reducer"] = SearchOptions(linear_reduce=True)
    profiles = Profiles.from_json(json.load(open(a.profiles))) if a.profiles else None
    cases = corpus([m for m in a.models.split(",") if m])
    rows = evaluate(cases, budgets, comm, configurations, profiles)
    summary = summarize(rows)
    print(f"{len(cases)} programs x {len(configurations)} configurations")
    for label, c in summary.items():
        print(f"  {label:22s} feasible {c['feasible']:3d}/{c['cases']:3d}  best-or-tied {c['wins']:3d}  "
              f"median search {c['median_search_ms']:.1f} ms")
    if a.compare_reducers:
        a_rows = {r["case"]: r for r in rows if r["configuration"] == "all"}
        b_rows = {r["case"]: r for r in rows if r["configuration"] == "all-scanning-reducer"}
        differ = [c for c in a_rows if a_rows[c].get("simulated_ms") != b_rows[c].get("simulated_ms")]
        print(f"  reducers disagree on {len(differ)} programs" + (f": {differ[:4]}" if differ else ""))
    if a.json:
        with open(a.json, "w") as f:
            json.dump({"budgets": asdict(budgets), "summary": summary, "rows": rows}, f, indent=1)
    return 0


if __name__ == "__main__":
    sys.exit(main())
