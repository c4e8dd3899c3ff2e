"""Measure an existing plan: open a prepared bundle, run updates, report what they cost.

    python -m shadowspill_b200.execution.measure_plan --bundle training.ssp --setup setup.json \\
        --steps 7 --warmup 1 --output runs/measurement

Nothing is built, profiled or searched when the bundle matches the setup (the session says so in
its log and this tool refuses to go on otherwise, unless ``--allow-prepare`` is given): the point is
to time the plan one already has, for instance after a driver update or on another box of the same
kind. Inputs come from ``inputs(update_index) -> list[HostMicrobatch]``; the command line uses the
synthetic packed batches. Per update the report has the device-timed step, the end-to-end time
through ``TrainingSession.step``, the loss, and the runtime's transfer counters; the summary adds
units per second (tokens by default) and the simulated step of the plan beside the measured one.

Reference: tools/measure_plan (``run(plan, initializer=..., inputs=..., steps=..., warmup_steps=...,
units_per_step=..., unit_label=...)``, api.py / report.py / updates.py).
"""
from __future__ import annotations

import argparse
import json
import statistics
import sys
import time
from pathlib import Path
from typing import Callable

from ..training.session import TrainingSession, TrainingSetup


def run(setup: TrainingSetup, inputs: Callable[[int], list] | None = None, steps: int = 7,
        warmup_steps: int = 1, output_dir: str | Path | None = None, units_per_step: int | None = None,
        unit_label: str = "tokens", allow_prepare: bool = False, log=None) -> dict:
    """Runs ``warmup_steps + steps`` updates of the plan in ``setup.bundle`` and returns the report
    (also written to ``output_dir`` as ``measurement.json`` and ``measurement.md``)."""
    if not setup.bundle:
        raise ValueError("measure_plan needs TrainingSetup.bundle: the prepared plan to measure")
    session = TrainingSession(setup, log=log)
    try:
        if not session.prepared_from_bundle and not allow_prepare:
            raise RuntimeError(f"{setup.bundle} does not match this setup (or does not exist): measuring it "
                               "would first build, profile and plan. Pass allow_prepare=True to do that.")
        if inputs is None:
            from ..data.synthetic import make_batch
            cfg = session.cfg

            def inputs(i: int):
                return make_batch(i, vocab=cfg.vocab_size, tokens_per_step=setup.tokens_per_step,
                                  microbatch_tokens=setup.microbatch_tokens, slots=session.slots,
                                  max_len=min(8192, setup.microbatch_tokens))
        units = units_per_step if units_per_step is not None else setup.tokens_per_step
        updates = []
        before = session.executor.rt.stats()
        for i in range(warmup_steps + steps):
            batch = inputs(i)
            t0 = time.perf_counter()
            res = session.step(batch)
            wall = time.perf_counter() - t0
            now = session.executor.rt.stats()
            updates.append({"update": i + 1, "warmup": i < warmup_steps, "loss": res.loss,
                            "device_seconds": res.device_seconds, "wall_seconds": wall,
                            "fetch_bytes": now["fetch_bytes"] - before["fetch_bytes"],
                            "evict_bytes": now["evict_bytes"] - before["evict_bytes"]})
            before = now
        timed = [u for u in updates if not u["warmup"]]
        dev = [u["device_seconds"] or u["wall_seconds"] for u in timed]
        summary = {"bundle": str(setup.bundle), "prepared_from_bundle": session.prepared_from_bundle,
                   "steps": steps, "warmup_steps": warmup_steps, "unit": unit_label,
                   "units_per_step": units,
                   "median_step_seconds": statistics.median(dev), "min_step_seconds": min(dev),
                   "max_step_seconds": max(dev),
                   f"{unit_label}_per_second": units / statistics.median(dev),
                   "simulated_step_seconds": session.plan.summary.duration_seconds,
                   "measured_over_simulated": statistics.median(dev) / max(session.plan.summary.duration_seconds, 1e-12),
                   "plan": {"ordering": session.plan.summary.ordering, "selection": session.plan.summary.selection,
                            "strategy": session.plan.summary.strategy, "fetch_rule": session.plan.summary.fetch_rule,
                            "device_pool_bytes": session.plan.device_bytes, "spill_bytes": session.plan.spill_bytes}}
        report = {"summary": summary, "updates": updates}
        if output_dir:
            out = Path(output_dir)
            out.mkdir(parents=True, exist_ok=True)
            (out / "measurement.json").write_text(json.dumps(report, indent=1))
            lines = [f"# Plan measurement: {setup.bundle}", "",
                     f"{steps} timed updates after {warmup_steps} warm-up; median step "
                     f"{summary['median_step_seconds'] * 1e3:.1f} ms "
                     f"({summary[unit_label + '_per_second']:.0f} {unit_label}/s), simulated "
                     f"{summary['simulated_step_seconds'] * 1e3:.1f} ms "
                     f"(measured / simulated = {summary['measured_over_simulated']:.3f}).", "",
                     "| update | loss | device ms | wall ms | fetched MB | evicted MB |", "|---|---|---|---|---|---|"]
            for u in updates:
                lines.append(f"| {u['update']}{' (warm-up)' if u['warmup'] else ''} | {u['loss']:.5f} | "
                             f"{(u['device_seconds'] or 0) * 1e3:.2f} | {u['wall_seconds'] * 1e3:.2f} | "
                             f"{u['fetch_bytes'] / 1e6:.1f} | {u['evict_bytes'] / 1e6:.1f} |")
            (out / "measurement.md").write_text("\n".join(lines) + "\n")
        return report
    finally:
        session.close()


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--bundle", required=True, help="training.ssp written by a preparation")
    ap.add_argument("--setup", required=True, help="JSON file with the TrainingSetup fields the bundle was made for")
    ap.add_argument("--steps", type=int, default=7)
    ap.add_argument("--warmup", type=int, default=1)
    ap.add_argument("--output", default="")
    ap.add_argument("--allow-prepare", action="store_true")
    a = ap.parse_args(argv)
    fields = json.load(open(a.setup))
    fields["bundle"] = a.bundle
    setup = TrainingSetup(**fields)
    rep = run(setup, steps=a.steps, warmup_steps=a.warmup, output_dir=a.output or None,
              allow_prepare=a.allow_prepare, log=lambda m: print(f"[measure_plan] {m}", file=sys.stderr))
    print(json.dumps(rep["summary"]))
    return 0


if __name__ == "__main__":
    sys.exit(main())
