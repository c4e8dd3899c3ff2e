"""Compare hypothetical memory budgets and host-link rates without a GPU or a service.

    python examples/offline_sweep.py --export measurements.zip     # on the training machine, once
    python examples/offline_sweep.py measurements.zip               # anywhere: laptop, CI

The first form prepares a job (build, profile, calibrate, plan) and exports what planning
consumed. The second plans every candidate program again for three device budgets and three
transfer-rate assumptions and writes ``sweep.html`` with a link to the timeline and memory report
of every combination that fits. All timings are predictions for the measured machine.
"""
import argparse
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))


def export(path: str, model: str, device: str) -> str:
    from shadowspill_b200.planning.plan import SearchOptions
    from shadowspill_b200.training.session import TrainingSession, TrainingSetup
    cpu = device == "cpu"
    setup = TrainingSetup(model=model, device=device, dtype="float32" if cpu else "bfloat16",
                          device_gib=0.53 if cpu else 24.0, spill_gib=0.25 if cpu else 128.0,
                          tokens_per_step=512 if cpu else 65536, microbatch_tokens=256 if cpu else 8192,
                          profile=not cpu, calibrate=not cpu, recompute_shares=(100, 50, 0),
                          search=SearchOptions(minimum_object_bytes_evict_eligible=1024 if cpu else 1 << 20, workers=2))
    session = TrainingSession(setup)
    try:
        session.planning_inputs().save(path)
    finally:
        session.close()
    return path


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("measurements", nargs="?", help="exported planning inputs (measurements.zip)")
    ap.add_argument("--export", default="", help="prepare a job here and write its planning inputs to this path")
    ap.add_argument("--model", default="llama3-tiny")
    ap.add_argument("--device", default="cpu", choices=["cpu", "cuda"])
    ap.add_argument("--device-gib", type=float, nargs="*", default=None)
    ap.add_argument("--transfer-scale", type=float, nargs="*", default=[0.5, 1.0, 2.0])
    ap.add_argument("--output", default="sweep.html")
    a = ap.parse_args(argv)
    if a.export:
        print("planning inputs written to", export(a.export, a.model, a.device))
        return None
    from shadowspill_b200 import PlanningInputs
    inputs = PlanningInputs.load(a.measurements)
    own = inputs.budgets.device_bytes / (1 << 30)
    sweep = inputs.sweep(device_gib=a.device_gib or [own * 0.75, own, own * 1.5], transfer_scale=a.transfer_scale)
    sweep.write_report(a.output)
    for row in sweep.table():
        if row["feasible"]:
            print(f"{row['device_gib']:7.2f} GiB  link x{row['transfer_scale']:<4g} {row['seconds'] * 1e3:9.1f} ms  "
                  f"{row['tokens_per_second']:10,.0f} tokens/s  {row['candidate']}")
        else:
            print(f"{row['device_gib']:7.2f} GiB  link x{row['transfer_scale']:<4g} does not fit")
    print(f"open {a.output} beside its report directory")
    return sweep


if __name__ == "__main__":
    main()
