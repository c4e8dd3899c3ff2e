"""Prepare once, train many times: save a run's plans and start later runs from them.

    python examples/saved_plan.py                      # CPU workers, tiny model, service in this process

The first run prepares (build, profile, calibrate, plan) and its plans are exported to
``plans.tar``; the second run uploads that file and starts from it, which skips preparation. The
command table shows each step's service time beside the plan's prediction. On a real deployment
the two halves are different days, or different services: only the file travels.
"""
import sys
import tempfile
from pathlib import Path

import numpy as np

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))

from shadowspill_b200.client import (BatchConfig, CommandTable, Memory, Model, Optimizer, Preparation,
                                     ProfilingOptions, Resources, ServiceClient, text_batch,
                                     text_batch_statistics)
from shadowspill_b200.client.config import PlanningOptions
from shadowspill_b200.server.service import Server


def sequences(seed, n=8, vocab=512):
    rng = np.random.default_rng(seed)
    return [rng.integers(0, vocab, size=int(rng.integers(16, 60))) for _ in range(n)]


def main(steps: int = 3) -> dict:
    settings = dict(model=Model("llama3-tiny", dtype="float32"),
                    optimizer=Optimizer(lr=3e-3, parameter_rounding="nearest"),
                    batch=BatchConfig(tokens_per_step=512, microbatch_tokens=256),
                    memory=Memory(device_gib=0.53, spill_gib=0.25), resources=Resources(gpus=1, backend="cpu"),
                    preparation=Preparation(profiling=ProfilingOptions(enabled=False), calibrate=False,
                                            planning=PlanningOptions(minimum_object_bytes_evict_eligible=1024,
                                                                     workers=1)))
    out = {}
    with tempfile.TemporaryDirectory() as root, Server(root, token="secret") as server:
        saved = Path(root) / "plans.tar"
        with ServiceClient(server.url, token="secret") as svc:                 # day one: prepare and save
            prepared = svc.prepare_training(**settings).result()
            plans = svc.plans_of(prepared["run"])
            first = plans.summary().result()["plans"][0]
            print(f"prepared: simulated step {first['duration_seconds'] * 1e3:.2f} ms, "
                  f"{first['fetch_bytes'] / 1e6:.1f} MB fetched per step")
            plans.export(saved).result()
            out["prepared_seconds"] = first["duration_seconds"]
        with ServiceClient(server.url, token="secret") as svc:                 # later: start from the file
            trainer = svc.create_training_client(settings["model"], settings["optimizer"],
                                                 plans=svc.import_plans(saved).result(), timeout=300,
                                                 progress=True, **{k: v for k, v in settings.items()
                                                                   if k not in ("model", "optimizer")}).result()
            table = CommandTable()
            losses = []
            for i in range(steps):
                batch = text_batch(sequences(i % 2))
                check = trainer.validate_batch(batch)
                fut = table.track("step", trainer.step(batch), batch=text_batch_statistics(batch),
                                  planned_seconds=check.estimated_seconds)
                losses.append(fut.result().loss)
            out["losses"] = losses
            out["skipped_preparation"] = any("skipped" in ln for ln in svc.get_progress(trainer.run).result()["lines"])
            trainer.close()
    return out


if __name__ == "__main__":
    main()
