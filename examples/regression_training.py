"""Train the small non-text regression model through the service on CPU workers.

    python examples/regression_training.py [--ranks 2] [--steps 10]

The caller owns the data: every update gets ``ranks x samples`` rows drawn from a seeded
generator, each row a ``tensor_datum`` with its input ``value`` (16 floats), its
``target_values`` (8 floats) and the weight that makes the summed loss the batch mean.
"""
import argparse
import sys
import tempfile
from pathlib import Path

import numpy as np

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))

from shadowspill_b200.client import (BatchConfig, Memory, Model, Objective, Optimizer, Preparation,
                                     ProfilingOptions, Resources, ServiceClient, data_parallel,
                                     tensor_datum)
from shadowspill_b200.client.config import PlanningOptions
from shadowspill_b200.server.service import Server


def rows(update: int, ranks: int, samples: int, seed: int = 711):
    batch = []
    for rank in range(ranks):
        g = np.random.Generator(np.random.PCG64(seed + rank * 1_000_003))     # a fixed task per rank
        values = g.standard_normal((samples, 16), np.float32)
        targets = np.tanh(values[:, :8] * 0.5 + values[:, 8:] * 0.25)
        weight = 1.0 / (ranks * samples * 8)
        batch += [tensor_datum({"value": v, "target_values": t}, weight) for v, t in zip(values, targets)]
    return batch


def main(argv=None) -> list[float]:
    ap = argparse.ArgumentParser()
    ap.add_argument("--ranks", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--samples", type=int, default=8, help="rows per rank and update")
    a = ap.parse_args(argv)
    losses = []
    with tempfile.TemporaryDirectory() as root, Server(root, token="example") as server, \
            ServiceClient(server.url, token="example") as service:
        training = service.create_training_client(
            Model("shadowspill/regression", dtype="float32"), Optimizer(lr=2e-2, parameter_rounding="nearest"),
            objective=Objective("shadowspill/weighted_squared_error@1"),
            batch=BatchConfig(tokens_per_step=a.samples, microbatch_tokens=a.samples),
            memory=Memory(device_gib=0.53, spill_gib=0.05),
            resources=Resources(gpus=a.ranks, backend="cpu"),
            parallelism=data_parallel(a.ranks) if a.ranks > 1 else None,
            preparation=Preparation(profiling=ProfilingOptions(enabled=False), calibrate=False,
                                    planning=PlanningOptions(minimum_object_bytes_evict_eligible=64,
                                                             workers=1)),
            timeout=600).result()
        for update in range(a.steps):
            result = training.step(rows(update, a.ranks, a.samples)).result()
            losses.append(result.loss)
            print(f"update {update + 1}: loss {result.loss:.5f}")
        training.close()
    return losses


if __name__ == "__main__":
    main()
