"""Start the HTTP service in this process, connect with the NumPy-only client, train a
few steps, checkpoint, and read the run's metrics back.

    python examples/service_quickstart.py             # CPU worker, tiny model
"""
import sys
import tempfile
from pathlib import Path

import numpy as np

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))

from shadowspill_b200.client import (BatchConfig, Memory, Model, Optimizer, Preparation,
                                     ProfilingOptions, Resources, ServiceClient, text_batch)
from shadowspill_b200.client.config import PlanningOptions
from shadowspill_b200.server.service import Server


def sequences(seed, n=8, vocab=512):
    rng = np.random.default_rng(seed)
    return [rng.integers(0, vocab, size=int(rng.integers(16, 60))) for _ in range(n)]


def main() -> list[float]:
    with tempfile.TemporaryDirectory() as root, Server(root, token="secret") as server:
        with ServiceClient(server.url, token="secret") as svc:
            trainer = svc.create_training_client(
                Model("llama3-tiny", dtype="float32"),
                Optimizer(lr=3e-3, parameter_rounding="nearest"),
                batch=BatchConfig(tokens_per_step=512, microbatch_tokens=256),
                memory=Memory(device_gib=0.53, spill_gib=0.25),
                resources=Resources(gpus=1, backend="cpu"),
                preparation=Preparation(profiling=ProfilingOptions(enabled=False), calibrate=False,
                                        planning=PlanningOptions(
                                            minimum_object_bytes_evict_eligible=1024, workers=1)),
                timeout=300).result()
            losses = [trainer.step(text_batch(sequences(i % 2))).result().loss for i in range(4)]
            print("losses:", [round(x, 4) for x in losses])
            print("checkpoint:", trainer.save_checkpoint("quickstart").result().outputs)
            metrics = svc.get_metrics(trainer.run).result()["metrics"]
            print(f"{len(metrics)} metric records; last: {metrics[-1]}")
            trainer.close()
    return losses


if __name__ == "__main__":
    main()
