"""A clipped-policy (PPO-style) update loop through the service, on CPU workers.

    python examples/policy_training.py [--iterations 3]

Each iteration: (1) a ``forward`` call scores the sampled responses under the current
weights, which gives the behaviour policy's per-token log-probabilities; (2) the caller
turns rewards into advantages; (3) a few ``step`` calls optimise the clipped surrogate
against those fixed log-probabilities. Sampling itself is outside the framework: here the
"responses" are random tokens and the reward prefers even token ids.
"""
import argparse
import sys
import tempfile
from pathlib import Path

import numpy as np

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))

from shadowspill_b200.client import (BatchConfig, Memory, Model, Objective, Optimizer, Preparation,
                                     ProfilingOptions, Resources, ServiceClient, policy_datum, text_batch)
from shadowspill_b200.client.config import PlanningOptions
from shadowspill_b200.server.service import Server

PROMPT, RESPONSE, VOCAB = 8, 24, 512


def rollouts(rng, n=8):
    tokens = [rng.integers(0, VOCAB, size=PROMPT + RESPONSE) for _ in range(n)]
    mask = np.r_[np.zeros(PROMPT), np.ones(RESPONSE)]
    rewards = np.array([(t[PROMPT:] % 2 == 0).mean() for t in tokens])
    return tokens, mask, rewards


def main(argv=None) -> list[float]:
    ap = argparse.ArgumentParser()
    ap.add_argument("--iterations", type=int, default=3)
    ap.add_argument("--epochs", type=int, default=2, help="policy steps per batch of rollouts")
    a = ap.parse_args(argv)
    rng = np.random.default_rng(0)
    history = []
    with tempfile.TemporaryDirectory() as root, Server(root, token="example") as server, \
            ServiceClient(server.url, token="example") as service:
        training = service.create_training_client(
            Model("llama3-tiny", dtype="float32"), Optimizer(lr=1e-3, parameter_rounding="nearest"),
            objective=Objective("shadowspill/clipped_policy@1", {"clip_ratio": 0.2}),
            batch=BatchConfig(tokens_per_step=512, microbatch_tokens=256),
            memory=Memory(device_gib=0.53, spill_gib=0.25), resources=Resources(gpus=1, backend="cpu"),
            preparation=Preparation(profiling=ProfilingOptions(enabled=False), calibrate=False,
                                    planning=PlanningOptions(minimum_object_bytes_evict_eligible=1024,
                                                             workers=1)),
            operations=("step", "forward"), timeout=600).result()
        for it in range(a.iterations):
            tokens, mask, rewards = rollouts(rng)
            zeros = np.zeros(PROMPT + RESPONSE)
            # 1. score the responses: out[i] is log p(token i+1 | tokens <= i), 0 where masked
            scored = training.forward(text_batch([policy_datum(t, mask, zeros, zeros) for t in tokens])).result()
            old = []
            for out in scored.outputs["per_datum"]:
                per_token = np.zeros(PROMPT + RESPONSE, np.float32)
                per_token[1:] = out[:-1, 0]          # back from predicting position to predicted token
                old.append(per_token)
            # 2. advantages: reward minus the batch mean, the same for every response token
            advantage = rewards - rewards.mean()
            batch = text_batch([policy_datum(t, mask, o, np.full(PROMPT + RESPONSE, adv))
                                for t, o, adv in zip(tokens, old, advantage)])
            # 3. optimise the clipped surrogate; the first step starts at ratio 1
            losses = [training.step(batch).result().loss for _ in range(a.epochs)]
            history += losses
            print(f"iteration {it}: mean reward {rewards.mean():.3f}, surrogate {losses[0]:+.5f} -> {losses[-1]:+.5f}")
        training.close()
    return history


if __name__ == "__main__":
    main()
