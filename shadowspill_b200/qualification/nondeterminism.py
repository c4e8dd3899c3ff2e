"""Bitwise divergence probe: does the same run give the same bits twice?

    python -m shadowspill_b200.qualification.nondeterminism --model llama3-tiny --device cpu --updates 4

Two sessions are built from the same settings and seed and fed the same batches. After every
update the losses and every tensor of the state (weights, both moments) are compared bit for bit;
the probe reports the first update at which anything differs, the tensors that differ there, how
many of their elements and by how much, and whether the two runs had made the same plan (a run
that profiles may pick another plan, which changes summation orders legitimately). With
stochastic rounding the rounding bits come from a counter RNG keyed on (seed, update, element), so
they repeat too: a divergence then points at an accumulation whose order is not fixed (atomics,
split-K reductions, a collective that sums in arrival order).

Exit status 0 when the runs agree, 1 when they diverge. ``--record PATH`` writes the JSON record.

Reference: qualification/nondeterminism/ of the reference repository (bitwise divergence probe).
"""
from __future__ import annotations

import argparse
import json
import sys

import torch

from ..data.synthetic import make_batch
from ..planning.plan import SearchOptions
from ..training.session import TrainingSession, TrainingSetup


def _bits(t: torch.Tensor) -> torch.Tensor:
    return t.detach().contiguous().cpu().reshape(-1).view(torch.uint8)


def _plan_key(plan):
    return (plan.program.digest(), tuple((a.kind, a.object, getattr(a, "trigger_task", None))
                                         for a in plan.schedule.actions))


def compare_states(a: dict, b: dict, limit: int = 8) -> list[dict]:
    """Tensors that differ in any bit, largest first."""
    out = []
    for name in sorted(a):
        x, y = a[name], b[name]
        if x.shape != y.shape or x.dtype != y.dtype:
            out.append({"tensor": name, "reason": f"{tuple(x.shape)} {x.dtype} vs {tuple(y.shape)} {y.dtype}"})
            continue
        if torch.equal(_bits(x), _bits(y)):
            continue
        xf, yf = x.detach().float().cpu().reshape(-1), y.detach().float().cpu().reshape(-1)
        differ = (x.detach().cpu().reshape(-1) != y.detach().cpu().reshape(-1))
        out.append({"tensor": name, "elements": int(x.numel()), "differing": int(differ.sum()),
                    "max_abs": float((xf - yf).abs().max()), "first_index": int(differ.nonzero()[0]) if differ.any() else -1})
    out.sort(key=lambda d: -d.get("differing", 1 << 60))
    return out[:limit]


def probe(model: str = "llama3-tiny", device: str = "cpu", updates: int = 4, tokens: int = 512,
          microbatch: int = 256, stochastic_rounding: bool | None = None, frontend: str = "stages",
          profile: bool = False, seed: int = 7, perturb_at: int = 0) -> dict:
    """``perturb_at`` > 0 flips one bit of one weight of the second run after that update: the
    probe's own check that a divergence is found and named."""
    cpu = device == "cpu"
    sr = (not cpu) if stochastic_rounding is None else stochastic_rounding

    def session() -> TrainingSession:
        return TrainingSession(TrainingSetup(
            model=model, device_gib=0.53 if cpu else 8.0, spill_gib=0.25 if cpu else 16.0,
            tokens_per_step=tokens, microbatch_tokens=microbatch, lr=1e-3, seed=seed, device=device,
            dtype="float32" if cpu else "bfloat16", stochastic_rounding=sr, profile=profile and not cpu,
            calibrate=False, frontend=frontend,
            search=SearchOptions(minimum_object_bytes_evict_eligible=1024, workers=1, deterministic=True)))
    first, second = session(), session()
    record = {"model": model, "device": device, "updates": updates, "stochastic_rounding": sr,
              "frontend": frontend, "same_plan": _plan_key(first.plan) == _plan_key(second.plan),
              "diverged_at": None, "losses": [], "tensors": []}
    try:
        start = compare_states(first.executor.state_dict(), second.executor.state_dict())
        if start:
            record.update(diverged_at=0, tensors=start)
            return record
        cfg = first.cfg
        for u in range(1, updates + 1):
            batch = make_batch(u, vocab=cfg.vocab_size, tokens_per_step=tokens, microbatch_tokens=microbatch,
                               median=max(16, microbatch // 4), min_len=8, max_len=microbatch // 2, slots=first.slots)
            la, lb = first.step(batch).loss, second.step(batch).loss
            record["losses"].append([la, lb])
            if perturb_at == u:
                name, t = next(iter(second.executor.named_tensors()))
                flat = t.reshape(-1)
                raw = flat[:1].clone().view(torch.uint8)
                raw[0] ^= 1
                flat[:1].copy_(raw.view(flat.dtype))
            differing = compare_states(first.executor.state_dict(), second.executor.state_dict())
            if la != lb or differing:
                record.update(diverged_at=u, tensors=differing, loss_bits_equal=la == lb)
                return record
        return record
    finally:
        first.close()
        second.close()


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", default="llama3-tiny")
    ap.add_argument("--device", default="cpu", choices=["cpu", "cuda"])
    ap.add_argument("--updates", type=int, default=4)
    ap.add_argument("--tokens", type=int, default=512)
    ap.add_argument("--microbatch", type=int, default=256)
    ap.add_argument("--frontend", default="stages", choices=["stages", "graph"])
    ap.add_argument("--nearest", action="store_true", help="round to nearest instead of stochastically")
    ap.add_argument("--profile", action="store_true", help="let each run profile (and possibly plan differently)")
    ap.add_argument("--record", default="")
    a = ap.parse_args(argv)
    rec = probe(a.model, a.device, a.updates, a.tokens, a.microbatch,
                stochastic_rounding=False if a.nearest else None, frontend=a.frontend, profile=a.profile)
    print(json.dumps(rec))
    if a.record:
        with open(a.record, "w") as f:
            json.dump(rec, f, indent=1)
    return 0 if rec["diverged_at"] is None else 1


if __name__ == "__main__":
    sys.exit(main())
