"""Learning-rate schedules evaluated on the client (reference: shadowspill_client/schedules.py:10,29)."""
from __future__ import annotations

import math
from dataclasses import dataclass


@dataclass(frozen=True)
class Constant:
    value: float

    def __call__(self, step: int) -> float:
        return self.value


@dataclass(frozen=True)
class WarmupCosine:
    peak: float
    warmup_steps: int
    total_steps: int
    floor: float = 0.0

    def __call__(self, step: int) -> float:
        if self.warmup_steps > 0 and step < self.warmup_steps:
            return self.peak * (step + 1) / self.warmup_steps
        span = max(1, self.total_steps - self.warmup_steps)
        frac = min(1.0, max(0.0, (step - self.warmup_steps) / span))
        return self.floor + 0.5 * (self.peak - self.floor) * (1 + math.cos(math.pi * frac))
