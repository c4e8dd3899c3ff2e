"""Terminal table of submitted operations with throughput (reference: shadowspill_client/display.py:177-240)."""
from __future__ import annotations

import sys
import time


class CommandTable:
    def __init__(self, tokens_per_step: int, stream=None):
        self.tokens, self.stream = tokens_per_step, stream or sys.stdout
        self.t0 = time.monotonic()
        self.rows = 0

    def add(self, step: int, result) -> None:
        if self.rows % 20 == 0:
            self.stream.write(f"{'step':>8} {'loss':>12} {'updates':>8} {'exec s':>9} {'tokens/s':>12}\n")
        tps = self.tokens / result.execution_seconds if result.execution_seconds else 0.0
        loss = f"{result.loss:.5f}" if result.loss is not None else "-"
        self.stream.write(f"{step:>8} {loss:>12} {result.completed_updates:>8} "
                          f"{result.execution_seconds:>9.3f} {tps:>12,.0f}\n")
        self.stream.flush()
        self.rows += 1
