"""Terminal tables of submitted operations: what was sent, when, how it ended, how fast it ran.

``CommandTable.track(operation, future, batch=...)`` adds a row when a call is submitted and
completes it from the future's done-callback; the table only observes, it never submits, waits
or retries. On a terminal the recent rows are repainted in place; on any other stream every
submission and every completion appends one line carrying the call's number, so a log file
stays readable. Clock columns come from this machine; durations and tokens per second use the
service's execution time. A stream that stops accepting writes silences the table (``error``)
without touching the tracked calls.

``LengthStatistics`` / ``BatchStatistics`` summarise the examples of a batch before packing
(``client.text.text_batch_statistics`` computes them from datums).

Reference: packages/client/src/shadowspill_client/display.py:22 (``LengthStatistics``), :97
(``BatchStatistics``), :177 (``CommandTable``).
"""
from __future__ import annotations

import math
import shutil
import statistics
import sys
import threading
import time
from collections import deque
from dataclasses import dataclass, field

COMPUTE_OPERATIONS = ("step", "forward_backward", "optim_step", "forward")
_DASH = "-"


def _count(value, what: str) -> int:
    if isinstance(value, bool) or not isinstance(value, int) or value < 0:
        raise ValueError(f"{what} must be a nonnegative int, got {value!r}")
    return value


@dataclass(frozen=True)
class LengthStatistics:
    count: int
    total: int
    minimum: int
    maximum: int
    average: float
    median: float

    @classmethod
    def from_lengths(cls, lengths) -> "LengthStatistics":
        values = [_count(v, "a sequence length") for v in lengths]
        if not values:
            raise ValueError("length statistics need at least one sequence")
        return cls(len(values), sum(values), min(values), max(values),
                   float(statistics.fmean(values)), float(statistics.median(values)))

    def summary(self) -> str:
        """``"min/max mean/median"`` with thousands separators, e.g. ``"345/3,507 1,126/1,013"``."""
        return f"{self.minimum:,}/{self.maximum:,} {self.average:,.0f}/{self.median:,.0f}"


@dataclass(frozen=True)
class BatchStatistics:
    """Lengths of a batch's examples (their own positions: no packing padding), and optionally
    how many positions of each are trained."""
    lengths: LengthStatistics
    supervised: LengthStatistics | None = None

    @classmethod
    def from_lengths(cls, lengths, *, supervised=None) -> "BatchStatistics":
        lengths = list(lengths)
        total = LengthStatistics.from_lengths(lengths)
        if supervised is None:
            return cls(total)
        supervised = list(supervised)
        trained = LengthStatistics.from_lengths(supervised)
        if len(supervised) != len(lengths) or any(s > n for s, n in zip(supervised, lengths)):
            raise ValueError("supervised lengths must match the sequences one to one and fit inside them")
        return cls(total, trained)


@dataclass
class _Call:
    number: int
    operation: str
    submitted: float                       # time.time()
    batch: BatchStatistics | None
    planned: float | None
    completed: float | None = None
    status: str = "pending"
    loss: float | None = None
    seconds: float | None = None

    def cells(self) -> tuple[str, ...]:
        clock = lambda t: _DASH if t is None else time.strftime("%H:%M:%S", time.localtime(t))
        b, s = self.batch, self.seconds
        return (str(self.number), f"{self.operation}()", clock(self.submitted), clock(self.completed), self.status,
                _DASH if self.loss is None else f"{self.loss:.4f}",
                _DASH if s is None else f"{s:.2f}s",
                _DASH if self.planned is None else f"{self.planned:.2f}s",
                _DASH if (not s or b is None) else f"{b.lengths.total / s:,.0f}",
                _DASH if b is None else f"{b.lengths.total:,}",
                _DASH if b is None else str(b.lengths.count),
                _DASH if b is None else b.lengths.summary(),
                _DASH if (b is None or b.supervised is None) else b.supervised.summary())


@dataclass
class CommandTable:
    """One row per tracked compute call. ``tokens_per_step`` is only used by the older ``add``
    form, which prints a finished result without having seen its submission."""
    tokens_per_step: int = 0
    stream: object = None
    max_rows: int = 20
    error: Exception | None = field(default=None, init=False)

    COLUMNS = (("Call", 4), ("Operation", 18), ("Submitted", 9), ("Completed", 9), ("Status", 7), ("Loss", 8),
               ("Time", 8), ("Planned", 8), ("Tokens/s", 9), ("Tokens", 9), ("Seqs", 5), ("Lengths", 23),
               ("Supervised", 23))

    def __post_init__(self):
        if isinstance(self.max_rows, bool) or not isinstance(self.max_rows, int) or self.max_rows < 1:
            raise ValueError("max_rows must be at least 1")
        self.stream = sys.stdout if self.stream is None else self.stream
        self._tty = bool(getattr(self.stream, "isatty", lambda: False)())
        self._calls: deque[_Call] = deque(maxlen=self.max_rows)
        self._lock = threading.RLock()
        self._issued = 0
        self._painted: list[str] = []
        self._opened = False
        self._plain_rows = 0

    # ------------------------------------------------------------------ tracking
    def track(self, operation: str, future, *, batch: BatchStatistics | None = None,
              planned_seconds: float | None = None):
        """Adds the row of a submitted call and fills it in when ``future`` completes: ``done`` with
        the loss and the service's execution time (tokens per second = the batch's own tokens over
        that time) or ``failed``. Returns ``future``."""
        if operation not in COMPUTE_OPERATIONS:
            raise ValueError(f"the command table follows compute calls only ({', '.join(COMPUTE_OPERATIONS)})")
        if batch is not None and not isinstance(batch, BatchStatistics):
            raise TypeError("batch must be a BatchStatistics")
        if operation == "optim_step" and batch is not None:
            raise ValueError("optim_step takes no batch")
        if planned_seconds is not None:
            planned_seconds = float(planned_seconds)
            if not math.isfinite(planned_seconds) or planned_seconds < 0:
                raise ValueError("planned_seconds must be a finite nonnegative number")
        with self._lock:
            self._issued += 1
            call = _Call(self._issued, operation, time.time(), batch, planned_seconds)
            self._calls.append(call)
            self._show(call)

        def finished(done) -> None:
            with self._lock:
                call.completed = time.time()
                if done.cancelled() or done.exception() is not None:
                    call.status = "failed"
                else:
                    result = done.result()
                    call.status = "done"
                    call.loss = getattr(result, "loss", None)
                    call.seconds = getattr(result, "execution_seconds", None)
                self._show(call)
        future.add_done_callback(finished)
        return future

    def add(self, step: int, result) -> None:
        """Prints one finished result (no submission row): step, loss, updates, time, tokens/s."""
        with self._lock:
            if self.error is not None:
                return
            try:
                if self._plain_rows % 20 == 0:
                    self.stream.write(f"{'step':>8} {'loss':>12} {'updates':>8} {'exec s':>9} {'tokens/s':>12}\n")
                tps = self.tokens_per_step / result.execution_seconds if result.execution_seconds else 0.0
                loss = f"{result.loss:.5f}" if result.loss is not None else _DASH
                self.stream.write(f"{step:>8} {loss:>12} {result.completed_updates:>8} "
                                  f"{result.execution_seconds:>9.3f} {tps:>12,.0f}\n")
                self.stream.flush()
                self._plain_rows += 1
            except (OSError, ValueError) as exc:
                self.error = exc

    # ------------------------------------------------------------------ drawing
    def _line(self, cells) -> str:
        return "  ".join(str(c).rjust(w) for c, (_, w) in zip(cells, self.COLUMNS))

    def _show(self, changed: _Call) -> None:
        if self.error is not None:          # a broken terminal must not reach the call or its callback
            return
        try:
            self._draw(changed)
        except (OSError, ValueError) as exc:
            self.error = exc

    def _draw(self, changed: _Call) -> None:
        heading = self._line([name for name, _ in self.COLUMNS])
        head = [heading, "-" * len(heading)]
        w = self.stream.write
        if not self._opened:
            zone = time.strftime("%Z (%z)", time.localtime(changed.submitted))
            w(f"Client clock: {zone}. Time: service execution. Lengths: min/max mean/median.\n")
        if not self._tty:
            if not self._opened:
                w("\n".join(head) + "\n")
            w(self._line(changed.cells()) + "\n")
        else:
            cols, rows_avail = shutil.get_terminal_size(fallback=(180, 40))
            wrapped = lambda line: max(1, math.ceil(len(line) / max(1, cols)))   # a resized terminal wraps lines
            rows = [self._line(c.cells()) for c in self._calls]
            room = max(1, rows_avail - sum(map(wrapped, head)) - 2)
            while len(rows) > 1 and sum(map(wrapped, rows)) > room:
                rows.pop(0)
            up = sum(map(wrapped, self._painted))
            if up:
                w(f"\x1b[{up}A\r\x1b[J")      # back to the top of the last frame, clear to the end
            self._painted = head + rows
            w("\n".join(self._painted) + "\n")
        self._opened = True
        self.stream.flush()
