"""Reads of a run's metric journal.

The service keeps one record per finished request of a run, of any operation, in completion
order, plus whatever the caller logged with ``log``. Reading needs no live writer: it works on a
run another client drives, after the workers closed, and after a service restart for runs that
were recovered from their journal. Inputs and tensor outputs are never part of it.

``query`` reads one page ``(after, through]``; to walk a fixed snapshot keep the first page's
``through`` and follow ``next_cursor`` until it is ``None``; to poll for later records start
after that ``through``. ``export_jsonl`` writes one snapshot as JSON Lines; ``series`` gives the
values of one name as parallel lists.

Reference: packages/client/src/shadowspill_client/metrics.py:33 (``MetricQueries``).
"""
from __future__ import annotations

import concurrent.futures as cf
import json
import os
from dataclasses import dataclass
from pathlib import Path
from typing import Any

MAX_PAGE = 128


@dataclass(frozen=True)
class MetricPage:
    after: int
    through: int
    records: tuple
    next_cursor: int | None


def _cursor(value, what: str) -> int:
    if isinstance(value, bool) or not isinstance(value, int) or not 0 <= value < 2 ** 63:
        raise ValueError(f"{what} must be a nonnegative int below 2**63")
    return value


class MetricQueries:
    def __init__(self, transport, session: str, run: str, pool: cf.Executor | None = None):
        self.transport, self.session_id, self.run_id = transport, session, run
        self.route = f"/v1/runs/{session}/{run}/metrics"
        self._pool = pool or cf.ThreadPoolExecutor(max_workers=2)

    # ------------------------------------------------------------------ reads
    def _read(self, after: int, through: int | None, limit: int) -> MetricPage:
        q: dict[str, Any] = {"after": after, "limit": limit}
        if through is not None:
            q["through"] = through
        _, data = self.transport.request("GET", self.route, query=q)
        records = tuple(data.get("metrics", ()))
        if len(records) > limit or int(data.get("after", after)) != after or \
                (through is not None and int(data.get("through", through)) != through):
            raise RuntimeError("metric reply differs from the requested page")
        return MetricPage(after, int(data.get("through", after + len(records))), records, data.get("next_cursor"))

    def query(self, *, after: int = 0, through: int | None = None, limit: int = 100) -> cf.Future:
        _cursor(after, "metric cursor")
        if through is not None and _cursor(through, "metric snapshot") < after:
            raise ValueError("metric cursor exceeds its snapshot")
        if isinstance(limit, bool) or not isinstance(limit, int) or not 1 <= limit <= MAX_PAGE:
            raise ValueError(f"metric query limit must be 1..{MAX_PAGE}")
        return self._pool.submit(self._read, after, through, limit)

    def snapshot(self, *, after: int = 0, through: int | None = None, limit: int = 100):
        """Generator over every record of one fixed snapshot (blocking, page by page)."""
        page = self.query(after=after, through=through, limit=limit).result()
        fixed = page.through
        while True:
            yield from page.records
            if page.next_cursor is None:
                return
            page = self.query(after=page.next_cursor, through=fixed, limit=limit).result()

    def series(self, name: str, *, after: int = 0) -> tuple[list[int], list[float]]:
        """``(positions, values)`` of every record that carries ``name`` (a top-level field such
        as ``loss`` or ``execution_seconds``, or a key of the record's ``values``)."""
        xs, ys = [], []
        for rec in self.snapshot(after=after):
            v = rec.get(name)
            if v is None:
                v = (rec.get("values") or {}).get(name)
            if isinstance(v, (int, float)) and not isinstance(v, bool):
                xs.append(int(rec.get("position", len(xs) + 1)))
                ys.append(float(v))
        return xs, ys

    def export_jsonl(self, path, *, after: int = 0, through: int | None = None, limit: int = 100) -> cf.Future:
        """One snapshot as JSON Lines in a NEW file (an existing one is refused); records finished
        after the first page was read are not added; a failure removes the partial file."""
        target = Path(path)

        def work() -> Path:
            fd = os.open(target, os.O_WRONLY | os.O_CREAT | os.O_EXCL, 0o644)
            try:
                with os.fdopen(fd, "w") as out:
                    for rec in self.snapshot(after=after, through=through, limit=limit):
                        out.write(json.dumps(rec, sort_keys=True) + "\n")
            except BaseException:
                target.unlink(missing_ok=True)
                raise
            return target
        return self._pool.submit(work)

    # ------------------------------------------------------------------ caller metrics
    def log(self, values: dict[str, float], *, step: int | None = None, request_id: str | None = None) -> cf.Future:
        """Appends caller-side values (evaluation scores, learning rate, anything numeric)."""
        clean = {}
        for k, v in values.items():
            if not isinstance(k, str) or isinstance(v, bool) or not isinstance(v, (int, float)) or v != v:
                raise ValueError(f"metric {k!r} must be a finite number")
            clean[k] = float(v)
        body = {"values": clean, "step": step, "request_id": request_id}
        return self._pool.submit(lambda: self.transport.request("POST", self.route, body)[1].get("record"))
