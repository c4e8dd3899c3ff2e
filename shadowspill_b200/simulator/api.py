"""Python face of the native event simulator (``ss_simulate``)."""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import numpy as np

from .. import native
from ..communication.info import CommunicationInfo
from ..ir.plan import MemorySchedule, Stay
from ..ir.program import Program


@dataclass
class SimulationConfig:
    capacity_bytes: int
    communication: CommunicationInfo
    alignment: int = 512

    def to_native(self) -> native.DeviceConfig:
        c = self.communication
        return native.DeviceConfig(int(self.capacity_bytes), c.fetch_solo_bps,
                                   c.fetch_concurrent_bps, c.evict_solo_bps,
                                   c.evict_concurrent_bps, int(c.fetch_latency_ns),
                                   int(c.evict_latency_ns), int(self.alignment))


@dataclass
class SimulationResult:
    status: int
    stalled_task: int
    makespan_ns: int
    compute_ns: int
    input_wait_ns: int
    capacity_wait_ns: int
    peak_bytes: int
    fetch_bytes: int
    evict_bytes: int
    fetch_busy_ns: int
    evict_busy_ns: int
    task_start_ns: list[int]
    task_end_ns: list[int]
    action_start_ns: list[int]
    action_end_ns: list[int]
    stays: list[Stay]

    @property
    def ok(self) -> bool:
        return self.status == native.OK


def stays_from_native(arr, n: int) -> list[Stay]:
    return [Stay(arr[i].object, arr[i].begin_action, arr[i].begin_task, arr[i].end_action,
                 arr[i].bytes, arr[i].start_ns, arr[i].end_ns, arr[i].offset) for i in range(n)]


def simulate(program: Program, schedule: MemorySchedule, config: SimulationConfig) -> SimulationResult:
    lib = native.core()
    prog, keep = program.to_native()
    cfg = config.to_native()
    acts = schedule.to_native()
    na, nt = len(schedule.actions), len(program.tasks)
    res = native.SimResult()
    ts, te = np.zeros(max(nt, 1), np.int64), np.zeros(max(nt, 1), np.int64)
    as_, ae = np.zeros(max(na, 1), np.int64), np.zeros(max(na, 1), np.int64)
    max_iv = na + sum(len(t.uses) for t in program.tasks) + 1
    ivs = (native.Interval * max_iv)()
    n_iv = native.i32(0)
    rc = lib.ss_simulate(C.byref(prog), C.byref(cfg), acts, na, C.byref(res), native.ptr64(ts),
                         native.ptr64(te), native.ptr64(as_), native.ptr64(ae), ivs, max_iv,
                         C.byref(n_iv))
    native.check(rc, "ss_simulate")
    del keep
    return SimulationResult(res.status, res.stalled_task, res.makespan_ns, res.compute_ns,
                            res.input_wait_ns, res.capacity_wait_ns, res.peak_bytes,
                            res.fetch_bytes, res.evict_bytes, res.fetch_busy_ns, res.evict_busy_ns,
                            ts[:nt].tolist(), te[:nt].tolist(), as_[:na].tolist(),
                            ae[:na].tolist(), stays_from_native(ivs, n_iv.value))


def check_schedule(program: Program, schedule: MemorySchedule) -> tuple[bool, int, int]:
    """``(ok, bad_action, bad_task)`` from the order-only validator."""
    lib = native.core()
    prog, keep = program.to_native()
    ba, bt = native.i32(-1), native.i32(-1)
    rc = lib.ss_check_schedule(C.byref(prog), schedule.to_native(), len(schedule.actions),
                               C.byref(ba), C.byref(bt))
    del keep
    return rc == native.OK, ba.value, bt.value


def place_lifetimes(nbytes, start_ns, end_ns, alignment: int = 512) -> tuple[list[int], int]:
    lib = native.core()
    b, s, e = native.as_i64(nbytes), native.as_i64(start_ns), native.as_i64(end_ns)
    off = np.zeros(max(len(b), 1), np.int64)
    span = native.i64(0)
    native.check(lib.ss_place_lifetimes(len(b), native.ptr64(b), native.ptr64(s), native.ptr64(e),
                                        alignment, native.ptr64(off), C.byref(span)),
                 "ss_place_lifetimes")
    return off[:len(b)].tolist(), span.value


def recover_layout_reuse(nbytes, start_ns, end_ns, offsets) -> tuple[list[int], list[int]]:
    lib = native.core()
    n = len(nbytes)
    b, s, e, o = (native.as_i64(x) for x in (nbytes, start_ns, end_ns, offsets))
    begin = np.zeros(n + 1, np.int32)
    cap = max(16, 8 * n)
    while True:
        idx = np.zeros(cap, np.int32)
        rc = lib.ss_recover_layout_reuse(n, native.ptr64(b), native.ptr64(s), native.ptr64(e),
                                         native.ptr64(o), native.ptr32(begin), native.ptr32(idx), cap)
        if rc == native.OOM:
            cap *= 4
            continue
        native.check(rc, "ss_recover_layout_reuse")
        return begin.tolist(), idx[:begin[n]].tolist()
