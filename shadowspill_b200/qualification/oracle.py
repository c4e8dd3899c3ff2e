"""Readable Python oracles for the native simulator and placement.

They restate the same rules with plain data structures and no attention to
speed, and exist only to be compared with the compiled implementations on
fixtures and generated cases (the reference keeps such oracles under
qualification/reference/python/{simulator,admission}).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field

from ..ir.plan import MemorySchedule
from ..ir.program import Program
from ..simulator.api import SimulationConfig

OK, NO_PROGRESS = 0, 3


@dataclass
class OracleResult:
    status: int
    makespan_ns: int
    task_start_ns: list[int]
    task_end_ns: list[int]
    action_start_ns: list[int]
    action_end_ns: list[int]
    peak_bytes: int
    stalled_task: int = -1


def simulate(program: Program, schedule: MemorySchedule, config: SimulationConfig) -> OracleResult:
    tasks, objs, acts = program.tasks, program.objects, schedule.actions
    c = config.communication
    nt, na = len(tasks), len(acts)
    by_trigger: dict[int, list[int]] = {}
    for i, a in enumerate(acts):
        by_trigger.setdefault(a.trigger_task, []).append(i)
    resident, ready, fetching, evicting = set(), set(), set(), set()
    used = peak = now = 0
    t_start, t_end = [-1] * nt, [-1] * nt
    a_start, a_end = [-1] * na, [-1] * na
    lanes = {"fetch": {"q": [], "cur": None, "lat": 0, "left": 0.0},
             "evict": {"q": [], "cur": None, "lat": 0, "left": 0.0}}

    def fire(trigger: int):
        nonlocal used
        for i in by_trigger.get(trigger, []):
            a = acts[i]
            if a.kind == "release":
                a_start[i] = a_end[i] = now
                resident.discard(a.object); ready.discard(a.object)
                used -= objs[a.object].bytes
            else:
                lanes[a.kind]["q"].append(i)

    fire(-1)
    ti, running, run_end = 0, False, 0
    while True:
        f, e = lanes["fetch"], lanes["evict"]
        if f["cur"] is None and f["q"]:
            i = f["q"][0]; o = acts[i].object
            blocked = o in resident            # previous stay still draining
            if not blocked and used + objs[o].bytes <= config.capacity_bytes:
                f["q"].pop(0)
                f.update(cur=i, lat=c.fetch_latency_ns, left=float(objs[o].bytes))
                used += objs[o].bytes; peak = max(peak, used)
                resident.add(o); fetching.add(o); a_start[i] = now
        if e["cur"] is None and e["q"]:
            i = e["q"].pop(0); o = acts[i].object
            e.update(cur=i, lat=c.evict_latency_ns, left=float(objs[o].bytes))
            evicting.add(o); a_start[i] = now
        if not running and ti < nt:
            need, ok, impossible = tasks[ti].workspace_bytes, True, False
            for u in tasks[ti].uses:
                if u.mode == "create":
                    need += objs[u.object].bytes
                elif not (u.object in resident and u.object in ready) or u.object in evicting:
                    ok = False
                    queued = any(acts[i].object == u.object for i in f["q"])
                    if u.object not in fetching and not queued:
                        impossible = True
            if impossible:
                return OracleResult(NO_PROGRESS, now, t_start, t_end, a_start, a_end, peak, ti)
            if ok and used + need <= config.capacity_bytes:
                for u in tasks[ti].uses:
                    if u.mode == "create":
                        resident.add(u.object); ready.add(u.object); used += objs[u.object].bytes
                used += tasks[ti].workspace_bytes; peak = max(peak, used)
                running, run_end = True, now + tasks[ti].duration_ns
                t_start[ti] = now
        moving = lambda L: L["cur"] is not None and L["lat"] == 0 and L["left"] > 0.0
        frate = c.fetch_concurrent_bps if moving(e) else c.fetch_solo_bps
        erate = c.evict_concurrent_bps if moving(f) else c.evict_solo_bps
        cands = []
        if running:
            cands.append(run_end)
        for L, rate in ((f, frate), (e, erate)):
            if L["cur"] is not None:
                cands.append(now + L["lat"] + int(L["left"] / rate * 1e9 + 0.999999))
                if L["lat"] > 0:
                    cands.append(now + L["lat"])
        if not cands:
            if ti >= nt and not f["q"] and not e["q"]:
                break
            return OracleResult(NO_PROGRESS, now, t_start, t_end, a_start, a_end, peak, ti if ti < nt else -1)
        nxt = min(cands)
        dt = nxt - now
        for L, rate in ((f, frate), (e, erate)):
            if L["cur"] is None:
                continue
            d = dt
            if L["lat"] > 0:
                take = min(L["lat"], d); L["lat"] -= take; d -= take
            if d > 0 and L["lat"] == 0:
                L["left"] -= rate * d / 1e9
        now = nxt
        if f["cur"] is not None and f["lat"] == 0 and f["left"] <= 0.5:
            o = acts[f["cur"]].object
            fetching.discard(o); ready.add(o); a_end[f["cur"]] = now; f["cur"] = None
        if e["cur"] is not None and e["lat"] == 0 and e["left"] <= 0.5:
            o = acts[e["cur"]].object
            evicting.discard(o); a_end[e["cur"]] = now; e["cur"] = None
            resident.discard(o); ready.discard(o); used -= objs[o].bytes
        if running and now >= run_end:
            running = False
            t_end[ti] = now
            used -= tasks[ti].workspace_bytes
            fire(ti)
            ti += 1
    return OracleResult(OK, now, t_start, t_end, a_start, a_end, peak)


def check_placement(nbytes, start_ns, end_ns, offsets, alignment: int = 1) -> None:
    """Raises if two leases that overlap in time also overlap in address."""
    n = len(nbytes)
    for i in range(n):
        if offsets[i] % alignment:
            raise AssertionError(f"lease {i} is misaligned")
        for j in range(i):
            if start_ns[i] < end_ns[j] and start_ns[j] < end_ns[i]:
                if offsets[i] < offsets[j] + nbytes[j] and offsets[j] < offsets[i] + nbytes[i]:
                    raise AssertionError(f"leases {i} and {j} collide")
