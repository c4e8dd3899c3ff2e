"""Readable Python statements of the planner's Reduce and Emit steps and of the placer.

They are written for reading, not speed: plain lists, linear scans, no indexes. The native planner
(``csrc/src/planner.cpp``: a segment tree of boundary pressure and an index of heaps over the gaps)
and placer (``csrc/src/placement.cpp``) must make the same decisions; ``tests/test_planner_oracles.py``
compares them on generated programs.

Reduce   every object starts resident from its first to its last use (a fetched object from the
         lead its fetch needs). While the largest task-boundary pressure exceeds the capacity, cut
         the gap (stretch between two consecutive uses of one object) that covers the leftmost peak
         and ranks best: ``stall`` prefers the gap whose evict + fetch is least exposed, then more
         bytes, then the longer gap; ``traffic`` the longest gap, then more bytes, then less exposed.
Emit     residency segments become release / evict actions at the segment's last use and a fetch per
         segment that does not start with the object's creation; the fetch trigger follows the rule.
Place    largest lease first (earlier start, then input order, break ties); each takes the lowest
         aligned offset free of every time-overlapping lease already placed.
Reuse    a lease that takes bytes another lease held earlier waits for the most recent holder.

Reference: qualification/reference/python/{pressurefit,admission} (independent oracles for the
search and for admission), docs/architecture/pressurefit.md:291-361.
"""
from __future__ import annotations

import bisect
from dataclasses import dataclass

from ..communication.info import CommunicationInfo
from ..ir.program import Program

STALL, TRAFFIC = 0, 1
DEMAND, LATEST_SAFE, PACKED_FIFO, PACKED_FIT = 0, 1, 2, 3
FETCH, EVICT, RELEASE = 0, 1, 2


def _transfer_ns(nbytes: int, bps: float, latency: int) -> int:
    if bps <= 0:
        return int(latency)
    return int(latency) + int(nbytes / bps * 1e9 + 0.5)


@dataclass
class Problem:
    """What Reduce and Emit look at: tasks (durations, workspaces), objects (bytes, flags) and the
    uses of every object in task order."""
    duration: list[int]
    workspace: list[int]
    nbytes: list[int]
    persistent: list[bool]
    pinned: list[bool]
    uses: list[list[tuple[int, str]]]           # per object: (task, mode) ascending by task
    fetch_ns: list[int]
    evict_ns: list[int]
    minimum_bytes: int
    resident_slice: bool = True

    @staticmethod
    def of(program: Program, communication: CommunicationInfo, minimum_bytes: int,
           resident_slice: bool = True) -> "Problem":
        uses: list[list[tuple[int, str]]] = [[] for _ in program.objects]
        for ti, t in enumerate(program.tasks):
            for u in t.uses:
                uses[u.object].append((ti, u.mode))
        c = communication
        fbps = c.fetch_concurrent_bps if c.fetch_concurrent_bps > 0 else c.fetch_solo_bps
        ebps = c.evict_concurrent_bps if c.evict_concurrent_bps > 0 else c.evict_solo_bps
        return Problem([t.duration_ns for t in program.tasks], [t.workspace_bytes for t in program.tasks],
                       [o.bytes for o in program.objects], [o.persistent for o in program.objects],
                       [o.pinned_resident for o in program.objects], uses,
                       [_transfer_ns(o.bytes, fbps, c.fetch_latency_ns) for o in program.objects],
                       [_transfer_ns(o.bytes, ebps, c.evict_latency_ns) for o in program.objects],
                       minimum_bytes, resident_slice)

    # ---- helpers shared by both steps
    @property
    def n_tasks(self) -> int:
        return len(self.duration)

    def starts(self) -> list[int]:
        out = [0]
        for d in self.duration:
            out.append(out[-1] + d)
        return out

    def lead_tasks(self, t: int, ns: int) -> int:
        """Tasks before ``t`` whose durations cover ``ns`` (at least one)."""
        lead = acc = 0
        while t - 1 - lead >= 0 and acc < ns:
            acc += self.duration[t - 1 - lead]
            lead += 1
        return max(lead, 1)

    def tail_tasks(self, t: int, ns: int) -> int:
        """Tasks after ``t`` during which an evict of ``ns`` still holds its bytes."""
        tail = acc = 0
        while t + 1 + tail < self.n_tasks and acc < ns:
            acc += self.duration[t + 1 + tail]
            tail += 1
        return tail

    def cuttable(self, o: int) -> bool:
        return not self.pinned[o] and self.nbytes[o] >= self.minimum_bytes

    def in_slice(self, o: int) -> bool:
        return (self.resident_slice and not self.pinned[o] and bool(self.uses[o])
                and self.nbytes[o] < self.minimum_bytes)


def reduce(p: Problem, capacity: int, strategy: int, tight: bool) -> list[tuple[int, int]] | None:
    """The cut gaps as ``(object, index of the use the gap follows)`` in the order they are cut, or
    ``None`` when the capacity cannot be met."""
    nt = p.n_tasks
    start = p.starts()
    pressure = list(p.workspace)

    def add(lo, hi, b):
        for t in range(max(lo, 0), min(hi, nt - 1) + 1):
            pressure[t] += b
    gaps = []                                    # [object, k, t_prev, t_next, cut]
    for o, us in enumerate(p.uses):
        if not us or p.in_slice(o):
            continue
        first, last = us[0][0], us[-1][0]
        created = us[0][1] == "create"
        add(first if (created or tight) else first - p.lead_tasks(first, p.fetch_ns[o]), last, p.nbytes[o])
        for k in range(len(us) - 1):
            if us[k + 1][0] - us[k][0] > 1 and p.cuttable(o):
                gaps.append([o, k, us[k][0], us[k + 1][0], False])
    cuts = []
    while nt:
        peak = max(range(nt), key=lambda t: (pressure[t], -t))       # leftmost maximum
        if pressure[peak] <= capacity:
            break
        best = None
        for g in gaps:
            o, k, t_prev, t_next, cut = g
            if cut or not (t_prev < peak < t_next):
                continue
            tail = 0 if tight else p.tail_tasks(t_prev, p.evict_ns[o])
            lead = 0 if tight else p.lead_tasks(t_next, p.fetch_ns[o])
            lo, hi = t_prev + 1 + tail, t_next - lead - 1
            if not lo <= peak <= hi:
                continue                         # the cut would not relieve this boundary
            span = start[t_next] - start[t_prev + 1]
            exposed = max(0.0, float(p.evict_ns[o] + p.fetch_ns[o] - span))
            key = ((-exposed, float(p.nbytes[o]), float(span)) if strategy == STALL
                   else (float(span), float(p.nbytes[o]), -exposed))
            if best is None or key > best[0]:
                best = (key, g, lo, hi)
        if best is None:
            return None
        _, g, lo, hi = best
        g[4] = True
        cuts.append((g[0], g[1]))
        add(lo, hi, -p.nbytes[g[0]])
    return cuts


def emit(p: Problem, cuts: list[tuple[int, int]], rule: int, capacity: int) -> list[tuple[int, int, int]]:
    """Actions ``(kind, object, trigger task)`` in issue order."""
    nt = p.n_tasks
    start = p.starts()
    cut = set(cuts)
    pressure = list(p.workspace)

    def add(lo, hi, b):
        for t in range(max(lo, 0), min(hi, nt - 1) + 1):
            pressure[t] += b
    fetches = []                                 # [object, need task, duration, trigger]
    ends = []                                    # (kind, object, trigger)
    for o, us in enumerate(p.uses):
        k, n = 0, len(us)
        while k < n:
            j, dirty = k, False
            created = k == 0 and us[0][1] == "create"
            if created:
                dirty = True
            while True:
                if us[j][1] == "mutate":
                    dirty = True
                if j + 1 < n and (o, j) not in cut:
                    j += 1
                else:
                    break
            seg_first, seg_last = us[k][0], us[j][0]
            if not created:
                fetches.append([o, seg_first, p.fetch_ns[o], -2])
            more = j + 1 < n
            kind = EVICT if (dirty and (more or p.persistent[o])) else RELEASE
            ends.append((kind, o, seg_last))
            tail = p.tail_tasks(seg_last, p.evict_ns[o]) if kind == EVICT else 0
            if not p.in_slice(o):
                add(seg_first, seg_last + tail, p.nbytes[o])
            k = j + 1

    def task_ending_by(when):                    # largest t with end(t) <= when, or -1
        return min(bisect.bisect_right(start, when, 1) - 1 - 1, nt - 1)

    def charged(o):
        return 0 if p.in_slice(o) else p.nbytes[o]
    if rule == DEMAND:
        for f in fetches:
            f[3] = f[1] - 1
    elif rule in (LATEST_SAFE, PACKED_FIT):
        margin = 1.25 if rule == PACKED_FIT else 1.0
        lane_free = None
        for f in sorted(fetches, key=lambda f: -f[1]):           # stable: latest need first
            finish = start[f[1]] if lane_free is None else min(start[f[1]], lane_free)
            begin = finish - int(float(f[2]) * margin)
            lane_free = begin
            trig = -1 if begin <= 0 else task_ending_by(begin)
            f[3] = min(trig, f[1] - 1)
        for f in sorted(fetches, key=lambda f: f[1]):            # capacity clamp, in need order
            trig = f[3]
            for t in range(f[1] - 1, trig, -1):
                if t >= 0 and pressure[t] + charged(f[0]) > capacity:
                    trig = t
                    break
            f[3] = trig
            add(trig + 1, f[1] - 1, charged(f[0]))
    else:                                        # packed-fifo: as early as the estimate allows
        floor = -1
        for f in sorted(fetches, key=lambda f: f[1]):
            trig = f[1] - 1
            max_lead = 4 * p.lead_tasks(f[1], f[2]) + 2
            while trig - 1 >= floor and trig - 1 >= -1 and (f[1] - trig) < max_lead:
                if trig >= 0 and pressure[trig] + charged(f[0]) > capacity:
                    break
                trig -= 1
            f[3] = trig
            floor = max(floor, trig)
            add(trig + 1, f[1] - 1, charged(f[0]))
    # the fetch lane is one queue over the whole step: need order, triggers never decreasing
    lane = sorted(fetches, key=lambda f: (max(f[3], -1), f[1]))  # the order a first assembly gives
    lane = sorted(lane, key=lambda f: f[1])
    run = -1
    keyed = [(trig, 0 if kind == RELEASE else 1, 0, (kind, o, trig)) for kind, o, trig in ends]
    for order, f in enumerate(lane):
        run = max(run, max(f[3], -1))
        keyed.append((run, 2, order, (FETCH, f[0], run)))
    # stable by (trigger, releases before evicts before fetches, lane order)
    out = sorted(enumerate(keyed), key=lambda e: (e[1][0], e[1][1], e[1][2], e[0]))
    return [e[1][3] for e in out]


def place(nbytes: list[int], start: list[int], end: list[int], alignment: int) -> tuple[list[int], int]:
    order = sorted(range(len(nbytes)), key=lambda i: (-nbytes[i], start[i], i))
    offsets = [0] * len(nbytes)
    placed, extent = [], 0
    for i in order:
        busy = sorted((offsets[j], offsets[j] + nbytes[j]) for j in placed
                      if start[j] < end[i] and start[i] < end[j] and nbytes[j] > 0)
        at = 0
        for lo, hi in busy:
            if lo - at >= nbytes[i]:
                break
            if hi > at:
                at = -(-hi // alignment) * alignment
        offsets[i] = at
        extent = max(extent, at + nbytes[i])
        placed.append(i)
    return offsets, extent


def reuse_predecessors(nbytes, start, end, offsets) -> list[list[int]]:
    """Per lease, the leases it must wait for: for every byte it takes, the most recent earlier
    holder of that byte (in order of first appearance)."""
    order = sorted(range(len(nbytes)), key=lambda i: (start[i], end[i], i))
    owner: dict[int, int] = {}                   # byte granule -> most recent holder
    grains = sorted({offsets[i] for i in order} | {offsets[i] + nbytes[i] for i in order})
    preds: list[list[int]] = [[] for _ in nbytes]
    for i in order:
        if nbytes[i] <= 0:
            continue
        lo, hi = offsets[i], offsets[i] + nbytes[i]
        for g in grains[bisect.bisect_left(grains, lo):bisect.bisect_left(grains, hi)]:
            who = owner.get(g)
            if who is not None and who not in preds[i]:
                if end[who] > start[i]:
                    raise AssertionError(f"leases {who} and {i} share bytes while both are live")
                preds[i].append(who)
            owner[g] = i
    return preds
