"""Native core against readable oracles, properties, and host-side fault injection."""
import ctypes as C
import random

import pytest
import torch
from hypothesis import HealthCheck, given, settings
from hypothesis import strategies as st

from shadowspill_b200 import native
from shadowspill_b200.communication.info import CommunicationInfo
from shadowspill_b200.ir.plan import MemoryAction, MemorySchedule
from shadowspill_b200.ir.program import ObjectSpec, Program, TaskSpec, UseSpec
from shadowspill_b200.planning.plan import MemoryBudgets, PlanningError, SearchOptions, plan_program
from shadowspill_b200.qualification import oracle
from shadowspill_b200.simulator.api import (SimulationConfig, check_schedule, place_lifetimes,
                                             recover_layout_reuse, simulate)

COMM = CommunicationInfo(fetch_solo_bps=40e9, fetch_concurrent_bps=25e9, evict_solo_bps=35e9,
                         evict_concurrent_bps=20e9, fetch_latency_ns=5000, evict_latency_ns=7000)


def _chain_program(rng: random.Random, layers: int, mbs: int) -> Program:
    """Forward then backward over `layers` stages with weights, activations and gradients."""
    p = Program()
    W = [p.add_object(ObjectSpec(f"w{i}", rng.randrange(1, 9) << 20, "weight", True)) for i in range(layers)]
    A = [[p.add_object(ObjectSpec(f"a{i}.{m}", rng.randrange(1, 5) << 20, "activation"))
          for m in range(mbs)] for i in range(layers)]
    G = [p.add_object(ObjectSpec(f"g{i}", p.objects[W[i]].bytes, "gradient")) for i in range(layers)]
    for i in range(layers):
        for m in range(mbs):
            uses = [UseSpec(W[i], "read"), UseSpec(A[i][m], "create")]
            if i:
                uses.append(UseSpec(A[i - 1][m], "read"))
            p.add_task(TaskSpec(f"F{i}.{m}", "forward", i, m, uses, rng.randrange(50, 400) * 1000,
                                rng.randrange(0, 3) << 20))
    for i in reversed(range(layers)):
        for m in range(mbs):
            uses = [UseSpec(W[i], "read"), UseSpec(A[i][m], "read"),
                    UseSpec(G[i], "create" if m == 0 else "mutate")]
            p.add_task(TaskSpec(f"B{i}.{m}", "backward", i, m, uses, rng.randrange(100, 800) * 1000,
                                rng.randrange(0, 3) << 20))
        p.add_task(TaskSpec(f"O{i}", "optimizer", i, -1,
                            [UseSpec(W[i], "mutate"), UseSpec(G[i], "read")], 60_000, 0))
    p.validate()
    return p


def _plan(prog: Program, frac: float, **opts):
    total = sum(o.bytes for o in prog.objects)
    ws = max(t.workspace_bytes for t in prog.tasks)
    for bump in range(12):
        try:
            return plan_program(prog, MemoryBudgets(int(ws * 2 + total * (frac + 0.08 * bump)), 1 << 34,
                                                    headroom_bytes=0), COMM,
                                SearchOptions(workers=2, minimum_object_bytes_evict_eligible=1 << 16, **opts))
        except PlanningError:
            continue
    raise AssertionError("never feasible")


def test_abi_struct_sizes_match():
    native.abi_check()
    assert native.core().ss_abi_version() == 1
    assert native.status_string(native.NO_PROGRESS) == "no progress"


@settings(max_examples=25, deadline=None, suppress_health_check=[HealthCheck.too_slow])
@given(seed=st.integers(0, 10_000), layers=st.integers(2, 6), mbs=st.integers(1, 3),
       frac=st.floats(0.25, 0.9))
def test_simulator_matches_python_oracle(seed, layers, mbs, frac):
    prog = _chain_program(random.Random(seed), layers, mbs)
    plan = _plan(prog, frac)
    cfg = SimulationConfig(plan.summary.logical_capacity_bytes, COMM)
    got = simulate(prog, plan.schedule, cfg)
    want = oracle.simulate(prog, plan.schedule, cfg)
    assert got.status == want.status == 0
    assert got.makespan_ns == want.makespan_ns
    assert got.task_start_ns == want.task_start_ns and got.task_end_ns == want.task_end_ns
    assert got.action_end_ns == want.action_end_ns
    assert got.peak_bytes == want.peak_bytes <= cfg.capacity_bytes
    ok, bad_a, bad_t = check_schedule(prog, plan.schedule)
    assert ok, (bad_a, bad_t)
    # the planner's own replay is the same replay
    assert plan.task_end_ns == got.task_end_ns


@settings(max_examples=25, deadline=None)
@given(seed=st.integers(0, 10_000), n=st.integers(1, 60))
def test_placement_never_collides_and_reuse_is_causal(seed, n):
    rng = random.Random(seed)
    nbytes = [rng.randrange(1, 64) * 512 for _ in range(n)]
    start = [rng.randrange(0, 1000) for _ in range(n)]
    end = [s + rng.randrange(1, 300) for s in start]
    off, span = place_lifetimes(nbytes, start, end, 512)
    oracle.check_placement(nbytes, start, end, off, 512)
    assert span == max(o + b for o, b in zip(off, nbytes))
    begin, idx = recover_layout_reuse(nbytes, start, end, off)
    for i in range(n):
        for p in idx[begin[i]:begin[i + 1]]:
            assert end[p] <= start[i]                                     # causal
            assert off[p] < off[i] + nbytes[i] and off[i] < off[p] + nbytes[p]   # really shared


def test_schedule_checker_rejects_broken_schedules():
    prog = _chain_program(random.Random(1), 3, 2)
    plan = _plan(prog, 0.5)
    acts = list(plan.schedule.actions)
    first_fetch = next(i for i, a in enumerate(acts) if a.kind == "fetch")
    broken = MemorySchedule(acts[:first_fetch] + acts[first_fetch + 1:])
    ok, _, bad_task = check_schedule(prog, broken)
    assert not ok and bad_task >= 0
    late = MemorySchedule([MemoryAction(a.kind, a.object, len(prog.tasks) - 1) if i == first_fetch else a
                           for i, a in enumerate(acts)])
    res = simulate(prog, late, SimulationConfig(plan.summary.logical_capacity_bytes, COMM))
    assert res.status == native.NO_PROGRESS and res.stalled_task >= 0


def test_infeasible_budget_is_reported_not_crashed():
    prog = _chain_program(random.Random(2), 3, 2)
    with pytest.raises(PlanningError) as e:
        plan_program(prog, MemoryBudgets(1 << 20, 1 << 34, headroom_bytes=0), COMM)
    assert "no schedule fits" in str(e.value)


def test_tighter_budget_moves_more_bytes():
    prog = _chain_program(random.Random(3), 6, 3)
    loose, tight = _plan(prog, 0.9), _plan(prog, 0.3)
    assert tight.summary.fetch_bytes >= loose.summary.fetch_bytes
    assert tight.device_bytes <= loose.device_bytes
    assert tight.summary.duration_seconds >= loose.summary.compute_seconds
