"""The native planner and placer against independent, readable Python statements of the same
decisions (qualification/pressurefit_oracle.py), on generated programs."""
import random

from hypothesis import HealthCheck, given, settings
from hypothesis import strategies as st

from shadowspill_b200.communication.info import CommunicationInfo
from shadowspill_b200.ir.program import ObjectSpec, Program, TaskSpec, UseSpec
from shadowspill_b200.planning.plan import SearchOptions, plan_program, MemoryBudgets, PlanningError, reduce_emit
from shadowspill_b200.qualification import pressurefit_oracle as oracle
from shadowspill_b200.simulator.api import place_lifetimes, recover_layout_reuse

MIN_BYTES = 4096
COMM = CommunicationInfo(fetch_solo_bps=40e9, fetch_concurrent_bps=30e9, evict_solo_bps=40e9,
                         evict_concurrent_bps=25e9, fetch_latency_ns=8_000, evict_latency_ns=9_000)


def generated_program(seed: int) -> Program:
    """A random program shaped like a training step: persistent state used several times, transients
    created once and read later, sizes on both sides of the eviction threshold."""
    rng = random.Random(seed)
    n_tasks = rng.randint(8, 60)
    n_objects = rng.randint(3, 24)
    objects, uses = [], [[] for _ in range(n_tasks)]
    for o in range(n_objects):
        size = rng.choice([256, 1024, 3000, 8192, 65536, 200_000, 1_000_000, 3_000_000])
        persistent = rng.random() < 0.5
        objects.append(ObjectSpec(f"o{o}", size, "weight" if persistent else "activation", persistent=persistent,
                                  pinned_resident=rng.random() < 0.05))
        k = rng.randint(1, 4)
        tasks = sorted(rng.sample(range(n_tasks), k))
        for i, t in enumerate(tasks):
            if i == 0 and not persistent:
                mode = "create"
            else:
                mode = rng.choice(["read", "read", "mutate"])
            uses[t].append(UseSpec(o, mode))
    tasks = [TaskSpec(f"t{t}", "forward", duration_ns=rng.choice([0, 20_000, 20_000, 60_000, 150_000, 900_000]),
                      workspace_bytes=rng.choice([0, 4096, 100_000, 1_500_000]), uses=uses[t])
             for t in range(n_tasks)]
    return Program(objects, tasks, {})


def _capacities(program: Program, rng: random.Random) -> list[int]:
    """From roomy to hopeless: most of the range needs cuts and can be met."""
    total = sum(o.bytes for o in program.objects) + max(t.workspace_bytes for t in program.tasks)
    return [total] + [int(total * f) + rng.randint(0, 4096) for f in (0.85, 0.7, 0.55, 0.4, 0.25, 0.1)]


@settings(max_examples=200, deadline=None, suppress_health_check=[HealthCheck.too_slow])
@given(st.integers(0, 10**9))
def test_reduce_and_emit_match_the_python_statement(seed):
    program = generated_program(seed)
    rng = random.Random(seed ^ 0x5EED)
    problem = oracle.Problem.of(program, COMM, MIN_BYTES)
    strategy = rng.choice(["stall", "traffic"])
    rule = rng.choice(["demand", "latest-safe", "packed-fifo", "packed-fit"])
    tight = rng.random() < 0.3
    for capacity in _capacities(program, rng):
        want_cuts = oracle.reduce(problem, capacity, ("stall", "traffic").index(strategy), tight)
        for linear in (False, True):
            got = reduce_emit(program, capacity, COMM,
                              SearchOptions(minimum_object_bytes_evict_eligible=MIN_BYTES, linear_reduce=linear),
                              strategy, rule, tight)
            if want_cuts is None:
                assert got is None, (seed, capacity, linear)
                continue
            assert got is not None, (seed, capacity, linear)
            assert got[0] == want_cuts, (seed, capacity, strategy, tight, linear)
            want_actions = oracle.emit(problem, want_cuts,
                                       ("demand", "latest-safe", "packed-fifo", "packed-fit").index(rule), capacity)
            assert got[1] == want_actions, (seed, capacity, rule, linear)


@settings(max_examples=200, deadline=None)
@given(st.integers(0, 10**9))
def test_placement_and_reuse_match_the_python_statement(seed):
    rng = random.Random(seed)
    n = rng.randint(1, 40)
    align = rng.choice([1, 256, 512])
    nbytes = [rng.choice([0, 1, 3, 8, 64]) * align for _ in range(n)]
    start = [rng.randint(0, 50) for _ in range(n)]
    end = [s + rng.randint(0, 20) for s in start]
    offsets, span = place_lifetimes(nbytes, start, end, align)
    want_offsets, want_span = oracle.place(nbytes, start, end, align)
    assert list(offsets) == want_offsets and span == want_span, seed
    oracle_preds = oracle.reuse_predecessors(nbytes, start, end, want_offsets)
    begin, index = recover_layout_reuse(nbytes, start, end, want_offsets)
    got = [list(index[begin[i]:begin[i + 1]]) for i in range(n)]
    assert got == oracle_preds, seed


def test_whole_search_is_the_same_with_either_reducer_and_honours_the_resident_slice():
    """The indexed and the linear reducer drive the whole search to the same plan; with the resident
    slice, every stay of an object under the eviction threshold has one static home behind the
    main layout and no two homes overlap."""
    for seed in range(40):
        program = generated_program(seed)
        total = sum(o.bytes for o in program.objects) + max(t.workspace_bytes for t in program.tasks)
        budgets = MemoryBudgets(max(total * 2 // 3, 1 << 16), 1 << 30, headroom_bytes=0)
        plans = []
        for linear in (False, True):
            try:
                plans.append(plan_program(program, budgets, COMM,
                                          SearchOptions(minimum_object_bytes_evict_eligible=MIN_BYTES, workers=1,
                                                        deterministic=True, linear_reduce=linear)))
            except PlanningError:
                plans.append(None)
        a, b = plans
        assert (a is None) == (b is None), seed
        if a is None:
            continue
        assert [(x.kind, x.object, x.trigger_task) for x in a.schedule.actions] == \
               [(x.kind, x.object, x.trigger_task) for x in b.schedule.actions], seed
        assert [s.offset for s in a.stays] == [s.offset for s in b.stays], seed
        small = {}
        main_end = 0
        for s in a.stays:
            o = program.objects[s.object]
            if o.bytes < MIN_BYTES and not o.pinned_resident:
                assert small.setdefault(s.object, s.offset) == s.offset, seed   # one home per object
            else:
                main_end = max(main_end, s.offset + s.bytes)
        homes = sorted((off, program.objects[o].bytes) for o, off in small.items())
        for (lo, nb), (nxt, _) in zip(homes, homes[1:]):
            assert lo + nb <= nxt, seed
        assert all(off >= main_end for off, _ in homes), seed


def test_search_trace_is_parsed_into_candidate_trajectories(tmp_path):
    """The trace tool: every candidate the search evaluated appears with its reductions and its
    placement; the planned pressure never exceeds the capacity."""
    import torch
    from shadowspill_b200.frontend.capture import BatchGeometry, StepDataOrdering, build_step
    from shadowspill_b200.models.config import preset
    from shadowspill_b200.planning import trace as tr
    cfg = preset("llama3-tiny")
    program, _ = build_step(cfg, BatchGeometry(256, 2, 16, 64), StepDataOrdering(), dtype=torch.float32)
    plan = None
    for percent in (100, 105, 110, 120):          # the tightest of these that still plans
        budgets = MemoryBudgets(max(tr.uncut_pressure(program)) * percent // 100, 64 << 20, headroom_bytes=0)
        try:
            plan = plan_program(program, budgets, COMM, SearchOptions(trace=True, workers=1,
                                                                      minimum_object_bytes_evict_eligible=1024))
            break
        except PlanningError:
            continue
    assert plan is not None
    got = tr.parse_trace(plan.communication["search_trace"])
    assert len(got) == 8 and {c["strategy"] for c in got} == {"stall", "traffic"}
    assert any(c["placed"] for c in got)
    winner = min((c for c in got if c["placed"]), key=lambda c: c["makespan_ns"])
    assert abs(winner["makespan_ns"] * 1e-9 - plan.summary.duration_seconds) < 1e-9
    assert all(any(e["kind"] == "reduce" for e in c["events"]) for c in got if c["placed"])
    text = tr.explain(got)
    assert "gaps cut" in text and "fits" in text
    uncut, planned = tr.uncut_pressure(program), tr.planned_pressure(plan)
    assert budgets.capacity >= max(planned) and plan.summary.fetch_bytes > 0 and len(uncut) == len(planned)
    svg = tr.pressure_svg(uncut, planned, budgets.capacity)
    assert svg.startswith("<svg") and "capacity" in svg
