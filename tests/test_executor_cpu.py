"""Planned execution on the mock backend must reproduce the resident trainer."""
import pytest
import torch

from shadowspill_b200.communication.info import CommunicationInfo
from shadowspill_b200.data.synthetic import make_batch, to_device
from shadowspill_b200.execution.executor import Executor, Hyperparameters
from shadowspill_b200.execution.resident import ResidentTrainer
from shadowspill_b200.frontend.capture import BatchGeometry, StepDataOrdering, build_step
from shadowspill_b200.models.config import preset
from shadowspill_b200.planning.plan import (MemoryBudgets, PlanningError, SearchOptions,
                                            plan_program)


def _setup(walk="breadth", selection=None, capacity=None, optimizer="stage_interleaved"):
    cfg = preset("llama3-tiny")
    geo = BatchGeometry(microbatch_tokens=256, n_microbatches=2, slots=16, mean_seqlen=64)
    prog, desc = build_step(cfg, geo, StepDataOrdering(walk=walk, optimizer=optimizer),
                            dtype=torch.float32, selection=selection)
    total = sum(o.bytes for o in prog.objects)
    ws = max(t.workspace_bytes for t in prog.tasks)
    opts = SearchOptions(minimum_object_bytes_evict_eligible=1024, workers=2)
    if capacity is not None:
        return cfg, plan_program(prog, MemoryBudgets(capacity, 64 << 20, headroom_bytes=0),
                                 CommunicationInfo(), opts), desc
    # the smallest budget (in steps of 5 % of all state) that still plans
    for pct in range(30, 101, 5):
        try:
            plan = plan_program(prog, MemoryBudgets(ws + total * pct // 100, 64 << 20,
                                                    headroom_bytes=0), CommunicationInfo(), opts)
            return cfg, plan, desc
        except PlanningError:
            continue
    raise AssertionError("no budget planned")


def _batches(cfg, seed=0):
    return make_batch(seed, vocab=cfg.vocab_size, tokens_per_step=512, microbatch_tokens=256,
                      median=60, min_len=8, max_len=128, slots=16)


def _check_against_resident(walk, selection=None, optimizer="stage_interleaved"):
    cfg, plan, desc = _setup(walk, selection, optimizer=optimizer)
    assert plan.summary.fetch_bytes > 0
    hyper = Hyperparameters(lr=3e-3)
    ex = Executor(plan, desc, device="cpu", seed=5, hyper=hyper)
    ex.initialize()
    ref = ResidentTrainer(cfg, device="cpu", dtype=torch.float32, seed=5, lr=3e-3)
    for step in range(3):
        host = _batches(cfg, step)
        res = ex.run(host)
        want = ref.step([to_device(m, "cpu") for m in host])
        assert abs(res.loss - want) < 1e-5 * max(1.0, abs(want)), (step, res.loss, want)
    got = ex.state_dict()
    for k, v in ref.state_dict().items():
        assert torch.allclose(got[k], v, rtol=1e-5, atol=1e-6), k
    stats = ex.rt.stats()
    assert stats["steps"] == 3 and stats["fetches"] > 0
    ex.close()


def test_breadth_recompute_matches_resident():
    _check_against_resident("breadth")


def test_depth_tail_matches_resident():
    _check_against_resident("depth", optimizer="tail")


def test_saved_variants_match_resident():
    _check_against_resident("breadth", selection={1: "save", 2: "save_attention"})
    _check_against_resident("breadth", selection={1: "save_attention_gu", 2: "save_attention"})


def test_steady_state_creates_no_events():
    cfg, plan, desc = _setup()
    ex = Executor(plan, desc, device="cpu", seed=1)
    ex.initialize()
    ex.run(_batches(cfg))
    before = ex.rt.stats()
    ex.run(_batches(cfg, 1))
    after = ex.rt.stats()
    assert after["events_created"] == before["events_created"]
    assert after["host_allocations"] == before["host_allocations"]
    ex.close()


def test_operations_share_state_across_plans():
    """forward_backward twice + optim_step, then forward, through four plans over one
    spill-resident state, against the resident trainer doing the same calls."""
    from shadowspill_b200.frontend.capture import (build_forward, build_forward_backward,
                                                   build_optimizer)
    from shadowspill_b200.planning.plan import StateLayout
    cfg = preset("llama3-tiny")
    geo = BatchGeometry(microbatch_tokens=256, n_microbatches=2, slots=16, mean_seqlen=64)
    built = {"step": build_step(cfg, geo, dtype=torch.float32),
             "forward_backward": build_forward_backward(cfg, geo, dtype=torch.float32),
             "optim_step": build_optimizer(cfg, geo, dtype=torch.float32),
             "forward": build_forward(cfg, geo, dtype=torch.float32)}
    layout = StateLayout.build([p for p, _ in built.values()])
    budgets = MemoryBudgets(24 << 20, 64 << 20, headroom_bytes=0)
    opts = SearchOptions(minimum_object_bytes_evict_eligible=1024, workers=1)
    plans = {k: (plan_program(p, budgets, CommunicationInfo(), opts, layout), d)
             for k, (p, d) in built.items()}
    hyper = Hyperparameters(lr=3e-3)
    step_plan, step_desc = plans.pop("step")
    ex = Executor(step_plan, step_desc, device="cpu", seed=5, hyper=hyper, extra_plans=plans)
    ex.initialize()
    assert ex.operations() == ["forward", "forward_backward", "optim_step", "step"]
    ref = ResidentTrainer(cfg, device="cpu", dtype=torch.float32, seed=5, lr=3e-3)
    for round_ in range(2):
        for call in range(2):
            host = _batches(cfg, 10 * round_ + call)
            got = ex.run(host, operation="forward_backward").loss
            ref.loss_sum.zero_()
            for m in host:
                ref.forward_backward(to_device(m, "cpu"))
            assert abs(got - float(ref.loss_sum)) < 1e-5 * max(1.0, abs(got))
        ex.run(operation="optim_step")
        ref.optim_step()
        assert ex.completed_updates == round_ + 1 and ex.accumulated == 0
    host = _batches(cfg, 99)
    fwd = ex.run(host, operation="forward")
    assert abs(fwd.loss - ref.evaluate([to_device(m, "cpu") for m in host])) < 1e-5
    # a forward-only program also returns log p(target) of every position, per microbatch
    assert len(fwd.outputs) == len(host) and fwd.outputs[0].shape == (256, 1)
    rebuilt = sum(float(-(o[:, 0] * m.weights)[m.targets >= 0].sum()) for o, m in zip(fwd.outputs, host))
    assert abs(rebuilt - fwd.loss) < 1e-4
    assert all((o[:, 0][m.targets < 0] == 0).all() and (o <= 0).all() for o, m in zip(fwd.outputs, host))
    want = ref.step([to_device(m, "cpu") for m in host])
    stepped = ex.run(host, operation="step")
    assert abs(stepped.loss - want) < 1e-5 * abs(want) and stepped.outputs == []
    got = ex.state_dict()
    for k, v in ref.state_dict().items():
        # microbatches accumulate in another order (reverse walk), hence a few fp32 ulps
        assert torch.allclose(got[k], v, rtol=1e-4, atol=2e-5), (k, float((got[k] - v).abs().max()))
    ex.close()


def test_traced_step_diagnostics_and_runtime_report(tmp_path):
    from shadowspill_b200.diagnostics.step import diagnose_step
    from shadowspill_b200.reporting.runtime import write_runtime_report
    cfg, plan, desc = _setup("breadth")
    ex = Executor(plan, desc, device="cpu", seed=5, hyper=Hyperparameters(lr=1e-3),
                  trace_capacity=1 << 14)
    ex.initialize()
    ex.run(_batches(cfg, 0))
    res = ex.run(_batches(cfg, 1), trace=True, time_tasks=True)
    n_moves = sum(a.kind != "release" for a in plan.schedule.actions)
    assert len(res.task_seconds) == len(plan.program.tasks)
    assert len(res.transfer_begin_ns) == len(plan.schedule.actions)
    diag = diagnose_step(plan, res, runtime_stats=ex.rt.stats())
    assert diag.trace_complete
    assert len(diag.tasks) == len(plan.program.tasks)
    assert len(diag.transfers) == n_moves          # every planned copy was seen issued
    assert all(t.real_s >= 0 for t in diag.transfers)
    assert diag.task_seconds_real > 0 and diag.makespan_s > 0
    total_idle = (diag.input_readiness_wait_seconds + diag.allocation_reuse_wait_seconds
                  + diag.frontend_overhead_seconds)
    assert abs(total_idle - diag.idle_seconds_real) < 1e-9
    assert set(diag.phases) >= {"forward", "backward", "optimizer"}
    page = write_runtime_report(plan, diag, tmp_path)
    text = page.read_text()
    assert "Runtime report" in text and "exposed frontend overhead" in text
    assert (tmp_path / "runtime_tasks.csv").read_text().count("\n") == len(plan.program.tasks) + 1
    assert (tmp_path / "runtime.json").exists() and (tmp_path / "runtime_transfers.csv").exists()
    ex.close()


def test_head_row_chunks_change_workspace_not_results():
    """The output projection evaluated in smaller row blocks: less task workspace, same numbers."""
    cfg = preset("llama3-tiny")
    geo = BatchGeometry(microbatch_tokens=256, n_microbatches=2, slots=16, mean_seqlen=64)
    losses, work = [], []
    for rows in (0, 64):
        prog, desc = build_step(cfg, geo, StepDataOrdering(), dtype=torch.float32, head_block_rows=rows)
        work.append(max(t.workspace_bytes for t in prog.tasks if t.kind == "head"))
        plan = plan_program(prog, MemoryBudgets(32 << 20, 64 << 20, headroom_bytes=0), CommunicationInfo(),
                            SearchOptions(minimum_object_bytes_evict_eligible=1024, workers=1))
        ex = Executor(plan, desc, device="cpu", seed=1)
        ex.initialize()
        losses.append([ex.run(_batches(cfg, s)).loss for s in range(2)])
        ex.close()
    assert work[1] < work[0]
    assert losses[1] == pytest.approx(losses[0], rel=1e-6)


def test_fp32_master_copies_keep_progress_that_bf16_rounding_loses():
    """bf16 weights with round-to-nearest and a small learning rate: for all but the smallest
    weights every single update is below half an ulp and is rounded away. With fp32 master copies
    the same updates accumulate in the master and surface in the weights after a few steps."""
    cfg = preset("llama3-tiny")
    geo = BatchGeometry(microbatch_tokens=256, n_microbatches=2, slots=16, mean_seqlen=64)
    moved = {}
    for master in (False, True):
        prog, desc = build_step(cfg, geo, StepDataOrdering(), dtype=torch.bfloat16, master_weights=master)
        assert any(o.name.endswith(".master") for o in prog.objects) == master
        plan = plan_program(prog, MemoryBudgets(32 << 20, 64 << 20, headroom_bytes=0), CommunicationInfo(),
                            SearchOptions(minimum_object_bytes_evict_eligible=1024, workers=1))
        ex = Executor(plan, desc, device="cpu", seed=1, stochastic_rounding=False,
                      hyper=Hyperparameters(lr=1e-5))
        ex.initialize()
        before = ex.state_dict()
        for s in range(12):
            ex.run(_batches(cfg, s))
        after = ex.state_dict()
        w = "layer0.wqkv"
        moved[master] = float((after[w] != before[w]).float().mean())
        if master:
            m = after["master." + w]
            assert m.dtype == torch.float32 and torch.equal(m.to(torch.bfloat16), after[w])
            assert float((m - after[w].float()).abs().max()) > 0      # the master holds what bf16 cannot
        ex.close()
    assert moved[False] < 0.25 and moved[True] > 0.3 and moved[True] > 2 * moved[False], moved


def test_a_task_that_raises_leaves_a_terminal_runtime_that_still_closes():
    """An exception inside a task ends the step on the native side too: the failure is latched
    with the exception's text, later steps are refused, and close() releases the plan."""
    from shadowspill_b200.runtime.core import RuntimeFailure
    cfg, plan, desc = _setup("breadth")
    ex = Executor(plan, desc, device="cpu", seed=5, hyper=Hyperparameters(lr=1e-3))
    ex.initialize()
    ex.run(_batches(cfg, 0))
    real, calls = ex.runner.run_task, [0]

    def failing(task, bound):
        calls[0] += 1
        if calls[0] == 7:
            raise ValueError("synthetic task failure")
        return real(task, bound)
    ex.runner.run_task = failing
    with pytest.raises(ValueError, match="synthetic task failure"):
        ex.run(_batches(cfg, 1))
    failure = ex.rt.failure()
    assert failure is not None and "synthetic task failure" in failure["message"]
    ex.runner.run_task = real
    with pytest.raises(RuntimeFailure):
        ex.run(_batches(cfg, 2))
    ex.close()                                      # no "plan is active" error


def test_parameter_groups_change_decay_and_learning_rate_per_parameter():
    """No decay on norm vectors and a tenth of the learning rate on the embedding, as groups of the
    planned update: equal to ``torch.optim.AdamW`` with the same three parameter groups on the same
    gradients (first matching group wins; everything else keeps the run's own values)."""
    import torch
    from shadowspill_b200.execution.executor import Hyperparameters
    h = Hyperparameters(lr=1e-2, weight_decay=0.1,
                        groups=((("*norm*",), 1.0, 0.0), (("embed.*",), 0.1, None)))
    assert h.rates("layer0.attn_norm") == (1e-2, 0.0)
    assert h.rates("embed.embed") == (1e-3, 0.1)
    assert h.rates("layer1.w13") == (1e-2, 0.1)
    from shadowspill_b200.frontend.capture import BatchGeometry, StepDataOrdering, build_step
    from shadowspill_b200.models.config import preset
    from shadowspill_b200.communication.info import CommunicationInfo
    from shadowspill_b200.planning.plan import MemoryBudgets, SearchOptions, plan_program
    from shadowspill_b200.execution.executor import Executor
    from shadowspill_b200.data.synthetic import make_batch
    cfg = preset("llama3-tiny")
    geo = BatchGeometry(256, 2, 16, 64)
    prog, desc = build_step(cfg, geo, StepDataOrdering(), dtype=torch.float32)
    total = sum(o.bytes for o in prog.objects) + max(t.workspace_bytes for t in prog.tasks)
    plan = plan_program(prog, MemoryBudgets(total, 64 << 20, headroom_bytes=0), CommunicationInfo(),
                        SearchOptions(minimum_object_bytes_evict_eligible=1024, workers=1))
    runs = {}
    for label, hyper in (("grouped", h), ("plain", Hyperparameters(lr=1e-2, weight_decay=0.1))):
        ex = Executor(plan, desc, device="cpu", seed=5, hyper=hyper)
        ex.initialize()
        start = {k: v.clone() for k, v in ex.state_dict().items()}
        batch = make_batch(0, vocab=cfg.vocab_size, tokens_per_step=512, microbatch_tokens=256, median=60,
                           min_len=8, max_len=128, slots=16)
        ex.run(batch)
        runs[label] = (start, ex.state_dict())
        ex.close()
    (s0, g), (_, p) = runs["grouped"], runs["plain"]
    # one AdamW step from zero moments moves every element by lr * sign(grad) after the decay:
    # |new - old * (1 - lr * wd)| = lr (up to eps)
    def step_size(state, key, lr, wd):
        moved = (state[key] - s0[key] * (1 - lr * wd)).abs()
        return float(moved[moved > 0].median())
    assert abs(step_size(g, "layer0.attn_norm", 1e-2, 0.0) - 1e-2) < 1e-4          # no decay on the norm
    assert abs(step_size(p, "layer0.attn_norm", 1e-2, 0.1) - 1e-2) < 1e-4          # the plain run decays it
    assert not torch.allclose(g["layer0.attn_norm"], p["layer0.attn_norm"])
    assert abs(step_size(g, "embed.embed", 1e-3, 0.1) - 1e-3) < 1e-5                # a tenth of the rate
    assert torch.allclose(g["layer1.w13"], p["layer1.w13"])                         # ungrouped: unchanged


def test_norm_observations_report_the_gradient_and_weight_norms_before_the_update():
    """``Hyperparameters(observe_norms=True)``: the step's result carries the L2 norm of the final
    (accumulated) gradients and of the weights as they were before the update; compared with eager
    PyTorch on the same module and batch. Sharded runs refuse the option."""
    import pytest
    import torch
    from shadowspill_b200.communication.info import CommunicationInfo
    from shadowspill_b200.data.synthetic import make_batch, to_device
    from shadowspill_b200.execution.executor import Executor, Hyperparameters
    from shadowspill_b200.frontend.capture import BatchGeometry, StepDataOrdering, build_step
    from shadowspill_b200.frontend.modules import DecoderLM
    from shadowspill_b200.models.config import preset
    from shadowspill_b200.planning.plan import MemoryBudgets, SearchOptions, plan_program
    cfg = preset("llama3-tiny")
    geo = BatchGeometry(256, 2, 16, 64)
    prog, desc = build_step(cfg, geo, StepDataOrdering(), dtype=torch.float32, frontend="graph")
    total = sum(o.bytes for o in prog.objects) + max(t.workspace_bytes for t in prog.tasks)
    plan = plan_program(prog, MemoryBudgets(total, 64 << 20, headroom_bytes=0), CommunicationInfo(),
                        SearchOptions(minimum_object_bytes_evict_eligible=1024, workers=1))
    ex = Executor(plan, desc, device="cpu", seed=5, hyper=Hyperparameters(lr=1e-3, observe_norms=True))
    ex.initialize()
    model = DecoderLM(cfg, torch.float32)
    state = ex.state_dict()
    rename = lambda k: ("layers." + k[len("layer"):] if k.startswith("layer") else k)
    with torch.no_grad():
        for name, p in model.named_parameters():
            p.copy_(next(v for k, v in state.items() if rename(k) == name))
    batch = make_batch(0, vocab=cfg.vocab_size, tokens_per_step=512, microbatch_tokens=256, median=60, min_len=8,
                       max_len=128, slots=16)
    for mb in batch:
        m = to_device(mb, "cpu")
        model(m.tokens, m.targets, m.weights, m.positions, m.cu_seqlens).sum().backward()
    want_g = float(torch.sqrt(sum(p.grad.float().square().sum() for p in model.parameters())))
    want_p = float(torch.sqrt(sum(p.detach().float().square().sum() for p in model.parameters())))
    first = ex.run(batch).metrics
    assert abs(first["grad_norm"] - want_g) < 1e-4 * want_g and abs(first["param_norm"] - want_p) < 1e-5 * want_p
    second = ex.run(batch).metrics
    assert second["param_norm"] != first["param_norm"] and second["grad_norm"] > 0      # sums start again every step
    ex.close()
    sharded, sdesc = build_step(cfg, geo, StepDataOrdering(), dtype=torch.float32, world_size=2, rank=0)
    splan = plan_program(sharded, MemoryBudgets(total, 64 << 20, headroom_bytes=0), CommunicationInfo(),
                         SearchOptions(minimum_object_bytes_evict_eligible=1024, workers=1))
    with pytest.raises(ValueError, match="single-worker"):
        Executor(splan, sdesc, device="cpu", hyper=Hyperparameters(observe_norms=True), collectives="dist")
