"""Planned execution on a B200 (native runtime + CUDA backend + sm_100a kernels)."""
import pytest
import torch

from shadowspill_b200.communication.info import CommunicationInfo
from shadowspill_b200.data.synthetic import make_batch, to_device
from shadowspill_b200.execution.executor import Executor, Hyperparameters
from shadowspill_b200.execution.resident import ResidentTrainer
from shadowspill_b200.frontend.capture import BatchGeometry, StepDataOrdering, build_step
from shadowspill_b200.models.config import DecoderConfig
from shadowspill_b200.ops import _lib
from shadowspill_b200.planning.plan import MemoryBudgets, PlanningError, SearchOptions, plan_program

pytestmark = pytest.mark.gpu


def _plan(cfg, geo, selection=None):
    prog, desc = build_step(cfg, geo, StepDataOrdering(), selection=selection)
    total = sum(o.bytes for o in prog.objects)
    ws = max(t.workspace_bytes for t in prog.tasks)
    for pct in range(25, 101, 5):
        try:
            return plan_program(prog, MemoryBudgets(2 * ws + total * pct // 100, 1 << 30,
                                                    headroom_bytes=0), CommunicationInfo(),
                                SearchOptions(minimum_object_bytes_evict_eligible=4096)), desc
        except PlanningError:
            continue
    raise AssertionError("no plan")


@pytest.mark.parametrize("selection", [None, {1: "save", 2: "save_attention"}])
def test_planned_step_matches_resident(selection):
    cfg = DecoderConfig("llama3", 3, 512, 4, 2, 128, 1024, 4096)
    geo = BatchGeometry(1024, 3, slots=32, mean_seqlen=200)
    plan, desc = _plan(cfg, geo, selection)
    assert plan.summary.fetch_bytes > 0 and plan.summary.evict_bytes > 0
    ex = Executor(plan, desc, device="cuda", seed=3, hyper=Hyperparameters(lr=1e-3),
                  stochastic_rounding=False)
    ex.initialize(on_device=False)
    ref = ResidentTrainer(cfg, device="cuda", seed=3, lr=1e-3, stochastic_rounding=False)
    for step in range(3):
        host = make_batch(step, vocab=cfg.vocab_size, tokens_per_step=3072, microbatch_tokens=1024,
                          median=200, min_len=16, max_len=512, slots=32)
        got = ex.run(host, time_tasks=(step == 2))
        want = ref.step([to_device(m, "cuda") for m in host])
        assert abs(got.loss - want) < 2e-3 * abs(want), (step, got.loss, want)
    _lib.check_status()
    mine = ex.state_dict()
    for k, v in ref.state_dict().items():
        # same kernels, but bf16 gradients accumulate over microbatches in a different order
        # (reverse-breadth walk) and embedding gradients use atomics: a few bf16 ulps apart
        # (Adam turns a sign flip of a near-zero gradient into a 2*lr difference, so the
        # comparison is the relative L2 / cosine one of a numerical gate, not elementwise)
        a, b = mine[k].float().cpu().reshape(-1), v.float().cpu().reshape(-1)
        rel = float((a - b).norm() / (b.norm() + 1e-12))
        cos = float(torch.dot(a, b) / (a.norm() * b.norm() + 1e-12))
        assert rel < 2.5e-2 and cos > 0.999, (k, rel, cos)
    assert len(got.task_seconds) == len(plan.program.tasks)
    stats = ex.rt.stats()
    assert stats["fetch_bytes"] > 0 and stats["evict_bytes"] > 0
    ex.close()


def test_forward_program_returns_target_logprobs():
    """A forward-only plan on the device: the per-position log-probabilities it returns add up
    (with the batch weights) to the loss it reports, and positions without a target read 0."""
    from shadowspill_b200.frontend.capture import build_forward
    cfg = DecoderConfig("llama3", 2, 512, 4, 2, 128, 1024, 4096)
    geo = BatchGeometry(1024, 2, slots=32, mean_seqlen=200)
    prog, desc = build_forward(cfg, geo, StepDataOrdering())
    total = sum(o.bytes for o in prog.objects)
    ws = max(t.workspace_bytes for t in prog.tasks)
    plan = plan_program(prog, MemoryBudgets(2 * ws + total, 1 << 30, headroom_bytes=0), CommunicationInfo(),
                        SearchOptions(minimum_object_bytes_evict_eligible=4096))
    ex = Executor(plan, desc, device="cuda", seed=3, stochastic_rounding=False)
    ex.initialize(on_device=False)
    host = make_batch(0, vocab=cfg.vocab_size, tokens_per_step=2048, microbatch_tokens=1024,
                      median=200, min_len=16, max_len=512, slots=32)
    res = ex.run(host)
    _lib.check_status()
    assert len(res.outputs) == 2 and res.outputs[0].shape == (1024, 1)
    rebuilt = sum(float(-(o[:, 0] * m.weights)[m.targets >= 0].sum()) for o, m in zip(res.outputs, host))
    assert abs(rebuilt - res.loss) < 2e-3 * abs(res.loss)
    for o, m in zip(res.outputs, host):
        assert (o[:, 0][m.targets < 0] == 0).all() and (o <= 0).all()
    ex.close()


@pytest.mark.parametrize("rule,master", [("adamw", True), ("lion", False), ("sgd", True)])
def test_unfused_update_paths_on_the_device(rule, master):
    """fp32 master copies and the update rules beyond AdamW run as tensor operations on the
    planned device ranges: the loss falls, masters round exactly into the weights."""
    cfg = DecoderConfig("llama3", 2, 512, 4, 2, 128, 1024, 4096)
    geo = BatchGeometry(1024, 2, slots=32, mean_seqlen=200)
    prog, desc = build_step(cfg, geo, StepDataOrdering(), master_weights=master)
    total = sum(o.bytes for o in prog.objects)
    ws = max(t.workspace_bytes for t in prog.tasks)
    plan = plan_program(prog, MemoryBudgets(2 * ws + total, 1 << 30, headroom_bytes=0), CommunicationInfo(),
                        SearchOptions(minimum_object_bytes_evict_eligible=4096))
    lr = {"adamw": 1e-3, "lion": 1e-4, "sgd": 3e-2}[rule]
    ex = Executor(plan, desc, device="cuda", seed=3, stochastic_rounding=False,
                  hyper=Hyperparameters(lr=lr, beta2=0.99 if rule == "lion" else 0.95, rule=rule))
    ex.initialize(on_device=False)
    host = make_batch(0, vocab=cfg.vocab_size, tokens_per_step=2048, microbatch_tokens=1024,
                      median=200, min_len=16, max_len=512, slots=32)
    losses = [ex.run(host).loss for _ in range(4)]
    _lib.check_status()
    assert all(l == l for l in losses) and losses[-1] < losses[0], losses
    state = ex.state_dict()
    if master:
        for k, v in state.items():
            if k.startswith("master."):
                assert v.dtype == torch.float32 and torch.equal(v.to(torch.bfloat16), state[k[7:]]), k
    ex.close()
