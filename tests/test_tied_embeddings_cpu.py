"""Tied input/output embeddings: one matrix, two gradient contributions."""
from dataclasses import replace

import torch

from shadowspill_b200.communication.info import CommunicationInfo
from shadowspill_b200.data.synthetic import make_batch, to_device
from shadowspill_b200.execution.executor import Executor, Hyperparameters
from shadowspill_b200.execution.resident import ResidentTrainer
from shadowspill_b200.frontend.capture import BatchGeometry, StepDataOrdering, build_forward, build_step
from shadowspill_b200.models import torch_reference as ref
from shadowspill_b200.models.config import preset
from shadowspill_b200.planning.plan import MemoryBudgets, SearchOptions, plan_program


def _cfg():
    return replace(preset("llama3-tiny"), tied_embeddings=True)


def _batch(cfg, seed, n=2):
    return make_batch(seed, vocab=cfg.vocab_size, tokens_per_step=256 * n, microbatch_tokens=256,
                      median=60, min_len=8, max_len=128, slots=16)


def test_catalog_has_the_tied_preset():
    c = preset("qwen35-2b")
    assert c.tied_embeddings and c.parameter_count() == 1_881_825_088


def test_tied_gradient_is_the_sum_of_both_uses():
    cfg = _cfg()
    tr = ResidentTrainer(cfg, device="cpu", dtype=torch.float32, seed=2)
    assert "head" not in tr.P[-1]
    host = _batch(cfg, 0)
    for mb in host:
        tr.forward_backward(to_device(mb, "cpu"))
    leaves = {f"{st.name}.{n}": t.clone().requires_grad_(True)
              for st, P in zip(tr.stages, tr.P) for n, t in P.items()}
    loss = sum(ref.model_loss(cfg, leaves, to_device(mb, "cpu")) for mb in host)
    loss.backward()
    assert abs(float(loss) - float(tr.loss_sum)) < 1e-4 * abs(float(loss))
    assert torch.allclose(tr.G[0]["embed"], leaves["embed.embed"].grad, rtol=2e-3, atol=2e-5)
    assert torch.allclose(tr.G[-1]["final_norm"], leaves["head.final_norm"].grad, rtol=2e-3, atol=2e-5)


def test_tied_planned_execution_matches_resident():
    cfg = _cfg()
    geo = BatchGeometry(microbatch_tokens=256, n_microbatches=2, slots=16, mean_seqlen=64)
    prog, desc = build_step(cfg, geo, StepDataOrdering(), dtype=torch.float32)
    head_tasks = [t for t in prog.tasks if t.kind == "head"]
    assert all(any(u.role == "tied_params" for u in t.uses) for t in head_tasks)
    fwd_prog, fwd_desc = build_forward(cfg, geo, StepDataOrdering(), dtype=torch.float32)
    total = sum(o.bytes for o in prog.objects) + max(t.workspace_bytes for t in prog.tasks)
    opts = SearchOptions(minimum_object_bytes_evict_eligible=1024, workers=1)
    budgets = MemoryBudgets(total, 64 << 20, headroom_bytes=0)
    from shadowspill_b200.planning.plan import StateLayout
    layout = StateLayout.build([prog, fwd_prog])
    plan = plan_program(prog, budgets, CommunicationInfo(), opts, layout)
    fwd_plan = plan_program(fwd_prog, budgets, CommunicationInfo(), opts, layout)
    ex = Executor(plan, desc, device="cpu", seed=5, hyper=Hyperparameters(lr=3e-3),
                  extra_plans={"forward": (fwd_plan, fwd_desc)})
    ex.initialize()
    tr = ResidentTrainer(cfg, device="cpu", dtype=torch.float32, seed=5, lr=3e-3)
    for step in range(3):
        host = _batch(cfg, step)
        got = ex.run(host).loss
        want = tr.step([to_device(m, "cpu") for m in host])
        assert abs(got - want) < 1e-5 * max(1.0, abs(want)), (step, got, want)
    host = _batch(cfg, 9)
    assert abs(ex.run(host, operation="forward").loss
               - tr.evaluate([to_device(m, "cpu") for m in host])) < 1e-4
    mine = ex.state_dict()
    for k, v in tr.state_dict().items():
        assert torch.allclose(mine[k], v, rtol=1e-5, atol=1e-6), k
    ex.close()
