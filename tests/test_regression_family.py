"""The non-text ``regression`` family through capture, planning, the runtime and the service."""
import numpy as np
import pytest
import torch

from shadowspill_b200.communication.info import CommunicationInfo
from shadowspill_b200.data.synthetic import HostMicrobatch
from shadowspill_b200.execution.executor import Executor, Hyperparameters
from shadowspill_b200.frontend.capture import BatchGeometry, StepDataOrdering, build_step
from shadowspill_b200.models.config import preset
from shadowspill_b200.models.regression import reference_module
from shadowspill_b200.planning.plan import MemoryBudgets, SearchOptions, plan_program

ROWS, MBS = 8, 2


def _rows(seed, n=ROWS * MBS):
    rng = np.random.Generator(np.random.PCG64(seed))
    return (rng.standard_normal((n, 16), np.float32), rng.standard_normal((n, 8), np.float32),
            np.full(n, 1.0 / (n * 8), np.float32))


def _microbatches(seed, valid=ROWS):
    """``valid`` real rows per microbatch, the rest padding of weight zero."""
    values, targets, weights = _rows(seed)
    out = []
    for m in range(MBS):
        sl = slice(m * ROWS, (m + 1) * ROWS)
        w = weights[sl].copy()
        w[valid:] = 0.0
        cu = np.minimum(np.arange(ROWS + 2), ROWS).astype(np.int32)
        out.append(HostMicrobatch(np.zeros(ROWS, np.int64), np.zeros(ROWS, np.int64), w,
                                  np.zeros(ROWS, np.int32), cu, 1,
                                  {"value": values[sl], "target_values": targets[sl]}))
    return out


@pytest.mark.parametrize("device", ["cpu", pytest.param("cuda", marks=pytest.mark.gpu)])
def test_planned_regression_matches_torch_autograd_and_adamw(device):
    cfg = preset("regression")
    assert cfg.parameter_count() == 16 * 32 + 32 + 32 * 8 + 8
    geo = BatchGeometry(ROWS, MBS, slots=ROWS + 1, mean_seqlen=1)
    prog, desc = build_step(cfg, geo, StepDataOrdering(), dtype=torch.float32)
    assert desc.geometry.extra_fields == ("value:16", "target_values:8")
    total = sum(o.bytes for o in prog.objects)
    ws = max(t.workspace_bytes for t in prog.tasks)
    plan = plan_program(prog, MemoryBudgets(ws + total, 16 << 20, headroom_bytes=0), CommunicationInfo(),
                        SearchOptions(minimum_object_bytes_evict_eligible=64, workers=1))
    hyper = Hyperparameters(lr=1e-2, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.0)
    ex = Executor(plan, desc, device=device, seed=5, hyper=hyper, stochastic_rounding=False)
    ex.initialize(on_device=False)
    state = ex.state_dict()
    ref = reference_module(cfg)
    with torch.no_grad():
        ref[0].weight.copy_(state["input.w1"]); ref[0].bias.copy_(state["input.b1"])
        ref[2].weight.copy_(state["head.w2"]); ref[2].bias.copy_(state["head.b2"])
    opt = torch.optim.AdamW(ref.parameters(), lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.0)
    for step in range(5):
        valid = ROWS if step % 2 == 0 else ROWS - 3
        mbs = _microbatches(step, valid)
        got = ex.run(mbs).loss
        opt.zero_grad()
        want = 0.0
        for mb in mbs:
            pred = ref(torch.from_numpy(mb.extras["value"]))
            w = torch.from_numpy(mb.weights)
            loss = ((pred - torch.from_numpy(mb.extras["target_values"])).square().sum(1) * w).sum()
            loss.backward()
            want += float(loss.detach())
        opt.step()
        assert got == pytest.approx(want, rel=2e-5), step
    mine = ex.state_dict()
    for name, t in (("input.w1", ref[0].weight), ("input.b1", ref[0].bias),
                    ("head.w2", ref[2].weight), ("head.b2", ref[2].bias)):
        assert torch.allclose(mine[name], t.detach(), rtol=1e-4, atol=1e-6), name
    ex.close()


def test_regression_through_the_service(tmp_path):
    """Rows as client datums -> packing -> wire -> server-side validation -> worker."""
    from shadowspill_b200.client import (BatchConfig, BatchError, Memory, Model, Objective, Optimizer,
                                         Preparation, ProfilingOptions, Resources, ServiceClient,
                                         tensor_datum)
    from shadowspill_b200.client.config import PlanningOptions
    from shadowspill_b200.server.service import Server

    def batch(seed):
        values, targets, weights = _rows(seed)
        return [tensor_datum({"value": v, "target_values": t}, w) for v, t, w in zip(values, targets, weights)]
    with Server(tmp_path, token="secret") as srv, ServiceClient(srv.url, token="secret") as svc:
        kinds = {c["id"] for c in svc.list_components().result()} if hasattr(svc, "list_components") else set()
        assert not kinds or "shadowspill/regression@1" in kinds
        trainer = svc.create_training_client(
            Model("shadowspill/regression", dtype="float32"),
            Optimizer(lr=1e-2, parameter_rounding="nearest"),
            objective=Objective("shadowspill/weighted_squared_error@1"),
            batch=BatchConfig(tokens_per_step=ROWS * MBS, microbatch_tokens=ROWS),
            memory=Memory(device_gib=0.53, spill_gib=0.05), resources=Resources(gpus=1, backend="cpu"),
            preparation=Preparation(profiling=ProfilingOptions(enabled=False), calibrate=False,
                                    planning=PlanningOptions(minimum_object_bytes_evict_eligible=64, workers=1)),
            operations=("step", "forward"), timeout=300).result()
        losses = [trainer.step(batch(0)).result().loss for _ in range(12)]
        assert losses[-1] < 0.8 * losses[0]
        pred = trainer.forward(batch(0)).result().outputs["per_datum"]
        assert len(pred) == ROWS * MBS and pred[0].shape == (1, 8)
        targets = _rows(0)[1]
        err = float(np.mean([(p[0] - t) ** 2 for p, t in zip(pred, targets)]))
        assert abs(err - trainer.forward(batch(0)).result().loss) < 1e-5       # weights make the sum a mean
        with pytest.raises(BatchError):          # a row without its regression target
            trainer.step([tensor_datum({"value": np.zeros(16)})])
        with pytest.raises(BatchError):          # a row of the wrong width
            trainer.step([tensor_datum({"value": np.zeros(4), "target_values": np.zeros(8)})])
        trainer.close()


@pytest.mark.parametrize("rule", ["sgd", "lion"])
def test_other_update_rules_match_their_textbook_forms(rule):
    """``sgd`` against ``torch.optim.SGD(momentum)``; ``lion`` against the published update."""
    cfg = preset("regression")
    geo = BatchGeometry(ROWS, MBS, slots=ROWS + 1, mean_seqlen=1)
    prog, desc = build_step(cfg, geo, StepDataOrdering(), dtype=torch.float32)
    total = sum(o.bytes for o in prog.objects)
    ws = max(t.workspace_bytes for t in prog.tasks)
    plan = plan_program(prog, MemoryBudgets(ws + total, 16 << 20, headroom_bytes=0), CommunicationInfo(),
                        SearchOptions(minimum_object_bytes_evict_eligible=64, workers=1))
    lr, b1, b2, wd = 2e-2, 0.9, 0.99, 0.01
    ex = Executor(plan, desc, device="cpu", seed=5, stochastic_rounding=False,
                  hyper=Hyperparameters(lr=lr, beta1=b1, beta2=b2, weight_decay=wd, rule=rule))
    ex.initialize()
    state = ex.state_dict()
    ref = reference_module(cfg)
    with torch.no_grad():
        ref[0].weight.copy_(state["input.w1"]); ref[0].bias.copy_(state["input.b1"])
        ref[2].weight.copy_(state["head.w2"]); ref[2].bias.copy_(state["head.b2"])
    params = list(ref.parameters())
    opt = torch.optim.SGD(params, lr=lr, momentum=b1) if rule == "sgd" else None
    moment = [torch.zeros_like(p) for p in params]
    for step in range(4):
        mbs = _microbatches(step)
        got = ex.run(mbs).loss
        for p in params:
            p.grad = None
        want = 0.0
        for mb in mbs:
            pred = ref(torch.from_numpy(mb.extras["value"]))
            loss = ((pred - torch.from_numpy(mb.extras["target_values"])).square().sum(1)
                    * torch.from_numpy(mb.weights)).sum()
            loss.backward()
            want += float(loss.detach())
        with torch.no_grad():
            if rule == "sgd":
                for p in params:
                    p.mul_(1 - lr * wd)          # decay on the weights, not folded into the gradient
                opt.step()
            else:
                for p, m in zip(params, moment):
                    u = torch.sign(b1 * m + (1 - b1) * p.grad)
                    p.sub_(lr * (u + wd * p))
                    m.mul_(b2).add_((1 - b2) * p.grad)
        assert got == pytest.approx(want, rel=2e-5), (rule, step)
    mine = ex.state_dict()
    for name, t in (("input.w1", ref[0].weight), ("head.b2", ref[2].bias)):
        assert torch.allclose(mine[name], t.detach(), rtol=2e-4, atol=2e-6), (rule, name)
    ex.close()
