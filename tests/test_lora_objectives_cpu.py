"""Low-rank adapters and the policy objective: stage math against autograd on the
merged weights, planned execution against the resident trainer (CPU, fp32)."""
import numpy as np
import pytest
import torch

from shadowspill_b200.communication.info import CommunicationInfo
from shadowspill_b200.data.synthetic import make_batch, to_device
from shadowspill_b200.execution.executor import Executor, Hyperparameters
from shadowspill_b200.execution.resident import ResidentTrainer
from shadowspill_b200.frontend.capture import BatchGeometry, StepDataOrdering, build_step
from shadowspill_b200.models import torch_reference as ref
from shadowspill_b200.models.config import preset
from shadowspill_b200.models.decoder import build_stages
from shadowspill_b200.models.lora import LoRAConfig
from shadowspill_b200.models.objectives import Objective, router_balance
from shadowspill_b200.ops import functional as F
from shadowspill_b200.ops import reference as opref
from shadowspill_b200.planning.plan import MemoryBudgets, SearchOptions, plan_program


def _batch(cfg, seed=0, n=1, extras=()):
    host = make_batch(seed, vocab=cfg.vocab_size, tokens_per_step=256 * n, microbatch_tokens=256,
                      median=60, min_len=8, max_len=128, slots=16)
    rng = np.random.default_rng(seed)
    for mb in host:
        for name in extras:
            scale = 1.0 if name == "advantages" else 0.1
            shift = 0.0 if name == "advantages" else -6.0
            mb.extras[name] = (rng.standard_normal(256) * scale + shift).astype(np.float32)
    return host


@pytest.mark.parametrize("model", ["llama3-tiny", "olmoe-tiny"])
def test_lora_gradients_match_autograd_on_merged_weights(model):
    cfg = preset(model)
    lora = LoRAConfig(rank=8, alpha=16.0, targets=("wq", "wv", "wo", "w13", "w2"))
    tr = ResidentTrainer(cfg, device="cpu", dtype=torch.float32, seed=3, lora=lora)
    g = torch.Generator().manual_seed(11)
    for P in tr.P:                                   # non-zero B factors, or the adapters are inert
        for name, t in P.items():
            if name.endswith("_lora_b"):
                t.normal_(0.0, 0.05, generator=g)
    meta = to_device(_batch(cfg)[0], "cpu")
    tr.forward_backward(meta)
    # oracle: the plain model on merged weights W + s B A; chain rule back to the factors
    merged, leaves = {}, {}
    for st, P in zip(tr.stages, tr.P):
        for name, t in P.items():
            if "_lora_" in name:
                continue
            w = t.clone()
            a, b = P.get(f"{name}_lora_a"), P.get(f"{name}_lora_b")
            if a is not None:
                w = w + lora.scale * (b @ a)
            leaves[f"{st.name}.{name}"] = w.requires_grad_(True)
    loss = ref.model_loss(cfg, leaves, meta, stages=tr.stages)
    loss.backward()
    assert abs(float(loss) - float(tr.loss_sum)) < 1e-4 * max(1.0, abs(float(loss)))
    checked = 0
    for st, P, G in zip(tr.stages, tr.P, tr.G):
        for name in P:
            if not name.endswith("_lora_a"):
                continue
            base = name[:-len("_lora_a")]
            dW = leaves[f"{st.name}.{base}"].grad
            a, b = P[name], P[f"{base}_lora_b"]
            want_a = lora.scale * (b.transpose(-1, -2) @ dW)
            want_b = lora.scale * (dW @ a.transpose(-1, -2))
            assert torch.allclose(G[name], want_a, rtol=2e-3, atol=2e-5), (st.name, name)
            assert torch.allclose(G[f"{base}_lora_b"], want_b, rtol=2e-3, atol=2e-5), (st.name, base)
            assert base not in G                     # the frozen base has no gradient buffer
            checked += 1
    assert checked >= 2 * cfg.n_layers
    assert "embed" not in tr.G[0] and "head" not in tr.G[-1]


def test_lora_planned_execution_matches_resident_and_shrinks_state():
    cfg = preset("llama3-tiny")
    lora = LoRAConfig(rank=8, alpha=16.0)
    geo = BatchGeometry(microbatch_tokens=256, n_microbatches=2, slots=16, mean_seqlen=64)
    prog, desc = build_step(cfg, geo, StepDataOrdering(), dtype=torch.float32, lora=lora)
    full, _ = build_step(cfg, geo, StepDataOrdering(), dtype=torch.float32)
    state = lambda p: sum(o.bytes for o in p.objects if o.kind in ("gradient", "optimizer_state"))
    assert state(prog) < 0.2 * state(full)
    assert not any(t.name.startswith(("O.embed", "O.head", "B.embed")) for t in prog.tasks)
    total = sum(o.bytes for o in prog.objects) + max(t.workspace_bytes for t in prog.tasks)
    plan = plan_program(prog, MemoryBudgets(total, 64 << 20, headroom_bytes=0), CommunicationInfo(),
                        SearchOptions(minimum_object_bytes_evict_eligible=1024, workers=1))
    ex = Executor(plan, desc, device="cpu", seed=5, hyper=Hyperparameters(lr=1e-2))
    ex.initialize()
    tr = ResidentTrainer(cfg, device="cpu", dtype=torch.float32, seed=5, lr=1e-2, lora=lora)
    for step in range(3):
        host = _batch(cfg, step, n=2)
        got = ex.run(host).loss
        want = tr.step([to_device(m, "cpu") for m in host])
        assert abs(got - want) < 1e-5 * max(1.0, abs(want)), (step, got, want)
    mine = ex.state_dict()
    for k, v in tr.state_dict().items():
        assert torch.allclose(mine[k], v, rtol=1e-5, atol=1e-6), k
    assert not any(k.startswith("exp_avg.embed") for k in mine)
    ex.close()


def test_clipped_policy_block_matches_autograd():
    torch.manual_seed(0)
    R, V = 64, 96
    logits = torch.randn(R, V)
    tgt = torch.randint(0, V, (R,))
    tgt[::7] = -1
    w = torch.rand(R)
    old = torch.log_softmax(logits, -1).gather(1, tgt.clamp(0)[:, None])[:, 0] + 0.3 * torch.randn(R)
    adv = torch.randn(R)
    refp = old + 0.1 * torch.randn(R)
    lf = logits.clone().requires_grad_(True)
    logp = torch.log_softmax(lf, -1).gather(1, tgt.clamp(0)[:, None])[:, 0]
    r = torch.exp(logp - old)
    per = -torch.minimum(r * adv, r.clamp(0.8, 1.2) * adv)
    d = refp - logp
    per = per + 0.05 * (torch.exp(d) - d - 1)
    want = (torch.where(tgt >= 0, w, torch.zeros(())) * per).sum()
    want.backward()
    got = torch.zeros(1)
    block = logits.clone()
    lp = torch.zeros(R)
    F.clipped_policy_(block, tgt, w, old, adv, got, clip=0.2, ref_logp=refp, ref_beta=0.05, logp=lp)
    assert torch.allclose(got[0], want.detach(), rtol=1e-5)
    assert torch.allclose(block, lf.grad, rtol=1e-4, atol=1e-6)
    assert torch.allclose(lp[tgt >= 0], logp.detach()[tgt >= 0], rtol=1e-5, atol=1e-6)
    clipped = ((r * adv) > (r.clamp(0.8, 1.2) * adv)) & (tgt >= 0)
    assert clipped.any() and (~clipped).any()        # both branches of the min were exercised


def test_policy_objective_through_the_planned_executor():
    cfg = preset("llama3-tiny")
    ob = Objective("clipped_policy", clip_ratio=0.2, reference_beta=0.02)
    assert ob.extra_fields == ("old_logprobs", "advantages", "reference_logprobs")
    geo = BatchGeometry(microbatch_tokens=256, n_microbatches=2, slots=16, mean_seqlen=64)
    prog, desc = build_step(cfg, geo, StepDataOrdering(), dtype=torch.float32, objective=ob)
    assert desc.geometry.extra_fields == ob.extra_fields
    total = sum(o.bytes for o in prog.objects) + max(t.workspace_bytes for t in prog.tasks)
    plan = plan_program(prog, MemoryBudgets(total, 64 << 20, headroom_bytes=0), CommunicationInfo(),
                        SearchOptions(minimum_object_bytes_evict_eligible=1024, workers=1))
    ex = Executor(plan, desc, device="cpu", seed=5, hyper=Hyperparameters(lr=1e-3))
    ex.initialize()
    tr = ResidentTrainer(cfg, device="cpu", dtype=torch.float32, seed=5, lr=1e-3, objective=ob)
    for step in range(2):
        host = _batch(cfg, step, n=2, extras=ob.extra_fields)
        got = ex.run(host).loss
        want = tr.step([to_device(m, "cpu") for m in host])
        assert abs(got - want) < 1e-5 * max(1.0, abs(want)), (step, got, want)
    ex.close()


def test_objective_records_and_balance_term():
    ob = Objective.from_component("shadowspill/sum@1", head="shadowspill/clipped_policy@1",
                                  head_config={"clip_ratio": 0.1}, moe_balance=0.01)
    assert ob.kind == "clipped_policy" and ob.clip_ratio == 0.1 and ob.moe_balance_coef == 0.01
    assert ob.component_id == "shadowspill/sum@1"
    assert Objective.from_json(ob.to_json()) == ob
    with pytest.raises(ValueError):
        Objective("nope")
    # perfectly balanced routing scores exactly 1; concentrating everything on one expert scores E
    E, T, k = 8, 64, 2
    uniform = router_balance(torch.full((E,), T / E), torch.full((E,), T * k // E), T, k)
    assert abs(float(uniform) - 1.0) < 1e-6
    probs = torch.zeros(E); probs[0] = T
    counts = torch.zeros(E, dtype=torch.long); counts[0] = T * k
    assert abs(float(router_balance(probs, counts, T, k)) - E) < 1e-5


def test_target_logprobs_head():
    cfg = preset("llama3-tiny")
    head = build_stages(cfg)[-1]
    P = {"final_norm": torch.ones(cfg.d_model), "head": torch.randn(cfg.vocab_size, cfg.d_model) * 0.1}
    meta = to_device(_batch(cfg)[0], "cpu")
    x = torch.randn(256, cfg.d_model)
    got = head.target_logprobs(P, x, meta)
    h = opref.rmsnorm_fwd(x, P["final_norm"], cfg.norm_epsilon)[0] if hasattr(opref, "rmsnorm_fwd") else None
    logits = (F.rmsnorm_fwd(x, P["final_norm"], cfg.norm_epsilon, False)[0] @ P["head"].t()).float()
    want = torch.log_softmax(logits, -1).gather(1, meta.targets.clamp(0)[:, None])[:, 0]
    ok = meta.targets >= 0
    assert torch.allclose(got[ok], want[ok], rtol=1e-4, atol=1e-5)


def test_router_balance_term_reaches_the_router_gradient():
    cfg = preset("olmoe-tiny")
    meta = to_device(_batch(cfg)[0], "cpu")
    grads = {}
    for coef in (0.0, 0.5, 1.0):
        tr = ResidentTrainer(cfg, device="cpu", dtype=torch.float32, seed=3,
                             objective=Objective(moe_balance_coef=coef) if coef else None)
        tr.forward_backward(meta)
        grads[coef] = tr.G[1]["router"].clone()
        if coef:
            assert float(tr.stages[1].aux_sum) > 0
    extra = grads[0.5] - grads[0.0]
    assert extra.abs().max() > 0                       # the term changed the router gradient
    # and it enters linearly in its coefficient
    assert torch.allclose(grads[1.0] - grads[0.0], 2 * extra, rtol=1e-3, atol=1e-7)
