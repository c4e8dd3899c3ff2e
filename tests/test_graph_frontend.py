"""The PyTorch graph frontend: strict export, stage partition, save / recompute graph pairs from
the AOTAutograd joint graph, gradient destinations, and planned execution of the result."""
import sys

import pytest
import torch

sys.path.insert(0, __file__.rsplit("/", 1)[0])
from test_executor_cpu import _batches  # noqa: E402

from shadowspill_b200.communication.info import CommunicationInfo
from shadowspill_b200.data.synthetic import to_device
from shadowspill_b200.execution.executor import Executor, Hyperparameters
from shadowspill_b200.execution.resident import ResidentTrainer
from shadowspill_b200.frontend import graph_pairs as gp
from shadowspill_b200.frontend.capture import BatchGeometry, StepDataOrdering, build_step
from shadowspill_b200.frontend.export import export_step, op_name, partition_export
from shadowspill_b200.frontend.graph_stage import _example_batch, capture_module
from shadowspill_b200.frontend.modules import DecoderLM
from shadowspill_b200.models.config import preset
from shadowspill_b200.planning.plan import MemoryBudgets, PlanningError, SearchOptions, plan_program

GEO = BatchGeometry(microbatch_tokens=256, n_microbatches=2, slots=16, mean_seqlen=64)


def _plan(prog, pct_from=30, spill=64 << 20):
    total = sum(o.bytes for o in prog.objects)
    ws = max(t.workspace_bytes for t in prog.tasks)
    opts = SearchOptions(minimum_object_bytes_evict_eligible=1024, workers=2)
    for pct in range(pct_from, 101, 5):
        try:
            return plan_program(prog, MemoryBudgets(ws + total * pct // 100, spill, headroom_bytes=0),
                                CommunicationInfo(), opts)
        except PlanningError:
            continue
    raise AssertionError("no budget planned")


def test_export_partition_and_pairs_of_a_dense_model():
    cfg = preset("llama3-plumbing")
    with torch.device("meta"):
        model = DecoderLM(cfg, torch.float32)
    ep = export_step(model, _example_batch(256, 16))
    ops = {op_name(n) for n in ep.graph_module.graph.nodes}
    assert {"ss.linear", "ss.rmsnorm", "ss.rope", "ss.attention", "ss.swiglu", "ss.embedding",
            "ss.head_loss"} <= ops
    exported = partition_export(ep)
    assert [s.name for s in exported.stages] == ["embed"] + [f"layer{i}" for i in range(cfg.n_layers)] + ["head"]
    keys = {s.key for s in exported.stages[1:-1]}
    assert len(keys) == 1                               # every layer is one structural contract
    layer = exported.stages[1]
    assert layer.param_names == ["attn_norm", "wqkv", "wo", "mlp_norm", "w13", "w2"]
    assert layer.boundary_in == "x" and layer.batch_fields == ["positions", "cu_seqlens"]
    whole = partition_export(ep, "whole")
    assert len(whole.stages) == 1 and whole.stages[0].boundary_in is None
    # ---- graph pairs of the layer contract
    pairs = gp.build_stage_pairs(layer, [True] * 6, grad_dtypes={"attn_norm": torch.float32,
                                                                "mlp_norm": torch.float32})
    assert set(pairs.pairs) == {"recompute", "save_attention", "save_attention_gu", "save"}
    assert len(pairs.pairs["save_attention_gu"].saved) == 4
    rec, att, sav = (pairs.pairs[v] for v in ("recompute", "save_attention", "save"))
    assert rec.saved == []
    fwd_ops = lambda pair: [op_name(n) for n in pair.backward.graph.nodes if op_name(n).startswith("ss.")]
    assert "ss.attention" in fwd_ops(rec) and "ss.attention" not in fwd_ops(att)      # kept, not redone
    assert fwd_ops(att).count("ss.linear") == 2 and "ss.linear" not in fwd_ops(sav)    # save redoes no GEMM
    assert fwd_ops(sav).count("ss.swiglu") == 1                                         # but the cheap SwiGLU
    assert len(att.saved) == 3 and len(att.saved) < len(sav.saved)
    # one fused q/k/v projection is kept once, through its base
    assert sum(s.shape == (256, (cfg.n_heads + 2 * cfg.n_kv_heads) * cfg.head_dim) for s in att.saved) == 1
    # every matrix gradient is written by the graph itself
    assert {"wqkv", "wo", "w13", "w2", "attn_norm", "mlp_norm"} <= rec.in_place
    assert any(n.target is gp.gemm_into for n in rec.backward.graph.nodes)


@pytest.mark.parametrize("name", ["llama3-tiny", "qwen3-tiny", "qwen35-tiny", "olmoe-tiny", "qwen35moe-tiny"])
def test_planned_graph_frontend_matches_the_resident_trainer(name):
    """The same 3 updates through export -> partition -> pairs -> plan (forced to spill) -> execute
    and through the resident hand-written stages; the planner mixes the variants."""
    cfg = preset(name)
    prog, desc = build_step(cfg, GEO, StepDataOrdering(), dtype=torch.float32,
                            selection={1: "save", 2: "save_attention"}, frontend="graph")
    hand, _ = build_step(cfg, GEO, StepDataOrdering(), dtype=torch.float32,
                         selection={1: "save", 2: "save_attention"})
    assert len(prog.tasks) == len(hand.tasks) and len(prog.objects) == len(hand.objects)
    assert [t.name for t in prog.tasks] == [t.name for t in hand.tasks]
    plan = _plan(prog)
    assert plan.summary.fetch_bytes > 0
    ex = Executor(plan, desc, device="cpu", seed=5, hyper=Hyperparameters(lr=3e-3))
    ex.initialize()
    ref = ResidentTrainer(cfg, device="cpu", dtype=torch.float32, seed=5, lr=3e-3)
    for step in range(3):
        host = _batches(cfg, step)
        res = ex.run(host)
        want = ref.step([to_device(m, "cpu") for m in host])
        assert abs(res.loss - want) < 1e-5 * max(1.0, abs(want)), (step, res.loss, want)
    got = ex.state_dict()
    for k, v in ref.state_dict().items():
        if k.startswith("exp_avg"):
            continue
        diff = (got[k] - v).float()
        # Adam turns the rounding noise of a near-zero gradient into a whole step, so a few elements
        # may differ by a step or two; the bulk agrees
        assert float(diff.norm() / v.float().norm().clamp_min(1e-9)) < 3e-3, k
        assert float(diff.abs().max()) <= 2 * 3e-3 + 1e-6, k        # two Adam steps
    if name == "qwen35-tiny":
        # the hybrid layers get real save variants: the DeltaNet layer and the gated-attention
        # layer keep different things, and neither is "recompute only"
        st = desc.stages()
        assert len(st[1].SAVE_SETS["save_attention"]) > 0 and len(st[2].SAVE_SETS["save"]) > 0
        assert st[1].graph.key != st[2].graph.key
    ex.close()


@pytest.mark.parametrize("name", ["llama3-tiny", "qwen35-tiny", "qwen35moe-tiny"])
def test_low_rank_adapters_train_through_the_graph_frontend(name):
    """Adapters on the attention and feed-forward matrices (and on both expert banks) of a frozen
    base: the exported stages carry the factors, frozen parameters have no gradient, moment or
    update, the layers get save variants, and three planned updates equal the resident trainer's."""
    from shadowspill_b200.models.lora import LoRAConfig
    cfg = preset(name)
    lora = LoRAConfig(rank=8, alpha=16.0, targets=("wq", "wk", "wv", "wo", "w13", "w2", "w_qkvz", "w_out"))
    sel = {1: "save", 2: "save_attention"}
    prog, desc = build_step(cfg, GEO, StepDataOrdering(), dtype=torch.float32, selection=sel, frontend="graph",
                            lora=lora)
    stages = desc.stages()
    assert type(stages[1]).__name__ == "GraphStage"                  # not the stage-class fallback
    assert len(stages[1].SAVE_SETS["save"]) > 0
    assert {p.name for p in stages[1].params if p.trainable} == {p.name for p in stages[1].params
                                                                 if "_lora_" in p.name}
    assert not any(t.name.startswith(("O.embed", "O.head", "B.embed")) for t in prog.tasks)
    full, _ = build_step(cfg, GEO, StepDataOrdering(), dtype=torch.float32, selection=sel, frontend="graph")
    state = lambda p: sum(o.bytes for o in p.objects if o.kind in ("gradient", "optimizer_state"))
    assert state(prog) < 0.25 * state(full)
    if cfg.is_moe:
        ops = [op_name(n) for n in stages[1].pairs.pairs["recompute"].backward.graph.nodes]
        assert "ss.moe_experts_lora_bwd" in ops and "ss.moe_experts_bwd" not in ops
    plan = _plan(prog)
    ex = Executor(plan, desc, device="cpu", seed=5, hyper=Hyperparameters(lr=1e-2))
    ex.initialize()
    ref = ResidentTrainer(cfg, device="cpu", dtype=torch.float32, seed=5, lr=1e-2, lora=lora)
    for step in range(3):
        host = _batches(cfg, step)
        res = ex.run(host)
        want = ref.step([to_device(m, "cpu") for m in host])
        assert abs(res.loss - want) < 1e-5 * max(1.0, abs(want)), (step, res.loss, want)
    got = ex.state_dict()
    moved = 0.0
    for k, v in ref.state_dict().items():
        if k.startswith("exp_avg"):
            continue
        diff = (got[k] - v).float()
        assert float(diff.abs().max()) <= 2 * 1e-2 + 1e-6, k
        assert float(diff.norm() / v.float().norm().clamp_min(1e-9)) < 3e-3 or float(v.float().norm()) < 1e-3, k
        if k.endswith("_lora_b"):
            moved = max(moved, float(got[k].abs().max()))
    assert moved > 0                      # the zero-initialised factors were trained
    ex.close()


@pytest.mark.parametrize("name", ["llama3-tiny", "qwen3-tiny", "qwen35-tiny"])
def test_axis_chunked_stage_graphs_compute_the_same_step(name):
    """Row-chunking the token-local regions of every layer graph (projections, norms, MLP; the
    sequence mixers stay whole) changes the graphs and their live intermediates, not the numbers:
    three planned updates agree with the unchunked graphs, and the gradients' in-place forms
    accumulate across chunks (created by the first chunk of the first microbatch only)."""
    from shadowspill_b200.frontend import chunking
    cfg = preset(name)
    sel = {1: "save", 2: "save_attention"}
    whole, desc_w = build_step(cfg, GEO, StepDataOrdering(), dtype=torch.float32, selection=sel, frontend="graph")
    prog, desc = build_step(cfg, GEO, StepDataOrdering(), dtype=torch.float32, selection=sel, frontend="graph",
                            axis_chunk_rows=96)                       # 256 rows: chunks of 96, 96, 64
    sw, sc = desc_w.stages(), desc.stages()
    regions = 0
    for a, b in zip(sw[1:-1], sc[1:-1]):
        for v in a.pairs.pairs:
            fa, fb = a.pairs.pairs[v].forward, b.pairs.pairs[v].forward
            cats = [n for n in fb.graph.nodes if op_name(n) == "aten.cat.default"]
            assert len(fb.graph.nodes) > len(fa.graph.nodes) and cats
            regions += len(cats)
            # barriers are never replicated
            for kind in ("ss.attention", "ss.gated_delta_rule", "ss.conv_silu"):
                assert (sum(op_name(n) == kind for n in fb.graph.nodes)
                        == sum(op_name(n) == kind for n in fa.graph.nodes))
            # the widest projection is evaluated once per chunk
            assert (sum(op_name(n) == "ss.linear" for n in fb.graph.nodes)
                    == 3 * sum(op_name(n) == "ss.linear" for n in fa.graph.nodes))
        assert ":rows96" in b.mixer and ":rows" not in a.mixer
    assert regions > 0
    assert {t.profile_key for t in prog.tasks} != {t.profile_key for t in whole.tasks}

    def run(program, description):
        ex = Executor(_plan(program), description, device="cpu", seed=5, hyper=Hyperparameters(lr=3e-3))
        ex.initialize()
        losses = [ex.run(_batches(cfg, step)).loss for step in range(3)]
        state = ex.state_dict()
        ex.close()
        return losses, state
    lw, stw = run(whole, desc_w)
    lc, stc = run(prog, desc)
    for a, b in zip(lw, lc):
        assert abs(a - b) < 1e-5 * max(1.0, abs(a)), (lw, lc)
    for k, v in stw.items():
        if k.startswith("exp_avg"):
            continue
        diff = (stc[k] - v).float()
        assert float(diff.norm() / v.float().norm().clamp_min(1e-9)) < 1e-3, k
    mixers = [n for st in sw[1:-1] for n in st.pairs.pairs["recompute"].forward.graph.nodes
              if op_name(n) in ("ss.attention", "ss.gated_delta_rule", "ss.conv_silu")]
    assert mixers and all(chunking.classify(n, 256)[0] == chunking.BARRIER for n in mixers)


def test_routed_expert_layers_get_save_variants_and_in_place_bank_gradients():
    """A routed-expert model goes through the graph frontend: every layer has the save variants
    the planner mixes, the routed experts are one operator (a barrier for axis chunks), and both
    bank gradients are written by the backward graph itself."""
    from shadowspill_b200.frontend import chunking
    from shadowspill_b200.frontend.graph_stage import build_graph_stages, supports
    from dataclasses import replace
    cfg = preset("olmoe-tiny")
    assert supports(cfg) and not supports(replace(cfg, router_aux_coef=0.01))
    stages = build_graph_stages(cfg, 256, 16, torch.float32)
    layer = stages[1]
    assert set(layer.SAVE_SETS) >= {"recompute", "save_attention", "save"}
    assert len(layer.SAVE_SETS["save"]) > len(layer.SAVE_SETS["save_attention"]) > 0
    pair = layer.pairs.pairs["save_attention"]
    assert {"router", "w13", "w2"} <= pair.in_place
    targets = [n.target for n in pair.backward.graph.nodes if n.op == "call_function"]
    assert gp.moe_experts_bwd_into in targets
    assert not any(op_name(n) == "ss.moe_experts_bwd" for n in pair.backward.graph.nodes)
    mixers = [n for n in pair.forward.graph.nodes if op_name(n) == "ss.moe_experts"]
    assert len(mixers) == 1 and chunking.classify(mixers[0], 256)[0] == chunking.BARRIER
    cut = build_graph_stages(cfg, 256, 16, torch.float32, chunk_rows=64)
    assert sum(op_name(n) == "ss.moe_experts" for n in cut[1].pairs.pairs["recompute"].forward.graph.nodes) == 1


def test_fused_forms_replace_copies_adds_and_zero_filled_slice_gradients():
    """The layer graphs run rotary in place on the fresh projection output, fold the residual add
    into the norm kernel, and build the gradient of the fused q/k/v projection by one concatenation
    instead of three zero-filled full-width tensors added together."""
    from shadowspill_b200.frontend import fusion
    from shadowspill_b200.frontend.graph_stage import build_graph_stages
    layer = build_graph_stages(preset("llama3-tiny"), 256, 16, torch.float32)[1]
    pair = layer.pairs.pairs["recompute"]
    fwd = [n.target for n in pair.forward.graph.nodes if n.op == "call_function"]
    bwd = [n for n in pair.backward.graph.nodes if n.op == "call_function"]
    assert fusion.rope_in_place in fwd and fusion.add_rmsnorm in fwd
    assert not any(op_name(n) == "ss.rope" for n in pair.forward.graph.nodes)
    assert not any(op_name(n) == "aten.slice_backward.default" for n in bwd)
    assert sum(op_name(n) == "aten.cat.default" for n in bwd) == 1
    assert sum(n.target is fusion.rope_in_place for n in bwd) == 2        # recomputed forward + its gradient
    # the first norm reads the stage input, which is never written: it stays a plain norm
    first_norm = next(n for n in pair.forward.graph.nodes if n.op == "call_function")
    assert op_name(first_norm) == "ss.rmsnorm" and first_norm.args[0].op == "placeholder"


def test_axis_chunks_shrink_the_live_intermediates_of_a_wide_layer():
    """With an MLP eight times wider than the model, the live intermediates of the chunked
    backward graph (counted from the traced shapes) are a fraction of the whole graph's."""
    from shadowspill_b200.frontend import chunking
    from shadowspill_b200.frontend.graph_stage import build_graph_stages
    from shadowspill_b200.models.config import DecoderConfig
    cfg = DecoderConfig("llama3", 2, 256, 4, 2, 64, 2048, 512)
    whole = build_graph_stages(cfg, 2048, 16, torch.bfloat16)
    cut = build_graph_stages(cfg, 2048, 16, torch.bfloat16, chunk_rows=256)
    for variant in ("recompute", "save_attention"):
        a = chunking.peak_intermediate_bytes(whole[1].pairs.pairs[variant].backward)
        b = chunking.peak_intermediate_bytes(cut[1].pairs.pairs[variant].backward)
        assert b < 0.6 * a, (variant, a, b)
    assert cut[1].workspace_bytes(2048) <= whole[1].workspace_bytes(2048)


def test_plumbing_config_twenty_steps_match_eager_pytorch():
    """BASELINE configuration 0: the tiny Llama through export, partition, profile-free planning with
    half of the state spilled, execution and the plan report, against plain eager PyTorch + AdamW."""
    from shadowspill_b200.data.synthetic import make_batch
    from shadowspill_b200.models import torch_reference as tr
    cfg = preset("llama3-plumbing")
    geo = BatchGeometry(microbatch_tokens=1024, n_microbatches=2, slots=16, mean_seqlen=256)
    prog, desc = build_step(cfg, geo, StepDataOrdering(), dtype=torch.float32,
                            selection={i: ("save" if i % 2 else "recompute") for i in range(1, cfg.n_layers + 1)},
                            frontend="graph")
    plan = _plan(prog, pct_from=50)
    assert plan.summary.fetch_bytes > 0 and plan.summary.evict_bytes > 0
    hyper = Hyperparameters(lr=1e-3, beta2=0.999, weight_decay=0.0)
    ex = Executor(plan, desc, device="cpu", seed=7, hyper=hyper)
    ex.initialize()
    params = {k: v.clone().requires_grad_(True) for k, v in ex.state_dict().items() if not k.startswith("exp_avg")}
    opt = torch.optim.AdamW(list(params.values()), lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0)
    for step in range(20):
        host = make_batch(step, vocab=cfg.vocab_size, tokens_per_step=2048, microbatch_tokens=1024,
                          median=200, min_len=64, max_len=512, slots=16)
        got = ex.run(host).loss
        opt.zero_grad()
        want = 0.0
        for m in host:
            loss = tr.loss(cfg, params, to_device(m, "cpu"))
            loss.backward()
            want += float(loss)
        opt.step()
        assert abs(got - want) < 1e-5 * max(1.0, abs(want)), (step, got, want)
    state = ex.state_dict()
    # weights: relative L2 error, and no element further off than two Adam steps (a gradient that
    # is zero up to rounding may take either sign)
    for k, v in params.items():
        diff = (state[k] - v.detach()).float()
        assert float(diff.norm() / v.detach().float().norm()) < 1e-3, k
        assert float(diff.abs().max()) <= 2 * 1e-3 + 1e-6, k
    ex.close()


@pytest.mark.gpu
@pytest.mark.parametrize("name", ["llama3-small", "qwen35-numerical-small", "qwen35moe-lora-small"])
def test_graph_frontend_on_the_gpu_matches_the_stage_classes(name):
    """bf16 on the GPU: the exported graphs run the same sm_100a kernels as the hand-written stages,
    so two planned updates give the same losses and weights up to bf16 rounding of reordered sums."""
    from dataclasses import replace
    from shadowspill_b200.data.synthetic import make_batch
    from shadowspill_b200.ops import _lib
    lora = None
    if name == "qwen35-numerical-small":
        # DeltaNet heads of width 128 (the chunk kernels), two layers of each mixer kind
        cfg = replace(preset("qwen35-numerical"), n_layers=4, d_model=512, d_ff=1024, n_heads=4, n_kv_heads=2,
                      head_dim=128, dn_qk_heads=2, dn_v_heads=4, vocab_size=2048)
    elif name == "qwen35moe-lora-small":
        # adapters on attention, DeltaNet and both expert banks of a frozen routed hybrid
        from shadowspill_b200.models.lora import LoRAConfig
        cfg = replace(preset("qwen35moe-tiny"), n_layers=4, d_model=256, n_heads=4, n_kv_heads=2, head_dim=64,
                      dn_qk_heads=2, dn_v_heads=4, dn_head_dim=128, vocab_size=2048)
        lora = LoRAConfig(rank=16, alpha=32.0, targets=("wq", "wk", "wv", "wo", "w13", "w2", "w_qkvz", "w_out"))
    else:
        cfg = replace(preset("llama3-tiny"), d_model=256, n_heads=4, n_kv_heads=2, head_dim=64, d_ff=512)
    geo = BatchGeometry(microbatch_tokens=1024, n_microbatches=2, slots=33, mean_seqlen=256)
    sel = {i: ("save" if i % 2 else "save_attention") for i in range(1, cfg.n_layers + 1)}
    losses, states = {}, {}
    for frontend in ("stages", "graph"):
        prog, desc = build_step(cfg, geo, StepDataOrdering(), dtype=torch.bfloat16,
                                selection=sel if frontend == "graph" else {}, frontend=frontend, lora=lora)
        if frontend == "graph":
            assert type(desc.stages()[1]).__name__ == "GraphStage"
        plan = _plan(prog, pct_from=60, spill=1 << 30)
        ex = Executor(plan, desc, device="cuda", seed=11, hyper=Hyperparameters(lr=1e-3),
                      stochastic_rounding=False)
        ex.initialize(on_device=False)
        out = []
        for step in range(2):
            host = make_batch(step, vocab=cfg.vocab_size, tokens_per_step=2048, microbatch_tokens=1024,
                              median=200, min_len=16, max_len=1024, slots=33)
            out.append(ex.run(host).loss)
        _lib.check_status()
        losses[frontend], states[frontend] = out, ex.state_dict()
        ex.close()
    for a, b in zip(losses["stages"], losses["graph"]):
        assert abs(a - b) < 2e-2 * max(1.0, abs(b)), (losses)
    for k, v in states["stages"].items():
        if k.startswith("exp_avg"):
            continue
        w = states["graph"][k].float()
        rel = float((w - v.float()).norm() / v.float().norm().clamp_min(1e-9))
        if k.endswith("_lora_b"):
            # starts at zero and moves by about lr per update whatever the gradient's size: compare directions
            cos = float(torch.dot(w.flatten(), v.float().flatten()) / (w.norm() * v.float().norm()).clamp_min(1e-12))
            assert cos > 0.8, (k, cos)
            continue
        if k.endswith("_lora_a"):
            # one update of about lr on values of size 0.02: a flipped sign is a 10 % change of that element
            assert rel < 6e-2, (k, rel)
            continue
        # norm vectors see the sum of many bf16-rounded terms in a different order
        assert rel < (5e-2 if v.dim() == 1 else 2.5e-2), (k, rel)


def test_an_operator_of_the_users_own_takes_part_through_its_rule():
    """A custom operator with a declared rule (memory-bound, rows in argument 0) is exported,
    differentiated, recomputed instead of kept by the ``save`` policy, and cut by row chunking."""
    from torch import nn
    from shadowspill_b200.frontend import modules as M
    from shadowspill_b200.frontend.chunking import ROWS, classify
    from shadowspill_b200.frontend.graph_stage import build_graph_stages
    from shadowspill_b200.frontend.operator_rules import OperatorRule, register_operator_rule, rule_of

    @torch.library.custom_op("acme::soft_gate", mutates_args=())
    def soft_gate(x: torch.Tensor, slope: float) -> torch.Tensor:
        return x * torch.sigmoid(slope * x.float()).to(x.dtype)

    @soft_gate.register_fake
    def _(x, slope):
        return torch.empty_like(x)

    def _bwd(ctx, gy):
        (x,) = ctx.saved_tensors
        s = torch.sigmoid(ctx.slope * x.float())
        return (gy * (s + ctx.slope * x.float() * s * (1 - s)).to(gy.dtype)), None
    soft_gate.register_autograd(_bwd, setup_context=lambda ctx, inputs, output: (ctx.save_for_backward(inputs[0]),
                                                                                  setattr(ctx, "slope", inputs[1])))
    if rule_of("acme.soft_gate") is None:
        register_operator_rule(OperatorRule("acme.soft_gate", "memory", (0,)))
    with pytest.raises(ValueError):
        register_operator_rule(OperatorRule("acme.soft_gate", "compute"))

    class GatedLayer(M.DenseLayer):
        def forward(self, x, positions, cu_seqlens):
            return super().forward(torch.ops.acme.soft_gate(x, 0.5), positions, cu_seqlens)

    class Model(M.DecoderLM):
        def __init__(self, cfg):
            super().__init__(cfg, torch.float32)
            self.layers = nn.ModuleList([GatedLayer(cfg, torch.float32) for _ in range(cfg.n_layers)])

    cfg = preset("llama3-tiny")
    with torch.device("meta"):
        meta_model = Model(cfg)
    stages = build_graph_stages(cfg, 256, 16, torch.float32, module=meta_model, chunk_rows=64)
    layer = stages[1]
    fwd_nodes = [n for n in layer.graph.gm.graph.nodes if n.op == "call_function"]
    mine = next(n for n in fwd_nodes if "soft_gate" in op_name(n))
    assert classify(mine, 256) == (ROWS, (0,))
    # the save policy recomputes it (its output is not among the kept values), and the backward graph redoes it
    save = layer.pairs.pairs["save"]
    assert any("soft_gate" in op_name(n) for n in save.backward.graph.nodes)
    # row chunking cut it: four copies in the chunked forward
    assert sum("soft_gate" in op_name(n) for n in layer.pairs.pairs["recompute"].forward.graph.nodes) == 4


def test_sparse_latent_attention_family_trains_like_eager_pytorch():
    """GLM 5.3 in small: sparse multi-head latent attention with a frozen indexer whose picks are
    reused by the next layer, sigmoid-scored routed experts with a shared expert, a dense first
    layer. Layers that share picks form one stage. Five planned updates (forced to spill) equal
    eager PyTorch + AdamW on the same module."""
    from shadowspill_b200.frontend.modules import DecoderLM, init_
    cfg = preset("glm53-tiny")
    assert cfg.layer_groups() == [[0, 1], [2, 3]]
    prog, desc = build_step(cfg, GEO, StepDataOrdering(), dtype=torch.float32, selection={1: "save", 2: "save_attention"})
    stages = desc.stages()
    assert [type(s).__name__ for s in stages] == ["GraphEmbeddingStage", "GraphStage", "GraphStage", "GraphHeadStage"]
    first, second = stages[1], stages[2]
    assert any(p.name == "members_1_kv_b" for p in first.params) and not any("ix_" in p.name and p.trainable for p in first.params)
    assert sum("ix_q" in p.name for p in first.params) == 1          # one indexer per group: the second layer shares
    ops_of = lambda st: [op_name(n) for n in st.graph.gm.graph.nodes]
    assert ops_of(first).count("ss.index_topk") == 1 and ops_of(first).count("ss.sparse_latent_attention") == 2
    assert "ss.moe_experts_routed" in ops_of(first) and ops_of(second).count("ss.moe_experts_routed") == 2
    assert first.graph.key != second.graph.key                        # the first group has the dense layer
    assert len(first.SAVE_SETS["save"]) > len(first.SAVE_SETS["save_attention"]) >= 0
    plan = _plan(prog)
    assert plan.summary.fetch_bytes > 0
    ex = Executor(plan, desc, device="cpu", seed=5, hyper=Hyperparameters(lr=3e-3))
    ex.initialize()
    model = DecoderLM(cfg, torch.float32)
    state = ex.state_dict()
    params = dict(model.named_parameters())
    names = {}
    for st, group in zip(stages, [["embed"], ["layers.0"], ["layers.1"], ["head"]]):
        for p in st.params:
            target = next(t for t in params if t.startswith(group[0] + ".") and
                          (t.split(".")[-1] == p.name or "_".join(t.split(".")[2:]) == p.name))
            names[f"{st.name}.{p.name}"] = target
    with torch.no_grad():
        for k, target in names.items():
            params[target].copy_(state[k])
    trainable = [p for p in model.parameters() if p.requires_grad]
    opt = torch.optim.AdamW(trainable, lr=3e-3, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.0)
    for step in range(5):
        host = _batches(cfg, step)
        got = ex.run(host).loss
        opt.zero_grad()
        want = 0.0
        for mb in host:
            m = to_device(mb, "cpu")
            loss = model(m.tokens, m.targets, m.weights, m.positions, m.cu_seqlens)
            loss.sum().backward()
            want += float(loss)
        opt.step()
        # the indexer's picks and the routers' top-k are discrete: a rounding-level difference between
        # the fused planned graphs and eager execution can flip a near-tie, which moves the loss in the
        # fourth digit; anything structural would be orders of magnitude larger
        assert abs(got - want) < 5e-4 * max(1.0, abs(want)), (step, got, want)
    state = ex.state_dict()
    for k, target in names.items():
        v = params[target].detach()
        diff = (state[k] - v).float()
        assert float(diff.abs().max()) <= 5 * 3e-3 + 1e-6, k
        assert float(diff.norm() / v.float().norm().clamp_min(1e-9)) < 2e-2 or float(v.float().norm()) < 1e-2, k
    ex.close()


@pytest.mark.gpu
def test_sparse_latent_attention_family_on_the_gpu_follows_the_cpu_run():
    """The GLM-shaped model in bf16 on the GPU (projections and routed experts on the tcgen05
    kernels, latent attention and the indexer as tensor operations) against the same planned run in
    fp32 on the CPU from the same seed: losses agree to bf16 accuracy over three updates."""
    from dataclasses import replace
    from shadowspill_b200.data.synthetic import make_batch
    from shadowspill_b200.ops import _lib
    cfg = replace(preset("glm53-tiny"), d_model=256, d_ff=256, vocab_size=2048, q_lora_rank=64, kv_lora_rank=64,
                  qk_nope_head_dim=64, v_head_dim=64, head_dim=128, index_n_heads=8, index_topk=32, d_expert=128,
                  d_shared_expert=128, n_experts=8)        # the router GEMM wants its width in multiples of 8
    geo = BatchGeometry(microbatch_tokens=1024, n_microbatches=2, slots=33, mean_seqlen=256)
    losses = {}
    for device, dtype in (("cpu", torch.float32), ("cuda", torch.bfloat16)):
        prog, desc = build_step(cfg, geo, StepDataOrdering(), dtype=dtype, selection={1: "save_attention"})
        plan = _plan(prog, pct_from=60, spill=1 << 30)
        ex = Executor(plan, desc, device=device, seed=11, hyper=Hyperparameters(lr=1e-3), stochastic_rounding=False)
        ex.initialize(on_device=False)
        out = []
        for step in range(3):
            host = make_batch(step, vocab=cfg.vocab_size, tokens_per_step=2048, microbatch_tokens=1024,
                              median=200, min_len=16, max_len=1024, slots=33)
            out.append(ex.run(host).loss)
        if device == "cuda":
            _lib.check_status()
        losses[device] = out
        ex.close()
    for a, b in zip(losses["cpu"], losses["cuda"]):
        assert abs(a - b) < 2e-2 * max(1.0, abs(a)), losses


def test_adapters_on_the_latent_attention_family():
    """Adapters on the latent projections (the absorbed key/value projection included), the dense
    and shared feed-forward and both routed banks of the GLM-shaped model: the adapted forward
    equals the forward with merged weights, only factors train, and three planned updates follow
    eager PyTorch on the same module."""
    from shadowspill_b200.frontend.modules import DecoderLM, init_
    from shadowspill_b200.models.lora import LoRAConfig
    cfg = preset("glm53-tiny")
    lora = LoRAConfig(rank=8, alpha=16.0, targets=("q_a", "q_b", "kv_a", "kv_b", "wo", "w13", "w2", "sw13", "sw2"))
    # ---- merged-weight equivalence, factors made non-trivial
    model = DecoderLM(cfg, torch.float32, lora=lora)
    init_(model, 0)
    gen = torch.Generator().manual_seed(1)
    with torch.no_grad():
        for n, p in model.named_parameters():
            if n.endswith("_lora_b"):
                p.copy_(torch.randn(p.shape, generator=gen) * 0.05)
    merged = DecoderLM(cfg, torch.float32)
    mine = dict(model.named_parameters())
    with torch.no_grad():
        for n, p in merged.named_parameters():
            w = mine[n].detach().clone()
            if n + "_lora_a" in mine:
                w = w + lora.scale * (mine[n + "_lora_b"] @ mine[n + "_lora_a"])
            p.copy_(w)
    host = _batches(cfg, 0)
    m0 = to_device(host[0], "cpu")
    args = (m0.tokens, m0.targets, m0.weights, m0.positions, m0.cu_seqlens)
    assert abs(float(model(*args)) - float(merged(*args))) < 1e-5
    assert all(("_lora_" in n) == p.requires_grad for n, p in model.named_parameters())
    # ---- planned execution against eager training of the same module
    prog, desc = build_step(cfg, GEO, StepDataOrdering(), dtype=torch.float32, selection={1: "save"}, lora=lora)
    stages = desc.stages()
    ops_of = [op_name(n) for n in stages[2].graph.gm.graph.nodes]
    assert "ss.moe_experts_routed_lora" in ops_of and "ss.moe_experts_routed" not in ops_of
    assert not any(t.name.startswith(("O.embed", "O.head", "B.embed")) for t in prog.tasks)
    plan = _plan(prog)
    ex = Executor(plan, desc, device="cpu", seed=5, hyper=Hyperparameters(lr=1e-2))
    ex.initialize()
    state = ex.state_dict()
    eager = DecoderLM(cfg, torch.float32, lora=lora)
    params = dict(eager.named_parameters())
    names = {}
    for st, group in zip(stages, ["embed", "layers.0", "layers.1", "head"]):
        for p in st.params:
            names[f"{st.name}.{p.name}"] = next(t for t in params if t.startswith(group + ".") and (
                t.split(".")[-1] == p.name or "_".join(t.split(".")[2:]) == p.name))
    with torch.no_grad():
        for k, target in names.items():
            params[target].copy_(state[k])
    opt = torch.optim.AdamW([p for p in eager.parameters() if p.requires_grad], lr=1e-2, betas=(0.9, 0.95),
                            eps=1e-8, weight_decay=0.0)
    for step in range(3):
        host = _batches(cfg, step)
        got = ex.run(host).loss
        opt.zero_grad()
        want = 0.0
        for mb in host:
            m = to_device(mb, "cpu")
            loss = eager(m.tokens, m.targets, m.weights, m.positions, m.cu_seqlens)
            loss.sum().backward()
            want += float(loss.detach())
        opt.step()
        assert abs(got - want) < 5e-4 * max(1.0, abs(want)), (step, got, want)
    state = ex.state_dict()
    moved = max(float(state[k].abs().max()) for k in names if k.endswith("_lora_b"))
    assert moved > 0
    for k, target in names.items():
        diff = (state[k] - params[target].detach()).float()
        assert float(diff.abs().max()) <= 3 * 1e-2 + 1e-6, k
    ex.close()


def test_row_chunks_on_the_latent_attention_family():
    """Row chunks cut the projections, norms and the feed-forward of the GLM-shaped stages (several
    layers each) while the indexer, the sparse latent attention and the routed experts stay whole;
    the chunked program follows the whole one."""
    cfg = preset("glm53-tiny")
    whole, desc_w = build_step(cfg, GEO, StepDataOrdering(), dtype=torch.float32)
    prog, desc = build_step(cfg, GEO, StepDataOrdering(), dtype=torch.float32, axis_chunk_rows=96)
    for a, b in zip(desc_w.stages()[1:-1], desc.stages()[1:-1]):
        fa, fb = a.pairs.pairs["recompute"].forward, b.pairs.pairs["recompute"].forward
        count = lambda g, kind: sum(op_name(n) == kind for n in g.graph.nodes)
        for kind in ("ss.index_topk", "ss.sparse_latent_attention", "ss.moe_experts_routed"):
            assert count(fb, kind) == count(fa, kind)
        assert count(fb, "ss.linear") > count(fa, "ss.linear") and ":rows96" in b.mixer

    def run(program, description):
        ex = Executor(_plan(program), description, device="cpu", seed=5, hyper=Hyperparameters(lr=3e-3))
        ex.initialize()
        losses = [ex.run(_batches(cfg, step)).loss for step in range(3)]
        ex.close()
        return losses
    for a, b in zip(run(whole, desc_w), run(prog, desc)):
        assert abs(a - b) < 5e-4 * max(1.0, abs(a))        # discrete picks: see the eager comparison above
