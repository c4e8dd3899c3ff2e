"""Stages whose forward and backward passes are FX graphs derived from an exported model.

``build_graph_stages`` runs the whole graph frontend for a catalog model (or any
``nn.Module`` with the same call contract): strict export, partition at the repeated child,
one joint graph per structural contract, save / recompute / rule-based graph pairs, gradient
destinations. The resulting ``GraphStage`` objects implement the same interface as the
hand-written stage classes of :mod:`shadowspill_b200.models.decoder`, so the program builder,
the profiler, the planner and the executor treat them alike; the difference is that nothing
about the layer's structure is written down here: a changed or new layer needs no new class.

Reference: packages/engine/src/shadowspill/build/training.py:162 (``_build_training``: capture ->
partition -> graph pairs -> lowering).
"""
from __future__ import annotations

import os

import operator
import threading

import torch
from torch import fx, nn

from ..models.decoder import BatchMeta, ParamSpec, Stage
from . import graph_pairs as gp
from .export import ExportedStep, StageGraph, export_step, op_name, partition_export


def _param_specs(stage: StageGraph, exported: ExportedStep, model_dtype: torch.dtype) -> list[ParamSpec]:
    specs = []
    for local, target in zip(stage.param_names, stage.param_targets):
        p = exported.parameters[target]
        specs.append(ParamSpec(local, tuple(p.shape), init=getattr(p, "ss_init", "normal"),
                               std=float(getattr(p, "ss_std", 0.02)),
                               dtype=None if p.dtype == model_dtype else p.dtype,
                               trainable=bool(p.requires_grad)))
    return specs


class GraphStage(Stage):
    """A stage executed as FX graphs. ``pairs`` holds one (forward, backward) pair per variant."""
    kind = "layer"

    def __init__(self, name: str, cfg, stage: StageGraph, pairs: gp.StagePairs, params: list[ParamSpec],
                 foreign: dict[str, str] | None = None):
        super().__init__(name, cfg)
        self.graph, self.pairs = stage, pairs
        # parameters another stage owns (a tied embedding read by the head): local name -> owner's name
        self.foreign = dict(foreign or {})
        self.params = [p for p in params if p.name not in self.foreign]
        self.mixer = stage.key                 # keeps profiles of different structures apart
        self.SAVE_SETS = {v: tuple(s.name for s in pair.saved) for v, pair in pairs.pairs.items()}
        self._by_keep = {names: v for v, names in self.SAVE_SETS.items()}
        # parameters the forward graph uses only as the weight of ss.linear: their gather can be
        # fused into that GEMM under sharded storage
        weight_of, other = set(), set()
        for n in stage.gm.graph.nodes:
            for i, a in enumerate(n.args if n.op == "call_function" else ()):
                if isinstance(a, fx.Node) and a.op == "placeholder" and str(a.target) in stage.param_names:
                    (weight_of if (op_name(n) == "ss.linear" and i == 1) else other).add(str(a.target))
        self.fused_gather_params = tuple(sorted(weight_of - other)) if self.kind == "layer" else ()

    # ---- sizes
    def saved_shapes(self, T, variant, dtype=torch.bfloat16):
        return [(s.name, s.shape, s.dtype) for s in self.pairs.pairs[variant].saved]

    def activation_bytes(self, T, variant, itemsize=2):
        return sum(int(torch.tensor([], dtype=s.dtype).element_size()) * _numel(s.shape)
                   for s in self.pairs.pairs[variant].saved)

    def workspace_bytes(self, T, itemsize=2):
        return int(self.pairs.intermediate_bytes * 1.5)

    def flops(self, T, mean_seqlen):
        fl = self.pairs.flops_linear
        for n in self.graph.gm.graph.nodes:
            if op_name(n) == "ss.attention":
                q = n.args[0].meta["val"]
                fl += 4.0 * q.shape[0] * (mean_seqlen / 2.0) * q.shape[1] * q.shape[2]
            elif op_name(n) == "ss.gated_delta_rule":
                v = n.args[2].meta["val"]
                fl += 6.0 * v.shape[0] * v.shape[1] * v.shape[2] * v.shape[2]
        return fl

    # ---- execution
    def _inputs(self, P, x, meta: BatchMeta, names: list[str], extra: dict | None = None):
        vals = []
        for nm in names:
            if extra is not None and nm in extra:
                vals.append(extra[nm])
            elif nm == "x":
                vals.append(x)
            elif nm in P:
                vals.append(P[nm])
            elif hasattr(meta, nm):
                vals.append(getattr(meta, nm))
            elif nm in meta.extras:
                vals.append(meta.extras[nm])
            else:
                raise KeyError(f"{self.name}: no value for graph input {nm!r}")
        return vals

    def forward(self, P, x, meta: BatchMeta, keep: tuple[str, ...] = (), out=None, saved_out=None):
        variant = self._by_keep.get(tuple(keep), "recompute")
        pair = self.pairs.pairs[variant]
        with torch.no_grad():
            res = _runnable(pair, "forward")(*self._inputs(P, x, meta, self.pairs.placeholders))
        y, kept = res[0], res[1:]
        if out is not None:
            out.copy_(y)
            y = out
        saved = {}
        for spec, val in zip(pair.saved, kept):
            if saved_out is not None and spec.name in saved_out:
                saved_out[spec.name].copy_(val.reshape(saved_out[spec.name].shape))
                saved[spec.name] = saved_out[spec.name]
            else:
                saved[spec.name] = val
        return y, saved

    def backward(self, P, G, x, dy, meta: BatchMeta, saved: dict, first: bool):
        variant = self._by_keep.get(tuple(sorted(saved, key=_saved_index)), None) if saved else "recompute"
        if variant is None:
            variant = next(v for v, names in self.SAVE_SETS.items() if set(names) == set(saved))
        pair = self.pairs.pairs[variant]
        extra = {"tangent_0": dy, "first": first}
        for nm in pair.backward_inputs:
            if nm.startswith("saved_"):
                extra[nm] = saved[nm]
            elif nm.startswith("grad_"):
                extra[nm] = G[nm[5:]]
        with torch.no_grad():
            grads = _runnable(pair, "backward")(*self._inputs(P, x, meta, pair.backward_inputs, extra))
        dx = None
        for target, g in zip(pair.grad_outputs, grads):
            if target is None or g is None:
                continue
            if target == "x":
                dx = g
            elif target not in pair.in_place and G and target in G:
                dst = G[target]
                if first:
                    dst.copy_(g.reshape(dst.shape))
                else:
                    dst.add_(g.reshape(dst.shape).to(dst.dtype))
        if dx is not None:
            dy.copy_(dx)
        return dy


def _runnable(owner, attr: str) -> fx.GraphModule:
    """The execution form of a graph held in ``owner.<attr>`` (made once, kept beside it)."""
    cached = getattr(owner, "_exec_" + attr, None)
    gm = getattr(owner, attr)
    if cached is None or cached[0] is not gm:
        from .fusion import lower_for_execution
        cached = (gm, lower_for_execution(gm) if os.environ.get("SS_GRAPH_LOWER", "1") != "0" else gm)
        setattr(owner, "_exec_" + attr, cached)
    return cached[1]


def _saved_index(name: str) -> int:
    return int(name.split("_")[1])


def _numel(shape) -> int:
    n = 1
    for d in shape:
        n *= int(d)
    return n


class GraphEmbeddingStage(GraphStage):
    kind = "embedding"

    def forward(self, P, x, meta: BatchMeta, keep=None, out=None, saved_out=None):
        return super().forward(P, None, meta, (), out=out)

    def backward(self, P, G, x, dy, meta: BatchMeta, saved, first: bool):
        pair = self.pairs.pairs["recompute"]
        extra = {"tangent_0": dy, "first": first}
        for nm in pair.backward_inputs:
            if nm.startswith("grad_"):
                extra[nm] = G[nm[5:]]
        with torch.no_grad():
            grads = _runnable(pair, "backward")(*self._inputs(P or {}, None, meta, pair.backward_inputs, extra))
        for target, g in zip(pair.grad_outputs, grads):
            if target and target != "x" and target not in pair.in_place and g is not None:
                (G[target].copy_ if first else G[target].add_)(g.reshape(G[target].shape))
        return None


class GraphHeadStage(GraphStage):
    """The last stage: its joint graph (forward and backward in one) runs as a single task."""
    kind = "head"
    output_width = 1

    def __init__(self, name, cfg, stage, pairs, params, foreign=None, block_rows: int = 2048):
        super().__init__(name, cfg, stage, pairs, params, foreign)
        self.block_rows = block_rows
        self._train: fx.GraphModule | None = None
        self._train_inputs: list[str] = []
        self._train_grads: list[str | None] = []

    def _train_graph(self):
        if self._train is None:
            self._train, self._train_inputs, self._train_grads = _head_training_graph(self.pairs, self.graph)
        return _runnable(self, "_train")

    def loss_and_backward(self, P, G, x, meta: BatchMeta, loss_sum, first: bool, dx=None, train: bool = True,
                          grad_scale: float = 1.0, tied: dict | None = None):
        P = dict(P)
        Gall = dict(G or {})
        first_of = {}
        for local, owner in self.foreign.items():
            P[local] = tied["params"][owner]
            if tied.get("grads"):
                Gall[local] = tied["grads"][owner]
                first_of[local] = bool(tied.get("first", False))
        if not train:
            with torch.no_grad():
                loss = _runnable(self.pairs.pairs["recompute"], "forward")(
                    *self._inputs(P, x, meta, self.pairs.placeholders))[0]
            loss_sum.add_(loss.reshape(loss_sum.shape))
            return None
        gm = self._train_graph()
        extra = {"first": first}
        for nm in self._train_inputs:
            if nm.startswith("grad_"):
                extra[nm] = Gall.get(nm[5:])
            elif nm.startswith("first_"):
                extra[nm] = first_of.get(nm[6:], first)
        with torch.no_grad():
            res = gm(*self._inputs(P, x, meta, self._train_inputs, extra))
        loss_sum.add_(res[0].reshape(loss_sum.shape))
        out = None
        for target, g in zip(self._train_grads, res[1:]):
            if target is None or g is None:
                continue
            if target == "x":
                out = g if dx is None else dx.copy_(g)
            elif target in Gall and Gall[target] is not None and g is not Gall[target]:
                dst = Gall[target]
                if first_of.get(target, first):
                    dst.copy_(g.reshape(dst.shape))
                else:
                    dst.add_(g.reshape(dst.shape).to(dst.dtype))
        return out

    def outputs(self, P, x, meta: BatchMeta, tied: dict | None = None):
        from ..models.decoder import HeadLossStage
        helper = HeadLossStage(self.name, self.cfg, self.block_rows)
        return helper.outputs(P, x, meta, tied)


def _head_training_graph(pairs: gp.StagePairs, stage: StageGraph):
    """The head's joint graph specialised for a training step: the loss tangent is 1, so the
    scaling of the gradients by it disappears, and ``ss::head_loss`` becomes its in-place form
    that creates or accumulates the output-matrix gradient in the stage's buffer."""
    import copy
    joint = copy.deepcopy(pairs.joint)
    g = joint.graph
    phs = [n for n in g.nodes if n.op == "placeholder"]
    names = list(pairs.placeholders)
    primals, tangents = phs[:len(names)], phs[len(names):]
    for p, nm in zip(primals, names):
        p.target = nm
    out_node = next(n for n in g.nodes if n.op == "output")
    outs = list(out_node.args[0])
    grads_of = [nm if (i < len(stage.param_names) and pairs.trainable[i]) else ("x" if nm == "x" else None)
                for i, nm in enumerate(names)]
    last = primals[-1]
    extra_inputs = []
    # ---- head_loss -> head_loss_into
    pending = []
    for n in list(g.nodes):
        if op_name(n) != "ss.head_loss":
            continue
        h, W, targets, weights, block = n.args
        w_name = str(W.target) if W.op == "placeholder" else None
        trainable = w_name is not None and grads_of[names.index(w_name)] is not None
        d = f = None
        if trainable:
            with g.inserting_after(last):
                d = g.placeholder(f"grad_{w_name}")
            with g.inserting_after(d):
                f = g.placeholder(f"first_{w_name}")
            last = f
            extra_inputs += [str(d.target), str(f.target)]
        with g.inserting_before(n):
            new = g.call_function(gp.head_loss_into, (d, h, W, targets, weights, block, f if f is not None else True))
        pending.append((n, new, d))
    # ---- tangent of the loss is the constant one: x * 1 -> x
    for t in tangents:
        for u in list(t.users):
            if op_name(u).startswith("aten.mul"):
                other = u.args[0] if u.args[1] is t else u.args[1]
                if isinstance(other, fx.Node):
                    u.replace_all_uses_with(other)
                    continue
            if op_name(u) in ("aten._to_copy.default", "aten.expand.default", "aten.view.default"):
                for uu in list(u.users):
                    if op_name(uu).startswith("aten.mul"):
                        other = uu.args[0] if uu.args[1] is u else uu.args[1]
                        if isinstance(other, fx.Node):
                            uu.replace_all_uses_with(other)
    # with the scaling gone, the gradient of the output matrix is head_loss's third result behind a
    # chain of detach nodes: it now lives in the destination
    def replace_chain(v: fx.Node, repl: fx.Node):
        for u in list(v.users):
            if op_name(u) in ("aten.detach.default", "aten.alias.default"):
                replace_chain(u, repl)
        v.replace_all_uses_with(repl)
    for n, new, d in pending:
        for u in list(n.users):
            if u.target is not operator.getitem:
                continue
            if u.args[1] in (0, 1):
                with g.inserting_before(u):
                    rep = g.call_function(operator.getitem, (new, u.args[1]))
                u.replace_all_uses_with(rep)
            elif d is not None:
                replace_chain(u, d)
    g.eliminate_dead_code()
    remaining = [t for t in tangents if t.users]
    if remaining:
        raise NotImplementedError("the head's loss gradient is used in a way the training graph does not fold")
    for t in tangents:
        g.erase_node(t)
    out_node.args = (tuple(out_node.args[0]),)
    g.eliminate_dead_code()
    g._codegen = fx.graph.CodeGen()          # plain positional inputs instead of (primals, tangents)
    g.lint()
    joint = fx.GraphModule(torch.nn.Module(), g)
    inputs = [str(n.target) for n in joint.graph.nodes if n.op == "placeholder"]
    return joint, inputs, grads_of


# ------------------------------------------------------------------------ the frontend, end to end
_cache: dict[tuple, tuple] = {}
_cache_lock = threading.Lock()


def _example_batch(T: int, slots: int):
    return (torch.zeros(T, dtype=torch.long, device="meta"), torch.zeros(T, dtype=torch.long, device="meta"),
            torch.zeros(T, dtype=torch.float32, device="meta"), torch.zeros(T, dtype=torch.int32, device="meta"),
            torch.zeros(slots + 1, dtype=torch.int32, device="meta"))


def capture_module(module: nn.Module, example_batch: tuple, partition="auto", policies=gp.DEFAULT_POLICIES,
                   grad_dtype: torch.dtype = torch.bfloat16, model_dtype: torch.dtype = torch.bfloat16):
    """export -> partition -> one ``StagePairs`` per structural contract. Returns
    ``(ExportedStep, {key: StagePairs})``."""
    ep = export_step(module, example_batch)
    exported = partition_export(ep, partition)
    by_key: dict[str, gp.StagePairs] = {}
    last = exported.stages[-1].index
    for st in exported.stages:
        if st.key in by_key:
            continue
        trainable = [bool(exported.parameters[t].requires_grad) for t in st.param_targets]
        grad_dtypes = {}
        for local, target in zip(st.param_names, st.param_targets):
            p = exported.parameters[target]
            grad_dtypes[local] = torch.float32 if p.dim() == 1 else grad_dtype
        pols = policies if 0 < st.index < last else (gp.RECOMPUTE,)
        by_key[st.key] = gp.build_stage_pairs(st, trainable, pols, grad_dtypes)
    return exported, by_key


def supports(cfg, lora=None, expert_parallel=None, objective=None) -> bool:
    """Catalog models the ``nn.Module`` families of :mod:`.modules` cover."""
    plain_objective = objective is None or (getattr(objective, "kind", "cross_entropy") == "cross_entropy"
                                            and not getattr(objective, "moe_balance_coef", 0))
    if lora is not None and cfg.is_moe and lora.routed_experts:
        # ss::moe_experts_lora adapts both banks of frozen experts; other mixes stay on the stage classes
        banks = {"w13", "w2"} & set(lora.targets)
        if (banks and banks != {"w13", "w2"}) or (banks and lora.train_base):
            return False
    return (cfg.family != "regression" and expert_parallel is None and plain_objective
            and not (cfg.is_moe and cfg.router_aux_coef > 0))


def build_graph_stages(cfg, T: int, slots: int, dtype: torch.dtype = torch.bfloat16,
                       grad_dtype: torch.dtype | None = None, head_block_rows: int = 0,
                       module: nn.Module | None = None, chunk_rows: int = 0, lora=None) -> list[Stage]:
    """The stage list of ``cfg`` (or of ``module``) through the graph frontend. ``chunk_rows`` > 0
    runs the token-local regions of every layer stage in row chunks of that many tokens."""
    from .modules import DecoderLM
    block = head_block_rows or 2048
    key = (cfg.to_json() if module is None else id(module), T, slots, str(dtype), str(grad_dtype), block,
           chunk_rows, lora.to_json() if lora is not None else None)
    with _cache_lock:
        hit = _cache.get(str(key))
    if hit is None:
        if module is None:
            with torch.device("meta"):
                module = DecoderLM(cfg, dtype, block, lora)
        hit = capture_module(module, _example_batch(T, slots), grad_dtype=grad_dtype or dtype, model_dtype=dtype)
        if 0 < chunk_rows < T:
            from .chunking import chunk_pairs, peak_intermediate_bytes
            exported, by_key = hit
            inner = {st.key for st in exported.stages[1:-1]} if len(exported.stages) > 2 else set()
            for k in inner:
                if chunk_pairs(by_key[k], T, chunk_rows):
                    by_key[k].intermediate_bytes = min(by_key[k].intermediate_bytes, max(
                        max(peak_intermediate_bytes(p.forward), peak_intermediate_bytes(p.backward))
                        for p in by_key[k].pairs.values()))
        with _cache_lock:
            _cache[str(key)] = hit
    exported, by_key = hit
    stages: list[Stage] = []
    n = len(exported.stages)
    owner: dict[str, tuple[str, str]] = {}          # model parameter -> (stage name, local name)
    for i, st in enumerate(exported.stages):
        specs = _param_specs(st, exported, dtype)
        foreign = {}
        for local, target in zip(st.param_names, st.param_targets):
            if target in owner:
                foreign[local] = owner[target][1]
            else:
                owner[target] = (st.name, local)
        pairs = by_key[st.key]
        if i == 0 and n > 1:
            stages.append(GraphEmbeddingStage(st.name, cfg, st, pairs, specs, foreign))
        elif i == n - 1:
            stages.append(GraphHeadStage(st.name, cfg, st, pairs, specs, foreign, block))
        else:
            stages.append(GraphStage(st.name, cfg, st, pairs, specs, foreign))
            if 0 < chunk_rows < T:
                stages[-1].mixer += f":rows{chunk_rows}"     # chunked and whole forms profile apart
    return stages
