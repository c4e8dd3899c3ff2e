"""Save / recompute graph pairs of a stage, derived from its AOTAutograd joint graph.

For every structural contract (stages with equal ``StageGraph.key`` share one) the joint
forward+backward graph is traced once on meta tensors (``aot_export_joint_simple``). A
*retention policy* then decides which forward values the forward graph hands to the
backward graph; everything else the backward graph needs is recomputed inside it from the
stage's inputs:

* ``recompute``        keeps nothing (budget 0.0 of the reference's min-cut partitioner);
* ``save``             keeps every forward value the backward pass reads, except values a
                       memory-bound operator can rebuild from what is kept anyway (the
                       arithmetic-intensity classing of the reference's retention, budget 1.0);
* rule-based policies  (``save_attention``) keep the outputs and the tensor inputs of the
                       named operators only.

A value that is a view is kept through its base, so q, k and v views of one fused projection
are stored once. Finally the gradient-destination pass rewrites the operators that produce
parameter gradients into their ``*_into`` forms, which create or accumulate the gradient in the
stage's gradient buffer in place.

Reference: packages/engine/src/shadowspill/pytorch/graph_pairs/build.py:53
(``build_default_graph_pairs``), pytorch/capture/retention.py:188,440 (``RetentionPolicy``,
the min-cut ``partition_function``), pytorch/capture/gradients/destinations.py.
"""
from __future__ import annotations

import operator
import os
from dataclasses import dataclass, field

import torch
from torch import fx

from ..ops import functional as F
from . import ops as ss_ops
from .export import StageGraph, is_view, op_name


# ------------------------------------------------------------------------ policies
@dataclass(frozen=True)
class RetentionRule:
    op: str                      # "ss.attention"
    keep: str = "outputs"        # "outputs" | "inputs"


@dataclass(frozen=True)
class RetentionPolicy:
    name: str
    mode: str = "rules"          # "all" | "none" | "rules"
    rules: tuple[RetentionRule, ...] = ()
    drop_memory_bound: bool = True


RECOMPUTE = RetentionPolicy("recompute", "none")
SAVE = RetentionPolicy("save", "all")
SAVE_ATTENTION = RetentionPolicy("save_attention", "rules", (
    RetentionRule("ss.attention", "outputs"), RetentionRule("ss.attention", "inputs"),
    RetentionRule("ss.gated_delta_rule", "outputs"), RetentionRule("ss.gated_delta_rule", "inputs")))
# also keeps the gate/up projection: the backward pass then redoes only the small output
# projection and the elementwise pieces
SAVE_ATTENTION_GU = RetentionPolicy("save_attention_gu", "rules",
                                    SAVE_ATTENTION.rules + (RetentionRule("ss.swiglu", "inputs"),))
DEFAULT_POLICIES = (RECOMPUTE, SAVE_ATTENTION, SAVE_ATTENTION_GU, SAVE)


@dataclass
class SavedValue:
    name: str
    shape: tuple[int, ...]
    dtype: torch.dtype


@dataclass
class GraphPair:
    """One variant of one stage contract."""
    variant: str
    forward: fx.GraphModule      # (params..., x?, batch...) -> (y, *saved)
    backward: fx.GraphModule     # see ``backward_inputs``
    saved: list[SavedValue]
    backward_inputs: list[str]   # placeholder names, in order
    grad_outputs: list[str | None]   # per backward output: parameter name, "x", or None
    in_place: set[str] = field(default_factory=set)   # parameters whose gradient the graph writes itself


@dataclass
class StagePairs:
    key: str
    joint: fx.GraphModule
    pairs: dict[str, GraphPair]
    placeholders: list[str]      # forward placeholder names (params, x, batch)
    trainable: list[bool]        # per parameter
    flops_linear: float          # 2*M*N*K summed over the forward's GEMM-shaped operators
    intermediate_bytes: int      # bytes of every forward intermediate (an upper bound on workspace)


# ------------------------------------------------------------------------ joint graph
def _meta_like(val, requires_grad: bool):
    t = torch.empty(val.shape, dtype=val.dtype, device="meta")
    return t.requires_grad_(requires_grad) if (requires_grad and t.is_floating_point()) else t


def joint_graph(stage: StageGraph, trainable: list[bool]) -> fx.GraphModule:
    """(primals..., tangents...) -> (outputs..., one gradient per primal or None)."""
    from torch._functorch.aot_autograd import aot_export_joint_simple
    phs = [n for n in stage.gm.graph.nodes if n.op == "placeholder"]
    n_params = len(stage.param_names)
    args = []
    for i, ph in enumerate(phs):
        val = ph.meta["val"]
        if i < n_params:
            args.append(_meta_like(val, trainable[i]))
        else:
            args.append(_meta_like(val, ph.name == "x"))
    gm = stage.gm

    def fn(*a):
        return gm(*a)
    joint = aot_export_joint_simple(fn, args, trace_joint=True)
    for node in list(joint.graph.nodes):
        if node.op == "call_function" and "_assert_tensor_metadata" in str(node.target):
            joint.graph.erase_node(node)
        elif node.op == "call_function" and "device" in node.kwargs:
            # the trace ran on the meta device; a cast keeps its input's device when none is named
            if not node.all_input_nodes:
                raise ValueError(f"{node.name}: the backward pass creates a tensor on a fixed device")
            node.kwargs = {k: v for k, v in node.kwargs.items() if k not in ("device", "layout")}
    joint.graph.eliminate_dead_code()
    joint.recompile()
    return joint


def _placeholders(g: fx.Graph) -> list[fx.Node]:
    return [n for n in g.nodes if n.op == "placeholder"]


def _forward_nodes(joint: fx.GraphModule, n_primals: int) -> set[fx.Node]:
    """Compute nodes that do not depend on any tangent."""
    phs = _placeholders(joint.graph)
    tainted = set(phs[n_primals:])
    fwd = set()
    for n in joint.graph.nodes:
        if n.op != "call_function":
            continue
        if any(a in tainted for a in n.all_input_nodes):
            tainted.add(n)
        else:
            fwd.add(n)
    return fwd


def _base(node: fx.Node) -> fx.Node:
    while node.op == "call_function" and is_view(node) and isinstance(node.args[0], fx.Node):
        node = node.args[0]
    return node


def _is_memory_bound(node: fx.Node) -> bool:
    name = op_name(node)
    if name.startswith("ss."):
        return name in ss_ops.MEMORY_BOUND
    if node.target is operator.getitem:
        return _is_memory_bound(node.args[0])
    from .operator_rules import rule_of
    declared = rule_of(name)                 # an operator of the user's own, with a declared rule
    if declared is not None:
        return declared.cost == "memory"
    return name.startswith("aten.")          # pointwise / view / cast glue


def choose_retained(joint: fx.GraphModule, n_primals: int, n_outputs: int,
                    policy: RetentionPolicy) -> list[fx.Node]:
    """Forward values (nodes of the joint graph) the forward pass keeps for the backward pass."""
    if policy.mode == "none":
        return []
    fwd = _forward_nodes(joint, n_primals)
    phs = set(_placeholders(joint.graph))
    out_node = next(n for n in joint.graph.nodes if n.op == "output")
    needed: list[fx.Node] = []           # forward values read by backward nodes (through their bases)

    def want(v: fx.Node):
        b = _base(v)
        if b in fwd and b not in needed:
            val = b.meta.get("val")
            if isinstance(val, torch.Tensor):
                needed.append(b)
    if policy.mode == "all":
        for n in joint.graph.nodes:
            if n.op == "call_function" and n not in fwd:
                for a in n.all_input_nodes:
                    if a in fwd:
                        want(a)
    else:
        for n in joint.graph.nodes:
            if n.op != "call_function":
                continue
            for rule in policy.rules:
                if op_name(n) != rule.op or n not in fwd:
                    continue
                if rule.keep == "outputs":
                    for u in n.users:
                        if u.target is operator.getitem and isinstance(u.meta.get("val"), torch.Tensor):
                            if any(x not in fwd for x in u.users) or True:
                                want(u)
                    if isinstance(n.meta.get("val"), torch.Tensor):
                        want(n)
                else:
                    for a in n.all_input_nodes:
                        if a not in phs and isinstance(a.meta.get("val"), torch.Tensor) \
                                and a.meta["val"].is_floating_point():
                            want(a)
        # a rule may name values the backward pass never reads: keep only what it does read
        used = set()
        for n in joint.graph.nodes:
            if n.op == "call_function" and n not in fwd:
                for a in n.all_input_nodes:
                    used.add(_base(a))
        needed = [v for v in needed if v in used or any(_base(u) is v and u in used for u in v.users)]
    order = {n: i for i, n in enumerate(joint.graph.nodes)}
    needed.sort(key=lambda n: order[n])
    if not policy.drop_memory_bound or policy.mode != "all":
        return needed
    kept: list[fx.Node] = []
    available = set(phs)

    def rebuildable(v: fx.Node, depth: int = 0) -> bool:
        """Can ``v`` be recomputed from kept values and inputs through memory-bound operators only?"""
        if v in available:
            return True
        if v.op != "call_function" or not _is_memory_bound(v) or depth > 6:
            return False
        return all(rebuildable(a, depth + 1) for a in v.all_input_nodes)
    for v in needed:
        if rebuildable(v):
            continue
        kept.append(v)
        available.add(v)
    return kept


# ------------------------------------------------------------------------ split
def split_joint(joint: fx.GraphModule, n_primals: int, n_outputs: int, retained: list[fx.Node],
                names: list[str]) -> tuple[fx.GraphModule, fx.GraphModule, list[SavedValue], list[str]]:
    """Forward graph ``primals -> (outputs, retained)`` and backward graph
    ``(primals it needs, retained, tangents) -> gradients``."""
    phs = _placeholders(joint.graph)
    primals, tangents = phs[:n_primals], phs[n_primals:]
    out_node = next(n for n in joint.graph.nodes if n.op == "output")
    outs = list(out_node.args[0])
    fwd_outs, grads = outs[:n_outputs], outs[n_outputs:]

    # ---- forward
    fg = fx.Graph()
    env: dict[fx.Node, fx.Node] = {}
    for p, nm in zip(primals, names):
        env[p] = fg.placeholder(nm)
        env[p].meta = dict(p.meta)
    need = set()
    stack = [v for v in fwd_outs + retained if isinstance(v, fx.Node)]
    while stack:
        v = stack.pop()
        if v in need or v.op == "placeholder":
            continue
        need.add(v)
        stack.extend(v.all_input_nodes)
    for n in joint.graph.nodes:
        if n in need:
            env[n] = fg.node_copy(n, lambda a: env[a])
    fg.output(tuple(env[v] for v in fwd_outs) + tuple(env[v] for v in retained))
    fwd = fx.GraphModule(torch.nn.Module(), fg)

    # ---- backward
    bg = fx.Graph()
    benv: dict[fx.Node, fx.Node] = {}
    need = set()
    stack = [v for v in grads if isinstance(v, fx.Node)]
    retained_set = set(retained)
    while stack:
        v = stack.pop()
        if v in need:
            continue
        need.add(v)
        if v in retained_set or v.op == "placeholder":
            continue
        stack.extend(v.all_input_nodes)
    b_inputs = []
    for p, nm in zip(primals, names):
        if p in need:
            benv[p] = bg.placeholder(nm)
            benv[p].meta = dict(p.meta)
            b_inputs.append(nm)
    saved = []
    for i, v in enumerate(retained):
        nm = f"saved_{i}_{v.name}"
        benv[v] = bg.placeholder(nm)
        benv[v].meta = dict(v.meta)
        val = v.meta["val"]
        saved.append(SavedValue(nm, tuple(val.shape), val.dtype))
        b_inputs.append(nm)
    for i, t in enumerate(tangents):
        nm = f"tangent_{i}"
        benv[t] = bg.placeholder(nm)
        benv[t].meta = dict(t.meta)
        b_inputs.append(nm)
    for n in joint.graph.nodes:
        if n in need and n not in benv and n.op == "call_function":
            benv[n] = bg.node_copy(n, lambda a: benv[a])
    bg.output(tuple(benv[v] if isinstance(v, fx.Node) else None for v in grads))
    bwd = fx.GraphModule(torch.nn.Module(), bg)
    return fwd, bwd, saved, b_inputs


# ------------------------------------------------------------------------ gradient destinations
def gemm_into(dst: torch.Tensor, a: torch.Tensor, b: torch.Tensor, a_mn: bool, b_mn: bool, first: bool):
    """``dst (+)= op(a) op(b)``: the weight-gradient GEMM with its accumulation in the epilogue
    (the reference's ``shadowspill::accumulate_matmul_``, pytorch/operations.py:15)."""
    a = a if a.stride(-1) == 1 else a.contiguous()
    b = b if b.stride(-1) == 1 else b.contiguous()
    F.gemm(a, b, a_mn=a_mn, b_mn=b_mn, out=dst, accumulate=not first)
    return dst


def rmsnorm_bwd_into(dst: torch.Tensor, x, w, gy, rstd, zero_centered: bool, first: bool):
    if first:
        dst.zero_()
    return F.rmsnorm_bwd(x.contiguous(), w, gy.contiguous(), rstd, dst, zero_centered)


def embedding_bwd_into(dst: torch.Tensor, ids, g, first: bool):
    if first:
        dst.zero_()
    F.embedding_bwd(ids, g.contiguous(), dst)
    return dst


def head_loss_into(dst: torch.Tensor | None, h, W, targets, weights, block_rows: int, first: bool):
    """``ss::head_loss`` with the head-weight gradient created or accumulated in ``dst``."""
    return ss_ops.head_loss_run(h.contiguous(), W, targets, weights, block_rows, dst, not first)


def moe_experts_bwd_into(dst13: torch.Tensor, dst2: torch.Tensor, h, logits, w13, w2, gy, k: int, renorm: bool,
                         first: bool):
    """``ss::moe_experts_bwd`` with both bank gradients created in or added to their destinations
    by the grouped weight-gradient GEMMs; returns ``(dh, dlogits)``."""
    return ss_ops.moe_bwd_run(h, logits, w13, w2, gy, k, renorm, dst13, dst2, first)


def _strip_cast(node: fx.Node) -> fx.Node:
    """Looks through the dtype cast autograd appends to a gradient (fp32 -> parameter dtype)."""
    if node.op == "call_function" and op_name(node) == "aten._to_copy.default" and len(node.users) == 1:
        return node.args[0]
    return node


def rewrite_destinations(bwd: fx.GraphModule, param_grads: dict[int, str], dest_dtypes: dict[str, torch.dtype],
                         scale_nodes: tuple[str, ...] = ()) -> set[str]:
    """For every backward output ``i`` that is the gradient of parameter ``param_grads[i]``: when
    its producer has an in-place form, feed it the destination (new placeholders ``grad_<name>``
    and ``first``) and make the output the destination itself. Returns the parameters handled."""
    g = bwd.graph
    if not param_grads:                  # a stage whose parameters are all frozen
        return set()
    out_node = next(n for n in g.nodes if n.op == "output")
    outs = list(out_node.args[0])
    last_ph = [n for n in g.nodes if n.op == "placeholder"][-1]
    done: set[str] = set()
    first_ph = None

    def dest(name: str) -> tuple[fx.Node, fx.Node]:
        nonlocal first_ph, last_ph
        with g.inserting_after(last_ph):
            d = g.placeholder(f"grad_{name}")
            last_ph = d
        if first_ph is None:
            with g.inserting_after(last_ph):
                first_ph = g.placeholder("first")
            last_ph = first_ph
        return d, first_ph
    for i, name in param_grads.items():
        v = outs[i]
        if not isinstance(v, fx.Node):
            continue
        src = _strip_cast(v) if dest_dtypes.get(name) == torch.float32 else v
        prod = src
        if prod.op != "call_function" or len(prod.users) != 1:
            if not (prod.target is operator.getitem):
                continue
        kind = op_name(prod)
        if kind == "ss.gemm" and len(prod.users) == 1:
            a, b, a_mn, b_mn = prod.args
            d, f = dest(name)
            with g.inserting_before(prod):
                new = g.call_function(gemm_into, (d, a, b, a_mn, b_mn, f))
            new.meta["val"] = d.meta["val"] = prod.meta.get("val")
        elif kind == "ss.embedding_bwd" and len(prod.users) == 1:
            ids, gy, _rows = prod.args
            d, f = dest(name)
            with g.inserting_before(prod):
                new = g.call_function(embedding_bwd_into, (d, ids, gy, f))
            new.meta["val"] = d.meta["val"] = prod.meta.get("val")
        elif prod.target is operator.getitem and op_name(prod.args[0]) == "ss.rmsnorm_bwd" \
                and prod.args[1] == 1 and dest_dtypes.get(name) == torch.float32:
            call = prod.args[0]
            x, w, gy, rstd, zc = call.args
            d, f = dest(name)
            with g.inserting_before(call):
                dx = g.call_function(rmsnorm_bwd_into, (d, x, w, gy, rstd, zc, f))
            dx.meta["val"] = x.meta.get("val") if isinstance(x, fx.Node) else None
            d.meta["val"] = prod.meta.get("val")
            for u in list(call.users):
                if u.target is operator.getitem and u.args[1] == 0:
                    u.replace_all_uses_with(dx)
            new = d
        else:
            continue
        outs[i] = new if new is not None else d
        done.add(name)
    # routed experts: one call produces both bank gradients; rewrite when both are destinations
    for call in [n for n in g.nodes if n.op == "call_function" and op_name(n) == "ss.moe_experts_bwd"]:
        items = {u.args[1]: u for u in call.users if u.target is operator.getitem}
        slots = {}
        for i, name in param_grads.items():
            v = outs[i]
            if isinstance(v, fx.Node) and name not in done:
                src = _strip_cast(v)
                for which in (2, 3):
                    if items.get(which) is src and (src is v or len(src.users) == 1):
                        slots[which] = (i, name)
        if set(slots) != {2, 3}:
            continue
        (i13, n13), (i2, n2) = slots[2], slots[3]
        d13, f = dest(n13)
        d2, _ = dest(n2)
        d13.meta["val"], d2.meta["val"] = items[2].meta.get("val"), items[3].meta.get("val")
        with g.inserting_before(call):
            new = g.call_function(moe_experts_bwd_into, (d13, d2, *call.args, f))
            dh = g.call_function(operator.getitem, (new, 0))
            dl = g.call_function(operator.getitem, (new, 1))
        dh.meta["val"] = items[0].meta.get("val") if 0 in items else None
        dl.meta["val"] = items[1].meta.get("val") if 1 in items else None
        if 0 in items:
            items[0].replace_all_uses_with(dh)
        if 1 in items:
            items[1].replace_all_uses_with(dl)
        outs[i13], outs[i2] = d13, d2
        done.update((n13, n2))
    out_node.args = (tuple(outs),)
    g.eliminate_dead_code()
    bwd.recompile()
    return done


# ------------------------------------------------------------------------ driver
def build_stage_pairs(stage: StageGraph, trainable: list[bool], policies=DEFAULT_POLICIES,
                      grad_dtypes: dict[str, torch.dtype] | None = None) -> StagePairs:
    """Joint graph of one stage contract and one ``GraphPair`` per retention policy."""
    joint = joint_graph(stage, trainable)
    names = stage.placeholders
    n_primals = len(names)
    pairs: dict[str, GraphPair] = {}
    seen_sets: dict[tuple, str] = {}
    for pol in policies:
        retained = choose_retained(joint, n_primals, 1, pol)
        sig = tuple(v.name for v in retained)
        if sig in seen_sets and pol.mode == "rules":
            # the rules select nothing new for this stage kind: the name stays usable in a
            # selection and means the pair that already keeps exactly this set
            first = pairs[seen_sets[sig]]
            pairs[pol.name] = GraphPair(pol.name, first.forward, first.backward, first.saved,
                                        first.backward_inputs, first.grad_outputs, first.in_place)
            continue
        seen_sets[sig] = pol.name
        fwd, bwd, saved, b_inputs = split_joint(joint, n_primals, 1, retained, names)
        grad_outputs: list[str | None] = []
        param_grads: dict[int, str] = {}
        for i, nm in enumerate(names):
            if i < len(stage.param_names):
                grad_outputs.append(nm if trainable[i] else None)
                if trainable[i]:
                    param_grads[i] = nm
            else:
                grad_outputs.append("x" if nm == "x" else None)
        in_place = rewrite_destinations(bwd, param_grads, grad_dtypes or {})
        if os.environ.get("SS_GRAPH_FUSION", "1") != "0":
            from .fusion import fuse_graph
            fuse_graph(fwd)
            fuse_graph(bwd)
        b_inputs = [str(n.target) for n in bwd.graph.nodes if n.op == "placeholder"]
        pairs[pol.name] = GraphPair(pol.name, fwd, bwd, saved, b_inputs, grad_outputs, in_place)
    flops, inter = 0.0, 0
    for n in stage.gm.graph.nodes:
        val = n.meta.get("val")
        if n.op == "call_function" and isinstance(val, torch.Tensor) and not is_view(n):
            inter += val.numel() * val.element_size()
        if op_name(n) == "ss.linear":
            x, w = n.args[0].meta["val"], n.args[1].meta["val"]
            flops += 2.0 * x.shape[0] * w.shape[0] * w.shape[1]
        elif op_name(n) == "ss.head_loss":
            x, w = n.args[0].meta["val"], n.args[1].meta["val"]
            flops += 2.0 * x.shape[0] * w.shape[0] * w.shape[1]
    return StagePairs(stage.key, joint, pairs, names, trainable, flops, inter)
