"""``torch.export`` capture of a training step and its partition into stages.

``export_step`` traces ``module(*batch) -> loss`` strictly (``torch.export.export``, then
functionalisation through ``run_decompositions``) on the meta device, so a model of any size
is captured without allocating it. ``partition_export`` then cuts the flat ATen/``ss`` graph
into stages:

* ``"auto"``   one stage per element of the model's largest ``ModuleList`` (the repeated
               child), a prologue stage for what runs before it and an epilogue stage for
               what runs after it;
* ``"whole"``  the whole step as one stage;
* a ``PartitionPolicy`` whose ``assign_stages(node, module_path) -> int`` names a stage per
               node (stages must be visited in non-decreasing order of data flow).

Each stage becomes an ``fx.GraphModule`` whose placeholders are its parameters, the one
activation that crosses from the previous stage, and the batch fields it reads.

Reference: packages/engine/src/shadowspill/pytorch/capture/export.py:27-126 (strict export and
functionalisation), pytorch/partition/api.py:29 (``partition_export``), partition/policy.py.
"""
from __future__ import annotations

import hashlib
import re
from dataclasses import dataclass, field
from typing import Callable

import torch
from torch import fx, nn

_VIEW_OPS = {"aten.view.default", "aten.reshape.default", "aten._unsafe_view.default",
             "aten.slice.Tensor", "aten.permute.default", "aten.transpose.int", "aten.unsqueeze.default",
             "aten.squeeze.dim", "aten.select.int", "aten.expand.default", "aten.alias.default",
             "aten.detach.default", "aten.t.default"}


def op_name(node: fx.Node) -> str:
    """``"ss.linear"`` / ``"aten.add.Tensor"`` for call_function nodes, ``""`` otherwise."""
    if node.op != "call_function":
        return ""
    t = node.target
    name = getattr(t, "__qualname__", None) or str(t)
    if hasattr(t, "_schema"):
        ns, _, rest = t._schema.name.partition("::")
        return f"{ns}.{rest}" + ("" if ns == "ss" else f".{t._overloadname}")
    return name


def is_view(node: fx.Node) -> bool:
    return op_name(node) in _VIEW_OPS


@dataclass
class PartitionPolicy:
    """``assign_stages(node, module_path) -> stage index`` for every compute node; ``names`` gives
    the stages their names (default ``stage<i>``)."""
    assign_stages: Callable[[fx.Node, str], int]
    names: Callable[[int], str] | None = None


@dataclass
class StageGraph:
    name: str
    index: int
    gm: fx.GraphModule                    # placeholders: parameters, boundary input, batch fields
    param_names: list[str]                # names local to the stage ("wqkv")
    param_targets: list[str]              # names in the model ("layers.0.wqkv")
    boundary_in: str | None               # placeholder that carries the previous stage's output
    batch_fields: list[str]               # user inputs this stage reads, in placeholder order
    n_outputs: int
    key: str = ""                         # structural key: equal keys = one compiled pair serves all

    @property
    def placeholders(self) -> list[str]:
        return self.param_names + ([self.boundary_in] if self.boundary_in else []) + self.batch_fields


@dataclass
class ExportedStep:
    program: "torch.export.ExportedProgram"
    stages: list[StageGraph]
    parameters: dict[str, nn.Parameter]   # model name -> parameter (meta device)
    batch_fields: list[str]
    policy: str = "auto"
    boundary_shapes: list[tuple] = field(default_factory=list)


def export_step(module: nn.Module, example_batch: tuple, *, strict: bool = True):
    """Strict export + functionalisation of ``module(*example_batch)``. Tensors may live on the
    meta device; metadata assertions that pin the tracing device are removed."""
    ep = torch.export.export(module, tuple(example_batch), strict=strict)
    ep = ep.run_decompositions({})
    g = ep.graph_module.graph
    for node in list(g.nodes):
        if node.op == "call_function" and "_assert_tensor_metadata" in str(node.target):
            g.erase_node(node)
    for node in g.nodes:
        if node.op == "call_function" and "device" in node.kwargs:
            raise ValueError(f"{node.name}: the model creates a tensor on a fixed device "
                             f"({node.kwargs['device']}); build it from an input instead")
    ep.graph_module.recompile()
    return ep


def _module_path(node: fx.Node) -> str:
    stack = node.meta.get("nn_module_stack") or {}
    paths = [v[0] for v in stack.values()]
    return paths[-1] if paths else ""


def _repeated_container(gm: fx.GraphModule) -> str | None:
    """The module path prefix ``p`` with the most distinct children ``p.<int>`` seen in the graph."""
    seen: dict[str, set[int]] = {}
    for node in gm.graph.nodes:
        for v in (node.meta.get("nn_module_stack") or {}).values():
            m = re.match(r"^(.*)\.(\d+)$", v[0])
            if m:
                seen.setdefault(m.group(1), set()).add(int(m.group(2)))
    if not seen:
        return None
    return max(seen.items(), key=lambda kv: (len(kv[1]), -len(kv[0])))[0]


def _auto_policy(gm: fx.GraphModule) -> tuple[PartitionPolicy, int]:
    container = _repeated_container(gm)
    if container is None:
        return PartitionPolicy(lambda n, p: 0, lambda i: "step"), 1
    pat = re.compile("^" + re.escape(container) + r"\.(\d+)(\.|$)")
    indices = set()
    for node in gm.graph.nodes:
        for v in (node.meta.get("nn_module_stack") or {}).values():
            m = pat.match(v[0])
            if m:
                indices.add(int(m.group(1)))
    n = max(indices) + 1
    state = {"entered": False}

    def assign(node: fx.Node, path: str) -> int:
        for v in (node.meta.get("nn_module_stack") or {}).values():
            m = pat.match(v[0])
            if m:
                state["entered"] = True
                return 1 + int(m.group(1))
        return n + 1 if state["entered"] else 0

    def name(i: int) -> str:
        if i == 0:
            return "embed"
        if i == n + 1:
            return "head"
        return f"layer{i - 1}"
    return PartitionPolicy(assign, name), n + 2


def partition_export(ep, policy: "str | PartitionPolicy" = "auto") -> ExportedStep:
    gm = ep.graph_module
    sig = ep.graph_signature
    param_of = dict(sig.inputs_to_parameters)            # placeholder name -> model name
    user_inputs = list(sig.user_inputs)
    if sig.inputs_to_buffers:
        raise ValueError("models with registered buffers are not supported: pass them as inputs")
    if policy == "whole":
        pol, n_stages = PartitionPolicy(lambda n, p: 0, lambda i: "step"), 1
    elif policy == "auto":
        pol, n_stages = _auto_policy(gm)
    elif isinstance(policy, PartitionPolicy):
        pol, n_stages = policy, 0
    else:
        raise ValueError(f"unknown partition policy {policy!r}")

    # ---- stage of every compute node (in graph order; getitem and friends follow their producer)
    stage_of: dict[fx.Node, int] = {}
    last = 0
    for node in gm.graph.nodes:
        if node.op != "call_function":
            continue
        if node.meta.get("nn_module_stack") is None and node.args and isinstance(node.args[0], fx.Node) \
                and node.args[0] in stage_of:
            s = stage_of[node.args[0]]
        else:
            s = int(pol.assign_stages(node, _module_path(node)))
        if s < last:
            # a value may only flow forward: pull the straggler up to the running stage
            s = last
        stage_of[node] = s
        last = max(last, s)
    n_stages = max(n_stages, last + 1)
    out_node = next(n for n in gm.graph.nodes if n.op == "output")
    final_values = [a for a in out_node.args[0] if isinstance(a, fx.Node)]

    stages: list[StageGraph] = []
    boundary_shapes = []
    for si in range(n_stages):
        nodes = [n for n in gm.graph.nodes if stage_of.get(n) == si]
        if not nodes:
            continue
        g = fx.Graph()
        env: dict[fx.Node, fx.Node] = {}
        params, batch, boundary = [], [], []
        needed: list[fx.Node] = []
        for n in nodes:
            for a in n.all_input_nodes:
                if stage_of.get(a) != si and a not in needed:
                    needed.append(a)
        for a in needed:
            if a.op == "placeholder" and a.name in param_of:
                params.append(a)
            elif a.op == "placeholder":
                batch.append(a)
            else:
                boundary.append(a)
        if len(boundary) > 1 or (boundary and stage_of[boundary[0]] != stages[-1].index):
            raise ValueError(f"stage {si} reads {[b.name for b in boundary]} from earlier stages: "
                             "exactly one activation may cross a stage boundary")
        # placeholders in a canonical order: parameters (model order), boundary, batch fields
        # (the model's registration order, not the order of first use that the export signature has:
        # seed-only initialisation draws parameters in this order, whichever frontend built the stage)
        registered = {target: i for i, target in enumerate(ep.state_dict)}
        order = {name: (registered.get(target, len(registered)), i)
                 for i, (name, target) in enumerate(param_of.items())}
        params.sort(key=lambda a: order[a.name])
        batch.sort(key=lambda a: user_inputs.index(a.name))
        name = pol.names(si) if pol.names else f"stage{si}"
        local = _local_names([param_of[a.name] for a in params])
        for a, nm in zip(params, local):
            env[a] = g.placeholder(nm)
            env[a].meta = dict(a.meta)
        if boundary:
            env[boundary[0]] = g.placeholder("x")
            env[boundary[0]].meta = dict(boundary[0].meta)
        for a in batch:
            env[a] = g.placeholder(a.name)
            env[a].meta = dict(a.meta)
        for n in nodes:
            env[n] = g.node_copy(n, lambda a: env[a])
        users_outside = [n for n in nodes if any(stage_of.get(u) not in (si, None) for u in n.users)
                         or n in final_values]
        if len(users_outside) != 1:
            raise ValueError(f"stage {si} ({name}) has {len(users_outside)} values leaving it: "
                             "a stage must produce exactly one activation (or the loss)")
        g.output((env[users_outside[0]],))
        sgm = fx.GraphModule(torch.nn.Module(), g)
        val = users_outside[0].meta.get("val")
        boundary_shapes.append(tuple(val.shape) if val is not None else ())
        code = canonical_text(sgm.graph)
        key = hashlib.sha256((code + "|" + "|".join(
            f"{nm}:{tuple(a.meta['val'].shape)}:{a.meta['val'].dtype}" for a, nm in zip(params, local)))
            .encode()).hexdigest()[:16]
        stages.append(StageGraph(name, si, sgm, local, [param_of[a.name] for a in params],
                                 "x" if boundary else None, [a.name for a in batch], 1, key))
    parameters = {}
    sd = ep.state_dict
    for ph, target in param_of.items():
        parameters[target] = sd[target]
    return ExportedStep(ep, stages, parameters, user_inputs,
                        policy if isinstance(policy, str) else "policy", boundary_shapes)


def canonical_text(graph: fx.Graph) -> str:
    """The graph as text with nodes numbered in order: equal for stages that differ only in the
    names the exporter gave their nodes (layer 0 and layer 7 of one model)."""
    index = {n: i for i, n in enumerate(graph.nodes)}

    def ref(a):
        if isinstance(a, fx.Node):
            return f"%{index[a]}"
        if isinstance(a, (tuple, list)):
            return "(" + ",".join(ref(x) for x in a) + ")"
        return repr(a)
    lines = []
    for n in graph.nodes:
        target = n.target if n.op == "placeholder" else (op_name(n) or str(n.target))
        if n.op == "placeholder":
            val = n.meta.get("val")
            target = f"{target}:{tuple(val.shape)}:{val.dtype}" if val is not None else target
        kw = ",".join(f"{k}={ref(v)}" for k, v in sorted(n.kwargs.items()))
        lines.append(f"{index[n]} {n.op} {target} {ref(n.args)} {kw}")
    return "\n".join(lines)


def _local_names(targets: list[str]) -> list[str]:
    """Last path component of each parameter name; a clash inside one stage (a stage of several
    layers) keeps the parents below the stage's own module, so that two stages of the same structure
    still name their parameters alike."""
    short = [t.split(".")[-1] for t in targets]
    parts = [t.split(".") for t in targets]
    common = 0
    while parts and all(len(p) > common + 1 for p in parts) and len({p[common] for p in parts}) == 1:
        common += 1
    while common > 0 and any(p[common][:1].isdigit() for p in parts):
        common -= 1                          # a name must not start with a child's number
    rel = ["_".join(p[common:]) for p in parts]
    return [r if short.count(s_) > 1 else s_ for r, s_ in zip(rel, short)]
