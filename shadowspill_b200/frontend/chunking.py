"""Axis chunking inside a stage: token-local operators run in row chunks.

A stage graph (forward or backward) is cut into *regions* of consecutive operators that are
local in the token axis (each output row depends on the same input rows only): projections,
norms, rotary, SwiGLU, pointwise glue, and the in-place gradient forms that reduce over tokens
(weight-gradient GEMMs, norm-weight gradients). Sequence operators (attention, the gated delta
rule, the causal convolution), the head (which blocks its rows itself) and anything that mixes
rows are barriers. Inside a region the operators are replicated once per chunk of ``chunk_rows``
rows on slices of the region's inputs; values that leave the region are concatenated, reductions
accumulate into their destination (created by the first chunk only). The wide intermediates of
a region (the gate/up projection of an MLP, the fused q/k/v projection) then exist for one chunk
at a time, so a stage's workspace scales with the chunk, not with the microbatch: this is what
makes a single 64K-128K token sequence trainable on one GPU.

Reference: packages/engine/src/shadowspill/pytorch/chunking/transform.py:47 (``chunk_artifact``),
chunking/rules.py (axis and reduction rules), packages/workloads/src/shadowspill_workloads/
policies/text/chunking.py:22,80,133 (``TextAxisChunks``: projection / MLP / head chunks, sequence
mixers as barriers).
"""
from __future__ import annotations

import operator

import torch
from torch import fx

from . import fusion
from . import graph_pairs as gp
from .export import op_name

ROWS, REDUCE, BARRIER = "rows", "reduce", "barrier"

# operator -> positions of the arguments whose rows are the operator's rows (everything else,
# weights first of all, is passed whole, whatever its shape)
_ROW_ARGS_SS = {"ss.linear": (0,), "ss.rmsnorm": (0,), "ss.rope": (0, 1), "ss.swiglu": (0,),
                "ss.swiglu_bwd": (0, 1), "ss.embedding": (0,), "ss.l2norm": (0,), "ss.l2norm_bwd": (0, 1),
                "ss.gated_rmsnorm": (0, 1)}
_POINTWISE = ("aten.add.", "aten.sub.", "aten.mul.", "aten.div.", "aten.neg.", "aten.sigmoid.", "aten.silu.",
              "aten.exp.", "aten._to_copy.", "aten.clone.", "aten.detach.", "aten.alias.", "aten.rsub.",
              "aten.sigmoid_backward.", "aten.softplus.", "aten.softplus_backward.", "aten.where.",
              "aten.tanh.", "aten.zeros_like.", "aten.ones_like.")
_VIEWS = ("aten.view.default", "aten.reshape.default", "aten._unsafe_view.default")
_WRITERS = (gp.gemm_into, gp.rmsnorm_bwd_into, gp.embedding_bwd_into)


def _val(n):
    return n.meta.get("val") if isinstance(n, fx.Node) else None


def _leading(n, T: int) -> bool:
    v = _val(n)
    return isinstance(v, torch.Tensor) and v.dim() >= 1 and v.shape[0] == T


def classify(node: fx.Node, T: int) -> tuple[str, tuple[int, ...]]:
    """How ``node`` behaves when the token axis is cut into row chunks, and which of its
    arguments are cut with it. Cutting is valid whenever every row-aligned operand is cut the
    same way, so the decision is per operator and argument position, never by shape alone."""
    none = (BARRIER, ())
    if node.op != "call_function":
        return none
    name, t, a = op_name(node), node.target, node.args

    def lead(*pos):
        return all(isinstance(a[i], fx.Node) and _leading(a[i], T) for i in pos)
    if t is fusion.rope_in_place:
        return (ROWS, (0, 1)) if (lead(0, 1) and _leading(node, T)) else none
    if t is fusion.add_rmsnorm:
        return (ROWS, (0, 1)) if lead(0, 1) else none      # (sum, y, rstd): all with the rows of the operands
    if t is gp.gemm_into:
        return (REDUCE, (1, 2)) if (a[3] and a[4] and lead(1, 2)) else none
    if t is gp.rmsnorm_bwd_into:
        return (REDUCE, (1, 3, 4)) if lead(1, 3, 4) else none
    if t is gp.embedding_bwd_into:
        return (REDUCE, (1, 2)) if lead(1, 2) else none
    if t is operator.getitem:
        src = a[0]
        ok = isinstance(src, fx.Node) and _leading(node, T) and classify(src, T)[0] != BARRIER
        return (ROWS, (0,)) if ok else none
    if name == "ss.rmsnorm":
        return (ROWS, (0,)) if lead(0) else none            # both outputs have the rows of x
    if name in _ROW_ARGS_SS:
        pos = _ROW_ARGS_SS[name]
        return (ROWS, pos) if (lead(*pos) and _leading(node, T)) else none
    if not name.startswith(("ss.", "aten.")):
        from .operator_rules import rule_of
        declared = rule_of(name)             # an operator of the user's own: its rule names the row arguments
        if declared is not None and declared.row_args is not None:
            pos = declared.row_args
            return (ROWS, pos) if (lead(*pos) and _leading(node, T)) else none
        return none
    if name == "ss.gemm":
        return (ROWS, (0,)) if (not a[2] and lead(0) and _leading(node, T)) else none
    if name.startswith(_POINTWISE):
        out = _val(node)
        if not _leading(node, T):
            return none
        # operands of the output's rank with T rows are aligned row for row; lower ranks broadcast
        pos = tuple(i for i, x in enumerate(a) if isinstance(x, fx.Node) and _leading(x, T)
                    and _val(x).dim() == out.dim())
        same = all(not isinstance(x, fx.Node) or i in pos
                   or (isinstance(_val(x), torch.Tensor) and _val(x).dim() < out.dim())
                   for i, x in enumerate(a))               # a value of unknown shape: do not cut
        return (ROWS, pos) if (pos and same) else none
    if name == "aten.slice.Tensor":
        return (ROWS, (0,)) if (a[1] != 0 and lead(0) and _leading(node, T)) else none
    if name == "aten.slice_backward.default":
        return (ROWS, (0,)) if (a[2] != 0 and lead(0) and _leading(node, T)) else none
    if name in _VIEWS:
        # rows stay rows only if the view keeps the leading dimension apart
        src = _val(a[0])
        keeps = lead(0) and _leading(node, T) and isinstance(src, torch.Tensor)
        return (ROWS, (0,)) if keeps else none
    if name == "aten.cat.default":
        dim = a[1] if len(a) > 1 else 0
        parts = a[0]
        ok = dim != 0 and _leading(node, T) and all(isinstance(x, fx.Node) and _leading(x, T) for x in parts)
        return (ROWS, (0,)) if ok else none
    return none


def _regions(graph: fx.Graph, T: int, min_nodes: int = 2) -> list[list[fx.Node]]:
    """Maximal runs of consecutive chunkable call nodes that contain real work. A node that
    needs a value of the current run whole (not row by row) ends the run."""
    out, run, inside = [], [], set()

    def flush():
        nonlocal run, inside
        if run:
            out.append(run)
        run, inside = [], set()
    for n in graph.nodes:
        kind, pos = classify(n, T) if n.op == "call_function" else (BARRIER, ())
        if kind == BARRIER:
            flush()
            continue
        whole = []
        for i, x in enumerate(n.args):
            if i in pos:
                continue
            whole += [x] if isinstance(x, fx.Node) else [y for y in (x if isinstance(x, (list, tuple)) else ())
                                                        if isinstance(y, fx.Node)]
        if any(x in inside for x in whole):
            flush()                        # start a new run at this node
        run.append(n)
        inside.add(n)
    flush()
    heavy = lambda r: sum(1 for n in r if op_name(n).startswith("ss.") or n.target in _WRITERS) >= min_nodes
    return [r for r in out if heavy(r)]


def chunk_graph(gm: fx.GraphModule, T: int, chunk_rows: int,
                broadcast: set[str] = frozenset()) -> tuple[fx.GraphModule, int]:
    """Returns ``(chunked graph, regions chunked)``. ``T`` is the token count of the stage's
    microbatch, ``broadcast`` the placeholder names that are never cut (parameters, gradient
    destinations); a graph without a region comes back unchanged."""
    if chunk_rows <= 0 or chunk_rows >= T:
        return gm, 0
    del broadcast                           # roles are per operator argument; kept for callers
    bounds = [(r0, min(T, r0 + chunk_rows)) for r0 in range(0, T, chunk_rows)]
    regions = _regions(gm.graph, T)
    if not regions:
        return gm, 0
    first_of = {r[0]: r for r in regions}
    member = {n: i for i, r in enumerate(regions) for n in r}
    g = fx.Graph()
    env: dict[fx.Node, fx.Node] = {}
    done = 0
    for n in gm.graph.nodes:
        if n in member and n not in first_of:
            continue                                      # emitted with its region
        if n not in first_of:
            if n.op == "output":
                g.output(tuple(env[a] if isinstance(a, fx.Node) else a for a in n.args[0]))
            else:
                env[n] = g.node_copy(n, lambda a: env[a])
            continue
        region = first_of[n]
        inside = set(region)
        leaving = [m for m in region if any(u not in inside for u in m.users)]
        # a REDUCE node returns its destination (or row output for rmsnorm_bwd_into: rows)
        chunk_vals: dict[fx.Node, list[fx.Node]] = {m: [] for m in leaving}
        for ci, (r0, r1) in enumerate(bounds):
            local: dict[fx.Node, fx.Node] = {}

            cut: dict[fx.Node, fx.Node] = {}

            def rows(a, _local=local, _cut=cut, _r0=r0, _r1=r1):
                if not isinstance(a, fx.Node):
                    return a
                if a in _local:
                    return _local[a]
                if a not in _cut:
                    _cut[a] = g.call_function(torch.ops.aten.slice.Tensor, (env[a], 0, _r0, _r1))
                return _cut[a]

            def whole(a):
                return env[a] if isinstance(a, fx.Node) else a
            for m in region:
                kind, pos = classify(m, T)
                args = list(m.args)
                name = op_name(m)
                if m.target in _WRITERS and ci > 0:
                    args[-1] = False                       # only the first chunk creates the gradient
                new_args = tuple(fx.node.map_arg(a, rows if i in pos else whole) for i, a in enumerate(args))
                if name in _VIEWS:
                    shape = list(new_args[1])
                    shape[0] = r1 - r0
                    new_args = (new_args[0], shape)
                elif name == "aten.slice_backward.default":
                    shape = list(new_args[1])
                    shape[0] = r1 - r0
                    new_args = (new_args[0], shape) + tuple(new_args[2:])
                local[m] = g.call_function(m.target, new_args, dict(m.kwargs))
                local[m].meta = dict(m.meta)
                if kind == ROWS or m.target is gp.rmsnorm_bwd_into:
                    local[m].meta["ss_rows"] = (r1 - r0) / T
                if m in chunk_vals:
                    chunk_vals[m].append(local[m])
        for m in leaving:
            if classify(m, T)[0] == REDUCE and m.target is not gp.rmsnorm_bwd_into:
                env[m] = chunk_vals[m][-1]                # the destination buffer
            else:
                env[m] = g.call_function(torch.ops.aten.cat.default, (chunk_vals[m], 0))
                env[m].meta = dict(m.meta)
        done += 1
    writers = _WRITERS + (gp.head_loss_into, gp.moe_experts_bwd_into)
    g.eliminate_dead_code(is_impure_node=lambda n: n.op in ("placeholder", "output") or n.target in writers)
    g.lint()
    return fx.GraphModule(torch.nn.Module(), g), done


def chunk_pairs(pairs: gp.StagePairs, T: int, chunk_rows: int) -> int:
    """Chunks the forward and backward graph of every variant in place; returns regions chunked."""
    total = 0
    params = set(pairs.placeholders[:len(pairs.trainable)])
    whole = params | {"grad_" + p for p in params} | {"first"}
    done: dict[int, tuple] = {}                 # variants that keep the same set share their graphs
    for pair in pairs.pairs.values():
        for side in ("forward", "backward"):
            gm = getattr(pair, side)
            if id(gm) not in done:
                done[id(gm)] = chunk_graph(gm, T, chunk_rows, whole)
                total += done[id(gm)][1]
            setattr(pair, side, done[id(gm)][0])
    return total


def peak_intermediate_bytes(gm: fx.GraphModule) -> int:
    """Largest sum of live intermediate bytes over the graph's program order (from the shapes the
    nodes were traced with; chunk copies of a node count as their share of its rows)."""
    last_use: dict[fx.Node, fx.Node] = {}
    for n in gm.graph.nodes:
        for a in n.all_input_nodes:
            last_use[a] = n
    live, peak, size = 0, 0, {}
    frees: dict[fx.Node, list[fx.Node]] = {}
    for v, u in last_use.items():
        frees.setdefault(u, []).append(v)

    def nbytes(n: fx.Node) -> int:
        if n.op != "call_function" or n.target is operator.getitem:
            return 0
        if n.target in (gp.gemm_into, gp.embedding_bwd_into, gp.head_loss_into):
            return 0                                       # returns its destination
        name = op_name(n)
        if name.startswith(("aten.slice.", "aten.view.", "aten.reshape.", "aten.detach.", "aten.alias.")):
            return 0
        v = n.meta.get("val")
        vals = v if isinstance(v, (tuple, list)) else [v]
        b = sum(t.numel() * t.element_size() for t in vals if isinstance(t, torch.Tensor))
        # a chunk copy keeps the full-shape metadata of its original: scale by its row share
        rows = n.meta.get("ss_rows")
        return int(b * rows) if rows else b
    for n in gm.graph.nodes:
        size[n] = nbytes(n)
        live += size[n]
        peak = max(peak, live)
        for v in frees.get(n, []):
            live -= size.get(v, 0)
    return peak
