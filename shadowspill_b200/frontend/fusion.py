"""Graph rewrites that give the exported stage graphs the fused forms of the hand-written stages.

AOTAutograd produces functional graphs: every operator returns a new tensor, a rotary embedding
copies its input first, a residual add is its own kernel, and the gradient of three column slices
of one projection arrives as three zero-filled full-width tensors added together. The hand-written
stage classes avoid all of that with in-place kernels. These rewrites recover it on the graphs,
where it is provably safe:

  rope in place          ``ss.rope(x)`` whose input is a fresh intermediate with no other user runs
                         the rotary kernel on that buffer instead of on a copy
  add + RMSNorm          ``ss.rmsnorm(aten.add(a, b))`` where one operand is a fresh intermediate
                         with no other user: one kernel adds into that buffer, normalises, and
                         yields the sum for the residual stream (the kernel's ``delta`` input)
  slice gradients        ``slice_backward(a) + slice_backward(b) + ...`` over disjoint column ranges
                         that tile the full width becomes one concatenation

A value is *fresh* when a non-view operator of this graph produced it (never a graph input, a saved
value or a view of either), so writing into it cannot be seen by anything but its single user.

Reference: the fused operators of the reference's model code (packages/workloads/src/
shadowspill_workloads/models/shared/decoder.py:251-295: residual add folded into the norm, rotary
applied in place on the projection output).
"""
from __future__ import annotations

import operator

import torch
from torch import fx

from ..ops import functional as F
from .export import is_view, op_name


# ------------------------------------------------------------------------ fused forms (graph targets)
def rope_in_place(x: torch.Tensor, positions, heads: int, dh: int, rot: int, theta: float, inverse: bool):
    x2 = x if x.dim() == 2 else x.view(x.shape[0], -1)
    if x2.stride(-1) != 1:
        out = x2.contiguous()
        F.rope_(out, positions, col0=0, heads=heads, dh=dh, rot=rot, theta=theta, inverse=inverse)
        return out.view(x.shape)
    F.rope_(x2, positions, col0=0, heads=heads, dh=dh, rot=rot, theta=theta, inverse=inverse)
    return x


def add_rmsnorm(acc: torch.Tensor, other: torch.Tensor, w, eps: float, zero_centered: bool):
    """``acc += other`` in place, then RMSNorm of the sum: ``(sum, y, rstd)``."""
    if not acc.is_contiguous():
        acc = acc.contiguous()
    y, rstd = F.rmsnorm_fwd(acc, w, eps, zero_centered, delta=other.contiguous())
    return acc, y, rstd


FUSED_TARGETS = (rope_in_place, add_rmsnorm)


# ------------------------------------------------------------------------ analysis
_FRESH_ATEN = ("aten.add.", "aten.sub.", "aten.mul.", "aten.div.", "aten.cat.", "aten._to_copy.", "aten.clone.",
               "aten.sigmoid.", "aten.neg.", "aten.exp.", "aten.slice_backward.")


def _fresh(n) -> bool:
    """Produced by a non-view operator of this graph, as a tensor of its own."""
    if not isinstance(n, fx.Node) or n.op != "call_function" or is_view(n) or n.target is operator.getitem:
        return False
    name = op_name(n)
    if name.startswith("ss."):
        return name in ("ss.linear", "ss.gemm", "ss.swiglu", "ss.swiglu_bwd", "ss.embedding")
    return name.startswith(_FRESH_ATEN)


def _single_use(n: fx.Node) -> bool:
    return len(n.users) == 1


def _before(a: fx.Node, b: fx.Node) -> bool:
    for n in a.graph.nodes:
        if n is a:
            return True
        if n is b:
            return False
    return False


# ------------------------------------------------------------------------ rewrites
def _rope(g: fx.Graph) -> int:
    done = 0
    for n in list(g.nodes):
        if op_name(n) != "ss.rope":
            continue
        x = n.args[0]
        if _fresh(x) and _single_use(x):
            with g.inserting_before(n):
                new = g.call_function(rope_in_place, tuple(n.args), dict(n.kwargs))
            new.meta = dict(n.meta)
            n.replace_all_uses_with(new)
            g.erase_node(n)
            done += 1
    return done


def _add_rmsnorm(g: fx.Graph) -> int:
    done = 0
    for n in list(g.nodes):
        if op_name(n) != "ss.rmsnorm":
            continue
        s = n.args[0]
        if not (isinstance(s, fx.Node) and op_name(s) == "aten.add.Tensor" and len(s.args) == 2 and not s.kwargs):
            continue
        a, b = s.args
        va, vb = (x.meta.get("val") if isinstance(x, fx.Node) else None for x in (a, b))
        if not (isinstance(va, torch.Tensor) and isinstance(vb, torch.Tensor)
                and va.shape == vb.shape and va.dtype == vb.dtype and va.dim() == 2):
            continue
        if _fresh(b) and _single_use(b):
            acc, other = b, a
        elif _fresh(a) and _single_use(a):
            acc, other = a, b
        else:
            continue
        if any(isinstance(x, fx.Node) and x.op != "placeholder" and not _before(x, s) for x in n.args[1:]):
            continue                               # a norm weight computed after the add: leave it
        with g.inserting_before(s.next):           # where the sum was: its other users come later
            fused = g.call_function(add_rmsnorm, (acc, other, *n.args[1:]))
            total = g.call_function(operator.getitem, (fused, 0))
            y = g.call_function(operator.getitem, (fused, 1))
            rstd = g.call_function(operator.getitem, (fused, 2))
        total.meta = dict(s.meta)
        for u in list(n.users):
            if u.target is operator.getitem:
                repl = y if u.args[1] == 0 else rstd
                repl.meta = dict(u.meta)
                u.replace_all_uses_with(repl)
                g.erase_node(u)
        s.replace_all_uses_with(total)
        fused.meta["val"] = (total.meta.get("val"), y.meta.get("val"), rstd.meta.get("val"))
        for extra in (rstd, y):                    # the forward of a recompute variant drops rstd
            if not extra.users:
                g.erase_node(extra)
        if not n.users:
            g.erase_node(n)
        if not s.users:
            g.erase_node(s)
        done += 1
    return done


def _slice_sums(g: fx.Graph) -> int:
    """``add(add(sb0, sb1), sb2)`` over column ranges tiling the width -> ``cat``."""
    done = 0
    for root in list(g.nodes):
        if op_name(root) != "aten.add.Tensor" or any(op_name(u) == "aten.add.Tensor" for u in root.users):
            continue
        leaves, stack, ok = [], [root], True
        inner = []
        while stack and ok:
            m = stack.pop()
            if not isinstance(m, fx.Node):           # an add with a number: not a sum of slice gradients
                ok = False
            elif op_name(m) == "aten.add.Tensor" and len(m.args) == 2 and not m.kwargs and (m is root or _single_use(m)):
                inner.append(m)
                stack += [x for x in m.args]
            elif op_name(m) == "aten.slice_backward.default" and _single_use(m):
                leaves.append(m)
            else:
                ok = False
        if not ok or len(leaves) < 2:
            continue
        shape = list(leaves[0].args[1])
        if any(list(l.args[1]) != shape or l.args[2] != 1 or l.args[5] != 1 for l in leaves) or len(shape) != 2:
            continue
        width = shape[1]
        spans = sorted((max(0, l.args[3]), min(width, l.args[4]), l) for l in leaves)
        edge = 0
        for lo, hi, _ in spans:
            if lo != edge:
                break
            edge = hi
        else:
            if edge != width:
                continue
            with g.inserting_before(root):
                cat = g.call_function(torch.ops.aten.cat.default, ([l.args[0] for _, _, l in spans], 1))
            cat.meta = dict(root.meta)
            root.replace_all_uses_with(cat)
            for m in inner:
                if not m.users:
                    g.erase_node(m)
            for l in leaves:
                if not l.users:
                    g.erase_node(l)
            done += 1
    return done


def fuse_graph(gm: fx.GraphModule) -> dict[str, int]:
    """Applies the rewrites in place; returns how many of each were made."""
    g = gm.graph
    counts = {"slice_sums": _slice_sums(g), "add_rmsnorm": _add_rmsnorm(g), "rope_in_place": _rope(g)}
    if any(counts.values()):
        g.lint()
        gm.recompile()
    return counts


# ------------------------------------------------------------------------ lowering for execution
def lower_for_execution(gm: fx.GraphModule) -> fx.GraphModule:
    """A copy of ``gm`` whose ``ss::`` operator calls go straight to the Python functions behind
    them. The operators exist so that export, AOTAutograd and the rewrites above can see and
    differentiate them; a finished graph runs under ``no_grad`` and is never traced again, so the
    dispatcher round trip per call (tens of microseconds, thousands of calls per step) is only
    host time that the step has to hide."""
    from . import ops as ss_ops
    raw = {}
    for name in dir(ss_ops):
        obj = getattr(ss_ops, name)
        init = getattr(obj, "_init_fn", None)
        opname = getattr(obj, "_qualname", "") or getattr(obj, "_name", "")
        if init is not None and str(opname).startswith("ss::"):
            raw[str(opname)[4:]] = init
    g = fx.Graph()
    env: dict[fx.Node, fx.Node] = {}
    swapped = 0
    for n in gm.graph.nodes:
        if n.op == "call_function" and op_name(n) in ("aten.detach.default", "aten.alias.default"):
            env[n] = env[n.args[0]]              # nothing records a graph at execution: a no-op call
            continue
        new = g.node_copy(n, lambda a: env[a])
        if n.op == "call_function" and isinstance(n.target, torch._ops.OpOverload) and n.target.namespace == "ss":
            fn = raw.get(n.target._schema.name.split("::")[1])
            if fn is not None:
                new.target = fn
                swapped += 1
        env[n] = new
    out = fx.GraphModule(gm, g)
    out.ss_lowered_calls = swapped
    return out
