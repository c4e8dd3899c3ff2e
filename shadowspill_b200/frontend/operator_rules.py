"""What the graph frontend has to know about an operator, declared in one place.

Export, differentiation and execution need nothing but the operator itself (its fake and autograd
registrations). Three later decisions need facts the operator cannot tell:

  cost        ``memory``: the output is cheap to redo from its inputs (an elementwise or row-wise
              pass), so a ``save`` policy recomputes it instead of keeping it; ``compute``: dominated
              by tensor-core work, worth keeping
  row_args    which argument positions carry token rows, for row chunking: the operator then runs
              chunk by chunk on slices of those arguments and its row-shaped outputs are
              concatenated; ``None`` makes it a barrier (it sees whole sequences)
  flops       floating-point operations of one call, from the node's metadata, for the builder's
              estimate before anything is profiled

The built-in ``ss::`` operators are declared below; ``register_operator_rule`` adds a rule for an
operator of your own (any ``torch.library`` namespace), after which it takes part in retention and
row chunking like the built-ins. An operator without a rule is treated conservatively: kept when a
policy keeps everything, never chunked.

Reference: the reference's translation of operator metadata into planner rules
(packages/workloads/src/shadowspill_workloads/integrations/mlops.py:53-225: ``OperatorRule``,
``GradientDestinationRule``, ``ExecutionLifetimes``).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable


@dataclass(frozen=True)
class OperatorRule:
    op: str                                   # "namespace.name", as torch prints it without the overload
    cost: str = "compute"                     # compute | memory
    row_args: tuple[int, ...] | None = None   # None: a barrier for row chunking
    flops: Callable | None = None

    def __post_init__(self):
        if self.cost not in ("compute", "memory"):
            raise ValueError("cost is 'compute' or 'memory'")
        if "." not in self.op:
            raise ValueError("operators are named namespace.name")


_RULES: dict[str, OperatorRule] = {}


def register_operator_rule(rule: OperatorRule, replace: bool = False) -> OperatorRule:
    if rule.op in _RULES and not replace:
        raise ValueError(f"{rule.op} already has a rule")
    _RULES[rule.op] = rule
    return rule


def rule_of(name: str) -> OperatorRule | None:
    """``name`` as ``export.op_name`` gives it: ``ss.linear``, or ``acme.scale_rows.default`` for
    other namespaces (the overload is ignored)."""
    found = _RULES.get(name)
    if found is None and name.count(".") >= 2:
        found = _RULES.get(name.rsplit(".", 1)[0])
    return found


def registered() -> dict[str, OperatorRule]:
    return dict(_RULES)


def _linear_flops(n) -> float:
    x, w = n.args[0].meta["val"], n.args[1].meta["val"]
    return 2.0 * x.shape[0] * w.shape[0] * w.shape[1]


for _r in (
    OperatorRule("ss.linear", "compute", (0,), _linear_flops),
    OperatorRule("ss.gemm", "compute", None),            # rows only in its untransposed form: chunking checks that itself
    OperatorRule("ss.head_loss", "compute", None, _linear_flops),
    OperatorRule("ss.attention", "compute", None),
    OperatorRule("ss.gated_delta_rule", "compute", None),
    OperatorRule("ss.moe_experts", "compute", None),
    OperatorRule("ss.moe_experts_lora", "compute", None),
    OperatorRule("ss.moe_experts_routed", "compute", None),
    OperatorRule("ss.moe_experts_routed_lora", "compute", None),
    OperatorRule("ss.sparse_latent_attention", "compute", None),
    OperatorRule("ss.index_topk", "compute", None),
    OperatorRule("ss.rmsnorm", "memory", (0,)),
    OperatorRule("ss.rope", "memory", (0, 1)),
    OperatorRule("ss.swiglu", "memory", (0,)),
    OperatorRule("ss.swiglu_bwd", "memory", (0, 1)),
    OperatorRule("ss.embedding", "memory", (0,)),
    OperatorRule("ss.l2norm", "memory", (0,)),
    OperatorRule("ss.l2norm_bwd", "memory", (0, 1)),
    OperatorRule("ss.gated_rmsnorm", "memory", (0, 1)),
    OperatorRule("ss.conv_silu", "memory", None),        # reads its neighbours in the sequence
):
    register_operator_rule(_r)
