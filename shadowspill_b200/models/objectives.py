"""Training objectives evaluated inside the chunked output head.

``cross_entropy``          weighted, masked next-token loss
``clipped_policy``         PPO-style clipped surrogate on the target tokens' probability
                           ratio against ``old_logprobs`` with ``advantages``, optional
                           penalty against ``reference_logprobs`` (k3 estimator)
``weighted_squared_error`` regression on a scalar head (the ``regression`` family)
plus ``moe_balance``: a router load-balancing term added per routed layer and
summed with the head objective ("sum" composition).

Each objective names the extra per-token batch fields it reads; they become part of
the packed microbatch object. Component ids follow the reference
(packages/workloads/src/shadowspill_workloads/components/token.py:208;
objectives/head/execution.py:17-60; objectives/moe.py:4): ``shadowspill/cross_entropy@1``,
``shadowspill/clipped_policy@1``, ``shadowspill/sum@1``.
"""
from __future__ import annotations

from dataclasses import asdict, dataclass
from typing import Any

KINDS = ("cross_entropy", "clipped_policy", "weighted_squared_error")
COMPONENT_IDS = {"cross_entropy": "shadowspill/cross_entropy@1",
                 "clipped_policy": "shadowspill/clipped_policy@1",
                 "weighted_squared_error": "shadowspill/weighted_squared_error@1",
                 "sum": "shadowspill/sum@1", "moe_balance": "shadowspill/moe_balance@1"}


@dataclass(frozen=True)
class Objective:
    kind: str = "cross_entropy"
    clip_ratio: float = 0.2
    reference_beta: float = 0.0          # > 0 reads reference_logprobs
    moe_balance_coef: float = 0.0        # > 0 adds the router balance term of every routed layer

    def __post_init__(self) -> None:
        if self.kind not in KINDS:
            raise ValueError(f"unknown objective {self.kind!r}; known: {KINDS}")
        if not 0.0 < self.clip_ratio < 1.0:
            raise ValueError("clip_ratio must lie in (0, 1)")
        if self.reference_beta < 0 or self.moe_balance_coef < 0:
            raise ValueError("coefficients must be non-negative")

    @property
    def extra_fields(self) -> tuple[str, ...]:
        """Per-token fp32 batch fields beyond tokens/targets/weights/positions."""
        if self.kind != "clipped_policy":
            return ()
        base = ("old_logprobs", "advantages")
        return base + (("reference_logprobs",) if self.reference_beta > 0 else ())

    @property
    def component_id(self) -> str:
        return COMPONENT_IDS["sum"] if self.moe_balance_coef > 0 else COMPONENT_IDS[self.kind]

    def to_json(self) -> dict[str, Any]:
        return asdict(self)

    @staticmethod
    def from_json(d: dict[str, Any] | None) -> "Objective":
        return Objective(**(d or {}))

    @staticmethod
    def from_component(component_id: str, **config: Any) -> "Objective":
        """``shadowspill/<kind>@1`` ids of the service protocol; a ``sum`` takes the head
        objective under ``head`` and the balance coefficient under ``moe_balance``."""
        inverse = {v: k for k, v in COMPONENT_IDS.items()}
        kind = inverse.get(component_id)
        if kind is None:
            raise ValueError(f"unknown objective component {component_id!r}")
        if kind == "sum":
            head = Objective.from_component(config.get("head", COMPONENT_IDS["cross_entropy"]),
                                            **config.get("head_config", {}))
            return Objective(head.kind, head.clip_ratio, head.reference_beta,
                             float(config.get("moe_balance", 0.0)))
        if kind == "moe_balance":
            raise ValueError("moe_balance is only usable inside a sum")
        return Objective(kind, **config)


def router_balance(probability_sums, counts, n_tokens: int, top_k: int):
    """Load-balancing term of one routed layer: ``E * sum_e f_e * P_e`` with ``f_e`` the
    fraction of assignments routed to expert ``e`` and ``P_e`` its mean router
    probability (``probability_sums[e] / n_tokens``). Differentiable through
    ``probability_sums``; the counts are treated as constants."""
    E = counts.numel()
    f = counts.to(probability_sums.dtype) / max(1, n_tokens * top_k)
    return E * (f.detach() * probability_sums / max(1, n_tokens)).sum()
