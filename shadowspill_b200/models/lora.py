"""Low-rank adapters.

A target matrix ``W [out, in]`` gains ``A [r, in]`` (normal init) and ``B [out, r]``
(zero init) and computes ``x W^T + (alpha / r) (x A^T) B^T``; the base weights are
frozen unless ``train_base``: they get no gradient buffer and no optimizer state,
which is where LoRA's memory saving comes from in a budgeted plan. Routed expert
banks ``[E, out, in]`` carry per-expert factors ``A [E, r, in]`` / ``B [E, out, r]``.

Reference: packages/workloads/src/shadowspill_workloads/lora/__init__.py:16
(``configure_lora``), models/shared/routed_lora.py:24 (``add_factors``), and the
client's ``LoRA`` record (packages/client/src/shadowspill_client/config/model.py:133).
"""
from __future__ import annotations

from dataclasses import asdict, dataclass
from typing import Any

DENSE_TARGETS = ("wq", "wk", "wv", "wo", "w13", "w2", "w_qkvz", "w_out", "sw13", "sw2",
                 "q_a", "q_b", "kv_a", "kv_b")          # the last four: latent-attention projections (GLM)


@dataclass(frozen=True)
class LoRAConfig:
    rank: int = 16
    alpha: float = 32.0
    targets: tuple[str, ...] = ("wq", "wk", "wv", "wo", "w13", "w2")
    routed_experts: bool = True          # adapt expert banks named in ``targets`` too
    train_base: bool = False

    def __post_init__(self) -> None:
        if self.rank < 8 or self.rank % 8:
            raise ValueError("LoRA rank must be a positive multiple of 8")
        unknown = [t for t in self.targets if t not in DENSE_TARGETS]
        if unknown:
            raise ValueError(f"unknown LoRA targets {unknown}; known: {DENSE_TARGETS}")

    @property
    def scale(self) -> float:
        return self.alpha / self.rank

    def to_json(self) -> dict[str, Any]:
        d = asdict(self)
        d["targets"] = list(self.targets)
        return d

    @staticmethod
    def from_json(d: dict[str, Any] | None) -> "LoRAConfig | None":
        if not d:
            return None
        d = dict(d)
        d["targets"] = tuple(d.get("targets", ()))
        return LoRAConfig(**d)


def factor_names(target: str) -> tuple[str, str]:
    return f"{target}_lora_a", f"{target}_lora_b"
