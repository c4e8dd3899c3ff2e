"""Server-side validation and routing of batch payloads.

The client validates what it sends, but the service does not trust it: before a payload is
routed to workers every microbatch is checked against the run's geometry (token count, vocabulary
range, sequence-boundary table, finite non-negative weights, the objective's per-token inputs).
A payload that fails is rejected before any worker sees it, so the training state stays valid
(reference: packages/engine/src/shadowspill/training/inputs/{adapters,staging,materialize}.py).
"""
from __future__ import annotations

import numpy as np


class InputError(ValueError):
    pass


def validate_microbatches(mbs, geometry: dict) -> None:
    """``geometry``: the run's ``microbatch_tokens``, ``microbatches``, ``workers``, ``slots``,
    ``vocab_size`` and ``extra_fields``."""
    T, slots, vocab = geometry["microbatch_tokens"], geometry["slots"], geometry["vocab_size"]
    want = geometry["microbatches"] * geometry["workers"]
    if len(mbs) != want:
        raise InputError(f"expected {want} microbatches, got {len(mbs)}")
    participating = 0.0
    for i, mb in enumerate(mbs):
        for name in ("tokens", "targets", "weights", "positions"):
            a = getattr(mb, name)
            if a.ndim != 1 or a.shape[0] != T:
                raise InputError(f"microbatch {i}: {name} must have {T} entries, has {a.shape}")
        if mb.tokens.min() < 0 or mb.tokens.max() >= vocab:
            raise InputError(f"microbatch {i}: token ids outside [0, {vocab})")
        if mb.targets.max() >= vocab or mb.targets.min() < -1:
            raise InputError(f"microbatch {i}: targets outside [-1, {vocab})")
        if not np.isfinite(mb.weights).all() or (mb.weights < 0).any():
            raise InputError(f"microbatch {i}: weights must be finite and non-negative")
        cu = mb.cu_seqlens
        if cu.ndim != 1 or not 2 <= cu.shape[0] <= slots + 1:
            raise InputError(f"microbatch {i}: the sequence table needs 2..{slots + 1} entries")
        if cu[0] != 0 or cu[-1] != T or (np.diff(cu) < 0).any():
            raise InputError(f"microbatch {i}: sequence boundaries must rise from 0 to {T}")
        if mb.positions.min() < 0 or mb.positions.max() >= T:
            raise InputError(f"microbatch {i}: positions outside [0, {T})")
        starts = cu[:-1][np.diff(cu) > 0]
        if (mb.positions[starts] != 0).any():
            raise InputError(f"microbatch {i}: a sequence does not start at position 0")
        if not 1 <= int(mb.max_seqlen) <= T:
            raise InputError(f"microbatch {i}: max_seqlen {mb.max_seqlen} outside [1, {T}]")
        if int(np.diff(cu).max()) > int(mb.max_seqlen):
            raise InputError(f"microbatch {i}: a sequence is longer than the declared max_seqlen")
        for spec in geometry.get("extra_fields", ()):
            name, _, width = spec.partition(":")
            shape = (T, int(width)) if width else (T,)
            a = (getattr(mb, "extras", None) or {}).get(name)
            if a is None or a.shape != shape or not np.isfinite(a).all():
                raise InputError(f"microbatch {i}: input {name!r} missing or malformed "
                                 f"(expected float32 {shape})")
        participating += float(mb.weights[mb.targets >= 0].sum())
    if participating <= 0:
        raise InputError("no position of the batch participates in the loss")


def route(mbs, workers: int, per_worker: int) -> list[list]:
    """Microbatches in order, ``per_worker`` consecutive ones to each rank."""
    return [list(mbs[r * per_worker:(r + 1) * per_worker]) for r in range(workers)]
