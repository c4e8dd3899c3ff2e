"""Local batch validation and deterministic packing of datums into microbatches.

``pack_batch`` bins datums into equal-capacity microbatches (first-fit
decreasing = ``best_fit``; ``balanced`` levels token counts), lays each bin out
as one packed row with per-sequence boundaries, and turns any remaining capacity
into padding that forms its own causal sequence with zero loss weight.
Reference: packages/client/src/shadowspill_client/inputs/packing.py:49,
batch_validation.py:70.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np

from .text import Datum


class BatchError(ValueError):
    pass


@dataclass
class PackedMicrobatch:
    tokens: np.ndarray
    targets: np.ndarray
    weights: np.ndarray
    positions: np.ndarray
    cu_seqlens: np.ndarray
    max_seqlen: int
    extras: dict = None       # objective inputs, float32 [T] each

    def __post_init__(self):
        if self.extras is None:
            self.extras = {}

    @property
    def nbytes(self) -> int:
        return sum(a.nbytes for a in (self.tokens, self.targets, self.weights, self.positions,
                                      self.cu_seqlens, *self.extras.values()))


class BatchValidator:
    def __init__(self, vocab_size: int, microbatch_tokens: int, microbatches: int, slots: int,
                 extra_fields: tuple = ()):
        self.vocab, self.capacity, self.bins, self.slots = vocab_size, microbatch_tokens, microbatches, slots
        self.extra_fields = tuple(extra_fields)     # per-token inputs the run's objective reads

    def validate(self, datums: list[Datum]) -> None:
        if not datums:
            raise BatchError("empty batch")
        participating = 0.0
        for i, d in enumerate(datums):
            if len(d) > self.capacity:
                raise BatchError(f"datum {i} has {len(d)} tokens; a microbatch holds {self.capacity}")
            if d.tokens.min() < 0 or d.tokens.max() >= self.vocab:
                raise BatchError(f"datum {i} has token ids outside [0, {self.vocab})")
            if not np.isfinite(d.weights).all() or (d.weights < 0).any():
                raise BatchError(f"datum {i} has negative or non-finite weights")
            for spec in self.extra_fields:
                name, _, width = spec.partition(":")
                values = getattr(d, "extras", {}).get(name)
                if values is None:
                    raise BatchError(f"datum {i} lacks {name!r}, which this run reads")
                values = np.asarray(values)
                shape = (len(d), int(width)) if width else (len(d),)
                if values.shape != shape or not np.isfinite(values).all():
                    raise BatchError(f"datum {i}: {name!r} must be finite with shape {shape}")
            participating += float(d.weights.sum())
        if participating <= 0:
            raise BatchError("no position of the batch participates in the loss")
        if sum(len(d) for d in datums) > self.capacity * self.bins:
            raise BatchError(f"batch has more than {self.capacity * self.bins} tokens")


def _bins(lengths: list[int], capacity: int, n_bins: int, policy: str) -> list[list[int]]:
    order = sorted(range(len(lengths)), key=lambda i: (-lengths[i], i))
    bins: list[list[int]] = [[] for _ in range(n_bins)]
    free = [capacity] * n_bins
    for i in order:
        cands = [b for b in range(n_bins) if lengths[i] <= free[b]]
        if not cands:
            raise BatchError("datums do not fit the configured microbatches; lower the batch or "
                             "raise tokens_per_step")
        if policy == "balanced":
            b = max(cands, key=lambda b: (free[b], -b))          # emptiest bin
        else:
            b = min(cands, key=lambda b: (free[b], b))            # tightest fit
        bins[b].append(i)
        free[b] -= lengths[i]
    return bins


def pack_batch(datums: list[Datum], *, microbatch_tokens: int, microbatches: int, slots: int,
               policy: str = "best_fit", placement: list | None = None) -> list[PackedMicrobatch]:
    """``placement`` (a list, filled in place): for every datum ``(microbatch, first row, rows)``,
    which is what maps per-row outputs of a forward call back to the datums."""
    bins = _bins([len(d) for d in datums], microbatch_tokens, microbatches, policy)
    out = []
    if placement is not None:
        placement[:] = [None] * len(datums)
    T = microbatch_tokens
    for members in bins:
        if len(members) + 1 > slots:
            raise BatchError(f"a microbatch would hold {len(members)} sequences; the plan has "
                             f"{slots - 1} slots")
        tokens = np.zeros(T, np.int64)
        targets = np.full(T, -1, np.int64)
        weights = np.zeros(T, np.float32)
        positions = np.zeros(T, np.int32)
        names = sorted({k for d in datums for k in getattr(d, "extras", {})})
        widths = {k: np.asarray(next(d.extras[k] for d in datums if k in d.extras)).shape[1:] for k in names}
        extras = {k: np.zeros((T,) + widths[k], np.float32) for k in names}
        cu, pos = [0], 0
        for i in sorted(members):
            d = datums[i]
            n = len(d)
            tokens[pos:pos + n], targets[pos:pos + n], weights[pos:pos + n] = d.tokens, d.targets, d.weights
            for k in names:
                if k not in d.extras:
                    raise BatchError(f"datum {i} lacks the objective input {k!r}")
                extras[k][pos:pos + n] = d.extras[k]
            positions[pos:pos + n] = np.arange(n, dtype=np.int32)
            if placement is not None:
                placement[i] = (len(out), pos, n)
            pos += n
            cu.append(pos)
        if pos < T:
            positions[pos:] = np.arange(T - pos, dtype=np.int32)
            cu.append(T)
        cu += [T] * (slots + 1 - len(cu))
        lens = np.diff(np.asarray(cu))
        out.append(PackedMicrobatch(tokens, targets, weights, positions,
                                    np.asarray(cu, np.int32), int(max(2, lens.max())), extras))
    return out
