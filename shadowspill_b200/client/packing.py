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


@dataclass(frozen=True)
class BatchValidation:
    """What checking a batch against a run's prepared geometry found (``TrainingClient.validate_batch``).

    ``capacities``: the batch's own totals (tokens, sequences, supervised positions), no padding.
    ``packing_checked``: whether the batch was actually packed into the run's microbatches;
    ``strategy`` is then the packing strategy that succeeded and ``scheduled_capacities`` the totals
    of the microbatches the step will run, padding included. ``guaranteed``: the coverage bound
    admits the batch, i.e. it packs whatever the order. ``estimated_seconds``: the simulated time
    of the run's plan for this operation. Reference: packages/client/src/shadowspill_client/
    batch_validation.py:31 (``BatchValidation``)."""
    operation: str
    capacities: dict
    packing_checked: bool
    strategy: str | None
    scheduled_capacities: dict
    guaranteed: bool = False
    note: str | None = None
    estimated_seconds: float | None = None


class BatchValidator:
    def __init__(self, vocab_size: int, microbatch_tokens: int, microbatches: int, slots: int,
                 extra_fields: tuple = (), estimated_seconds: dict | None = None, policy: str = "best_fit"):
        self.vocab, self.capacity, self.bins, self.slots = vocab_size, microbatch_tokens, microbatches, slots
        self.extra_fields = tuple(extra_fields)     # per-token inputs the run's objective reads
        self.estimated_seconds = dict(estimated_seconds or {})     # operation -> simulated seconds
        self.policy = policy

    def validate(self, datums: list[Datum], operation: str = "step", groups=None,
                 check_packing: bool = True) -> BatchValidation:
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
        lengths = [len(d) for d in datums]
        if sum(lengths) > self.capacity * self.bins:
            raise BatchError(f"batch has more than {self.capacity * self.bins} tokens")
        sequences = max(1, self.slots - 1)
        capacities = {"tokens": int(sum(lengths)), "sequences": len(datums),
                      "supervised": int(sum(int((d.weights > 0).sum()) for d in datums))}
        guaranteed = groups is None and CoverageBound(self.capacity, self.bins, sequences).admits(lengths)
        seconds = self.estimated_seconds.get(operation)
        if not check_packing:
            return BatchValidation(operation, capacities, False, None, {}, guaranteed,
                                   "packing was not asked for", seconds)
        pol = self.policy if self.policy in ("best_fit", "balanced") else "auto"
        try:
            found = assign_bins(lengths, self.capacity, self.bins, sequences, policy=pol, groups=groups)
        except BatchError:
            if pol == "auto":
                raise
            found = assign_bins(lengths, self.capacity, self.bins, sequences, policy="auto", groups=groups)
        scheduled = {"tokens": self.capacity * self.bins, "sequences": sequences * self.bins,
                     "microbatches_used": sum(1 for b in found.bins if b)}
        return BatchValidation(operation, capacities, True, found.strategy, scheduled, guaranteed, None, seconds)


@dataclass(frozen=True)
class Assignment:
    """Which microbatch every datum goes to, and how that was found."""
    bins: tuple[tuple[int, ...], ...]     # datum indices per microbatch
    strategy: str                         # best_fit | balanced | repair
    repair_nodes: int = 0                 # search nodes the repair spent (0 for the greedy strategies)


@dataclass(frozen=True)
class CoverageBound:
    """A sufficient condition under which a batch packs, checked without packing.

    A greedy pass can refuse a datum only when every microbatch is closed: ``k`` of them by their
    sequence slots (each holds ``sequences`` datums) and the others by tokens (each holds more than
    ``capacity - longest`` tokens, or the datum would fit). Counting what such a state must already
    hold gives, for every ``k``, a lower bound on the batch's datum count and token total; a batch
    below one of the two bounds for every ``k`` cannot reach any closed state, so every greedy order
    packs it. The reference ships such a bound with its prepared plans as a coverage certificate
    (packages/client/src/shadowspill_client/inputs/coverage.py); here it follows from the run's
    geometry alone."""
    capacity: int
    bins: int
    sequences: int        # datums a microbatch can hold (one slot is kept for the padding tail)

    def admits(self, lengths: list[int]) -> bool:
        if not lengths:
            return False
        longest, shortest, count, total = max(lengths), min(lengths), len(lengths), sum(lengths)
        if longest > self.capacity:
            return False
        for k in range(self.bins + 1):
            by_tokens = self.bins - k
            few_datums = count - 1 < k * self.sequences + by_tokens
            few_tokens = total - shortest < (by_tokens * (self.capacity - longest + 1)
                                             + k * self.sequences * shortest)
            if not (few_datums or few_tokens):
                return False
        return True


def atomic_groups(count: int, groups) -> list[tuple[int, ...]]:
    """Datums that must share a microbatch (``groups``), every other datum on its own."""
    if groups is None:
        return [(i,) for i in range(count)]
    out = [tuple(int(i) for i in g) for g in groups]
    flat = [i for g in out for i in g]
    if any(not g for g in out) or sorted(flat) != list(range(count)):
        raise BatchError("groups must name every datum exactly once")
    return out


def assign_bins(lengths: list[int], capacity: int, n_bins: int, sequences: int, *, policy: str = "auto",
                groups=None, max_repair_nodes: int = 10000) -> Assignment:
    """Deterministic packing of datums (or atomic groups of them) into ``n_bins`` microbatches of
    ``capacity`` tokens and ``sequences`` datums each. Largest first by the scarcer of the two
    resources; ``best_fit`` takes the tightest bin, ``balanced`` the emptiest (which keeps a bin
    from running out of sequence slots before tokens); when both greedy passes fail, a bounded
    depth-first ``repair`` moves earlier choices (at most ``max_repair_nodes`` nodes, at most 64
    groups; empty bins are interchangeable and tried once). ``policy`` ``best_fit`` / ``balanced``
    runs that pass alone; ``auto`` runs the sequence. Nothing is ever split or dropped: failure is
    a ``BatchError`` that says what was tried.

    Reference: packages/client/src/shadowspill_client/inputs/packing.py:49 (``pack_batch``:
    best_fit, balanced, bounded repair)."""
    atoms = atomic_groups(len(lengths), groups)
    cost = [(sum(lengths[i] for i in g), len(g)) for g in atoms]
    for a, (tok, cnt) in enumerate(cost):
        if tok > capacity or cnt > sequences:
            raise BatchError(f"datum group {atoms[a]} needs {tok} tokens and {cnt} sequences; a microbatch "
                             f"holds {capacity} and {sequences}")
    order = sorted(range(len(atoms)), key=lambda a: (-max(cost[a][0] / max(capacity, 1),
                                                          cost[a][1] / max(sequences, 1)), -cost[a][0], a))

    def greedy(balanced: bool):
        free_t, free_s = [capacity] * n_bins, [sequences] * n_bins
        bins = [[] for _ in range(n_bins)]
        for a in order:
            tok, cnt = cost[a]
            cands = [b for b in range(n_bins) if tok <= free_t[b] and cnt <= free_s[b]]
            if not cands:
                return None
            slack = lambda b: (free_t[b] - tok) / max(capacity, 1) + (free_s[b] - cnt) / max(sequences, 1)
            b = max(cands, key=lambda b: (slack(b), -b)) if balanced else min(cands, key=lambda b: (slack(b), b))
            bins[b].append(a)
            free_t[b] -= tok
            free_s[b] -= cnt
        return bins

    passes = {"best_fit": (False,), "balanced": (True,), "auto": (False, True)}.get(policy)
    if passes is None:
        raise BatchError(f"unknown packing policy {policy!r}")
    found, strategy, nodes = None, "", 0
    for balanced in passes:
        found = greedy(balanced)
        if found is not None:
            strategy = "balanced" if balanced else "best_fit"
            break
    if found is None and policy == "auto" and len(atoms) <= 64:
        free_t, free_s = [capacity] * n_bins, [sequences] * n_bins
        bins = [[] for _ in range(n_bins)]

        def place(pos: int) -> bool:
            nonlocal nodes
            if pos == len(order):
                return True
            if nodes >= max_repair_nodes:
                return False
            nodes += 1
            a = order[pos]
            tok, cnt = cost[a]
            tried_empty = False
            for b in sorted(range(n_bins), key=lambda b: (free_t[b], b)):
                if tok > free_t[b] or cnt > free_s[b]:
                    continue
                if not bins[b]:
                    if tried_empty:
                        continue
                    tried_empty = True
                bins[b].append(a); free_t[b] -= tok; free_s[b] -= cnt
                if place(pos + 1):
                    return True
                bins[b].pop(); free_t[b] += tok; free_s[b] += cnt
            return False
        if place(0):
            found, strategy = bins, "repair"
    if found is None:
        raise BatchError(f"datums do not fit the configured microbatches ({n_bins} x {capacity} tokens, "
                         f"{sequences} sequences each; tried {policy}"
                         + (f", repair spent {nodes} nodes" if nodes else "")
                         + "); lower the batch or raise tokens_per_step")
    return Assignment(tuple(tuple(sorted(i for a in members for i in atoms[a])) for members in found),
                      strategy, nodes)


def _bins(lengths: list[int], capacity: int, n_bins: int, policy: str, slots: int = 1 << 30,
          groups=None) -> list[list[int]]:
    sequences = max(1, slots - 1)
    pol = policy if policy in ("best_fit", "balanced") else "auto"
    if pol != "auto":
        try:
            return [list(b) for b in assign_bins(lengths, capacity, n_bins, sequences, policy=pol, groups=groups).bins]
        except BatchError:
            pass                       # the named strategy is a preference: fall through to the sequence
    return [list(b) for b in assign_bins(lengths, capacity, n_bins, sequences, policy="auto", groups=groups).bins]


def pack_batch(datums: list[Datum], *, microbatch_tokens: int, microbatches: int, slots: int,
               policy: str = "best_fit", placement: list | None = None, groups=None) -> list[PackedMicrobatch]:
    """``placement`` (a list, filled in place): for every datum ``(microbatch, first row, rows)``,
    which is what maps per-row outputs of a forward call back to the datums. ``groups``: lists of
    datum indices that must share a microbatch (every datum named once)."""
    bins = _bins([len(d) for d in datums], microbatch_tokens, microbatches, policy, slots, groups)
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
