"""Synthetic packed variable-length batches.

Sequence lengths are log-normal (median 1200 by default) clipped to
``[min_len, max_len]``, packed first-fit into fixed-capacity microbatches; any
remaining capacity is padding that forms its own causal sequence with zero loss
weight, as in the reference's packing adapter
(packages/workloads/src/shadowspill_workloads/inputs/text/preparation.py:46-70).
The loss mask alternates spans so that about half of the tokens carry loss, and
weights are ``1/N`` over all unmasked targets of the global batch (the
reference's ``text_batch`` convention, packages/client/src/shadowspill_client/text/__init__.py:84-146).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field

import numpy as np


@dataclass
class HostMicrobatch:
    """One packed microbatch as NumPy arrays (what a client sends)."""
    tokens: np.ndarray       # int64 [T]
    targets: np.ndarray      # int64 [T]
    weights: np.ndarray      # float32 [T]
    positions: np.ndarray    # int32 [T]
    cu_seqlens: np.ndarray   # int32 [slots+1]
    max_seqlen: int
    extras: dict = field(default_factory=dict)   # objective inputs: float32 [T] each

    @property
    def nbytes(self) -> int:
        return (self.tokens.nbytes + self.targets.nbytes + self.weights.nbytes
                + self.positions.nbytes + self.cu_seqlens.nbytes
                + sum(v.nbytes for v in self.extras.values()))


def sample_lengths(rng: np.random.Generator, total_tokens: int, *, median: float = 1200.0,
                   sigma: float = 1.0, min_len: int = 32, max_len: int = 8192) -> list[int]:
    out, acc = [], 0
    while acc < total_tokens:
        n = int(np.clip(rng.lognormal(math.log(median), sigma), min_len, max_len))
        n = min(n, total_tokens - acc)
        if n < 2:
            break
        out.append(n)
        acc += n
    return out


def pack_first_fit(lengths: list[int], capacity: int, n_bins: int | None = None) -> list[list[int]]:
    """Deterministic first-fit-decreasing packing of sequence indices into bins."""
    order = sorted(range(len(lengths)), key=lambda i: (-lengths[i], i))
    bins: list[list[int]] = [[] for _ in range(n_bins or 0)]
    free = [capacity] * len(bins)
    for i in order:
        for b in range(len(bins)):
            if lengths[i] <= free[b]:
                bins[b].append(i)
                free[b] -= lengths[i]
                break
        else:
            if n_bins is not None:
                raise ValueError("sequences do not fit the given number of microbatches")
            bins.append([i])
            free.append(capacity - lengths[i])
    return bins


def make_batch(seed: int, *, vocab: int, tokens_per_step: int, microbatch_tokens: int,
               max_len: int = 8192, median: float = 1200.0, min_len: int = 32,
               mask_span: int = 64, masked_fraction: float = 0.5,
               fixed_len: int | None = None, slots: int | None = None) -> list[HostMicrobatch]:
    """A global batch of ``tokens_per_step`` tokens as equal-capacity microbatches."""
    rng = np.random.default_rng(seed)
    n_mb = tokens_per_step // microbatch_tokens
    if fixed_len:
        per = microbatch_tokens // fixed_len
        groups = [[fixed_len] * per for _ in range(n_mb)]
    else:
        max_len = min(max_len, microbatch_tokens)
        groups = []
        for _ in range(n_mb):
            groups.append(sample_lengths(rng, microbatch_tokens, median=median, min_len=min_len,
                                         max_len=max_len))
    slots = slots or max(len(g) for g in groups) + 1
    mbs, unmasked_total = [], 0
    for g in groups:
        T = microbatch_tokens
        tokens = rng.integers(0, vocab, size=T, dtype=np.int64)
        targets = np.full(T, -1, dtype=np.int64)
        mask = np.zeros(T, dtype=bool)
        positions = np.zeros(T, dtype=np.int32)
        cu = [0]
        pos = 0
        for n in g:
            positions[pos:pos + n] = np.arange(n, dtype=np.int32)
            targets[pos:pos + n - 1] = tokens[pos + 1:pos + n]
            idx = np.arange(n - 1)
            if masked_fraction > 0:
                keep = ((idx // mask_span) % 2 == 0) if masked_fraction >= 0.5 else np.ones(n - 1, bool)
            else:
                keep = np.ones(n - 1, bool)
            mask[pos:pos + n - 1] = keep
            pos += n
            cu.append(pos)
        if pos < T:  # padding is its own causal sequence with no loss
            positions[pos:] = np.arange(T - pos, dtype=np.int32)
            cu.append(T)
        while len(cu) < slots + 1:
            cu.append(T)
        unmasked_total += int(mask.sum())
        lens = np.diff(np.asarray(cu))
        mbs.append(HostMicrobatch(tokens, np.where(mask, targets, -1), mask.astype(np.float32),
                                  positions, np.asarray(cu, dtype=np.int32),
                                  int(max(2, lens.max()))))
    scale = 1.0 / max(1, unmasked_total)
    for mb in mbs:
        mb.weights *= scale
    return mbs


def to_device(mb: HostMicrobatch, device):
    """Pageable-host convenience conversion (tests); the executor stages through pinned memory."""
    import torch
    from ..models.decoder import BatchMeta
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(device)
    return BatchMeta(t(mb.tokens), t(mb.targets), t(mb.weights), t(mb.positions),
                     t(mb.cu_seqlens), mb.max_seqlen, {k: t(v) for k, v in mb.extras.items()})
