"""Text helpers: next-token shifting, batch-mean weights, candidate cross-products.

``text_datum`` turns one token sequence (with an optional per-token loss mask)
into inputs/targets; ``text_batch`` gives every unmasked target of the *global*
batch the weight ``1/N`` so that the objective's plain sum is the batch mean
(reference: packages/client/src/shadowspill_client/text/__init__.py:13,84-146).
"""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np


@dataclass
class Datum:
    tokens: np.ndarray        # int64 [n]   model inputs
    targets: np.ndarray       # int64 [n]   next token, -1 where there is none
    weights: np.ndarray       # float32 [n] loss weight per position
    extras: dict = field(default_factory=dict)   # objective inputs, float32 [n] each, indexed like targets

    def __len__(self) -> int:
        return int(self.tokens.shape[0])


def text_datum(tokens, loss_mask=None) -> Datum:
    """Inputs are ``tokens``; the target of position ``i`` is ``tokens[i+1]``; the last
    position has no target. ``loss_mask[i]`` says whether token ``i`` is to be *predicted*."""
    tok = np.asarray(tokens, dtype=np.int64).reshape(-1)
    if tok.shape[0] < 2:
        raise ValueError("a text datum needs at least two tokens")
    targets = np.full(tok.shape[0], -1, dtype=np.int64)
    targets[:-1] = tok[1:]
    w = np.zeros(tok.shape[0], dtype=np.float32)
    if loss_mask is None:
        w[:-1] = 1.0
    else:
        m = np.asarray(loss_mask).reshape(-1)
        if m.shape[0] != tok.shape[0]:
            raise ValueError("loss_mask must have one entry per token")
        w[:-1] = m[1:].astype(np.float32)
    targets = np.where(w > 0, targets, -1)
    return Datum(tok, targets, w)


def policy_datum(tokens, response_mask, old_logprobs, advantages, reference_logprobs=None) -> Datum:
    """A datum for the clipped policy objective. The per-token arrays are given per TOKEN
    (``old_logprobs[i]`` is the behaviour policy's log-probability of token ``i``); they are
    shifted here to the position that predicts that token, like the targets."""
    d = text_datum(tokens, response_mask)
    n = len(d)

    def shifted(values, name):
        a = np.asarray(values, dtype=np.float32).reshape(-1)
        if a.shape[0] != n:
            raise ValueError(f"{name} must have one entry per token")
        out = np.zeros(n, dtype=np.float32)
        out[:-1] = a[1:]
        return out
    d.extras["old_logprobs"] = shifted(old_logprobs, "old_logprobs")
    d.extras["advantages"] = shifted(advantages, "advantages")
    if reference_logprobs is not None:
        d.extras["reference_logprobs"] = shifted(reference_logprobs, "reference_logprobs")
    return d


def tensor_datum(fields: dict, weight: float = 1.0) -> Datum:
    """One row of a non-text model (the ``regression`` family): ``fields`` are its named
    float vectors, e.g. ``{"value": x, "target_values": y}``; ``weight`` scales its loss term.
    It occupies one row of a microbatch (reference: the ``Datum(inputs, loss_inputs)`` form of
    packages/client/src/shadowspill_client/protocol/inputs.py used by examples/training/regression)."""
    if not np.isfinite(weight) or weight < 0:
        raise ValueError("weight must be finite and non-negative")
    extras = {k: np.asarray(v, dtype=np.float32).reshape(1, -1) for k, v in fields.items()}
    return Datum(np.zeros(1, np.int64), np.zeros(1, np.int64), np.full(1, weight, np.float32), extras)


def text_batch(sequences, loss_masks=None) -> list[Datum]:
    """Datums whose weights sum to one over the whole batch. ``sequences`` may also hold
    ready ``Datum`` objects (for example from ``policy_datum``), which are only re-weighted."""
    masks = loss_masks if loss_masks is not None else [None] * len(sequences)
    datums = [s if isinstance(s, Datum) else text_datum(s, m) for s, m in zip(sequences, masks)]
    total = sum(float(d.weights.sum()) for d in datums)
    if total <= 0:
        raise ValueError("the batch has no position that participates in the loss")
    for d in datums:
        d.weights /= total
    return datums


def build_candidates(projection_chunks=(), moe_chunks=(), retention=("cost-input",),
                     recompute_shares=(100, 50, 0), row_chunks=()) -> dict:
    """Preparation candidates as a cross product (policy ids follow the reference's
    ``shadowspill/text_chunks@1`` / ``shadowspill/text_retention@1``)."""
    cases = []
    for pc in (projection_chunks or (0,)):
        for mc in (moe_chunks or (0,)):
            for rows in (row_chunks or (0,)):
                for r in retention:
                    cases.append({"policies": [
                        {"id": "shadowspill/text_chunks@1", "config": {"projection": pc, "moe": mc, "rows": rows}},
                        {"id": "shadowspill/text_retention@1", "config": {"rule": r}}]})
    return {"cases": cases, "recompute_shares": list(recompute_shares)}


def text_batch_statistics(datums):
    """Lengths of a batch's datums and of their trained positions, for ``CommandTable.track``
    (reference: packages/client/src/shadowspill_client/text/statistics.py)."""
    from .display import BatchStatistics
    return BatchStatistics.from_lengths([len(d) for d in datums],
                                        supervised=[int((d.weights > 0).sum()) for d in datums])
