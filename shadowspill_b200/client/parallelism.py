"""Plain-dict parallelism declarations.

``data_parallel`` shards weights, gradients and optimizer state over a named
group (tensors below ``min_shard_bytes`` stay whole); ``expert_parallel`` shards
expert banks on dimension 0 and keeps dense parts replicated with a sharded
optimizer. Reference: packages/client/src/shadowspill_client/parallelism.py:12-120.
"""
from __future__ import annotations

MIN_SHARD_BYTES = 2 << 20


def data_parallel(ranks: int, *, weights: str = "sharded", gradients: str = "sharded",
                  optimizer: str = "sharded", replicas: int = 1,
                  min_shard_bytes: int = MIN_SHARD_BYTES) -> dict:
    for name, v in (("weights", weights), ("gradients", gradients), ("optimizer", optimizer)):
        if v not in ("sharded", "replicated"):
            raise ValueError(f"{name} must be 'sharded' or 'replicated'")
    if ranks < 1 or replicas < 1:
        raise ValueError("ranks and replicas must be positive")
    if replicas > 1 and ranks < 2:
        raise ValueError("replicas repeat a shard group of at least two ranks")
    if "sharded" in (weights, gradients) and optimizer != "sharded":
        raise ValueError("optimizer state must shard over the same group as sharded weights/gradients")
    return {"kind": "data_parallel", "ranks_per_replica": ranks, "num_replicas": replicas,
            "groups": {"all_ranks": list(range(ranks))},      # ranks of one replica
            "storage": {"weights": weights, "gradients": gradients, "optimizer": optimizer},
            "min_shard_bytes": min_shard_bytes, "inputs": {"placement": "split_microbatches"}}


def expert_parallel(ranks: int, *, n_experts: int, top_k: int, min_shard_bytes: int = MIN_SHARD_BYTES) -> dict:
    if not 2 <= ranks <= 128:
        raise ValueError("expert parallelism needs 2 to 128 ranks")
    if n_experts % ranks:
        raise ValueError("n_experts must be divisible by the number of ranks")
    if top_k > 32:
        raise ValueError("top_k may not exceed 32")
    return {"kind": "expert_parallel", "ranks_per_replica": ranks, "num_replicas": 1,
            "groups": {"all_ranks": list(range(ranks))},
            "placements": {"experts": {"sharded": "all_ranks", "dim": 0, "stored": "local"},
                           "dense": {"replicated": "all_ranks"}},
            "storage": {"weights": "replicated", "gradients": "replicated", "optimizer": "sharded"},
            "min_shard_bytes": min_shard_bytes, "experts_per_rank": n_experts // ranks}
