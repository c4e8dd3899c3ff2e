"""Ownership declarations: which ranks hold which part of each parameter and
how its weights, gradients and optimizer state are stored.

A ``Parallelism`` describes one replica of ``ranks_per_replica`` ranks repeated
``num_replicas`` times. Named group collections partition a replica; a
parameter is computed either ``Replicated`` or ``Sharded`` (split on one tensor
dimension across the ranks of a group), and each of its three state components
is stored ``sharded`` (flat 1/N slices gathered on use) or ``replicated`` over a
group. Selectors are parameter names or ``fnmatch`` patterns; an exact name
wins over a pattern, and among patterns the longest wins.

Same surface as the reference's declaration
(packages/engine/src/shadowspill/parallelism/spec.py:24-160, placements.py,
storage.py), kept to what the program builder and the executor consume:
``resolve(name, nbytes)`` answers with a ``ResolvedParameter`` for one rank.
"""
from __future__ import annotations

import fnmatch
from dataclasses import dataclass, field, replace
from typing import Any, Mapping, Sequence

MIN_SHARD_BYTES = 2 << 20
_MODES = ("sharded", "replicated")


@dataclass(frozen=True)
class GroupRef:
    """A named collection of disjoint rank groups covering one replica."""
    name: str
    groups: tuple[tuple[int, ...], ...]

    def __post_init__(self) -> None:
        if not self.name:
            raise ValueError("a group collection needs a name")
        seen: set[int] = set()
        for g in self.groups:
            if not g:
                raise ValueError(f"{self.name}: empty group")
            if seen & set(g) or len(set(g)) != len(g):
                raise ValueError(f"{self.name}: a rank appears twice")
            seen |= set(g)

    def group_of(self, rank: int) -> tuple[int, ...]:
        for g in self.groups:
            if rank in g:
                return g
        raise KeyError(f"rank {rank} is in no group of {self.name!r}")


@dataclass(frozen=True)
class Replicated:
    """Every rank computes with the whole parameter."""
    group: str = "all_ranks"


@dataclass(frozen=True)
class Sharded:
    """Each rank of ``group`` computes with one slice along ``dim`` (expert banks
    shard on dimension 0). ``stored='local'`` keeps only that slice in this rank's
    state; ``'flat'`` additionally splits the slice's storage over the group."""
    group: str = "all_ranks"
    dim: int = 0
    stored: str = "local"

    def __post_init__(self) -> None:
        if self.dim < 0:
            raise ValueError("dim must be non-negative")
        if self.stored not in ("local", "flat"):
            raise ValueError("stored must be 'local' or 'flat'")


Placement = Replicated | Sharded


@dataclass(frozen=True)
class ParameterStorage:
    """Storage mode of each state component over ``group``; ``None`` inherits the
    default declaration's value."""
    group: str | None = None
    weights: str | None = None
    gradients: str | None = None
    optimizer: str | None = None

    def __post_init__(self) -> None:
        for n in ("weights", "gradients", "optimizer"):
            v = getattr(self, n)
            if v is not None and v not in _MODES:
                raise ValueError(f"{n} must be 'sharded' or 'replicated'")

    def over(self, base: "ParameterStorage") -> "ParameterStorage":
        return ParameterStorage(*(getattr(self, n) if getattr(self, n) is not None else getattr(base, n)
                                  for n in ("group", "weights", "gradients", "optimizer")))

    @property
    def complete(self) -> bool:
        return None not in (self.group, self.weights, self.gradients, self.optimizer)


@dataclass(frozen=True)
class ResolvedParameter:
    """What one rank does with one parameter."""
    name: str
    placement: Placement
    storage: ParameterStorage
    compute_group: tuple[int, ...]       # ranks sharing this parameter's compute placement
    storage_group: tuple[int, ...]       # ranks its stored components divide over
    compute_index: int                   # this rank's slice index when Sharded, else 0
    storage_index: int

    @property
    def compute_shards(self) -> int:
        return len(self.compute_group) if isinstance(self.placement, Sharded) else 1

    def storage_shards(self, component: str) -> int:
        return len(self.storage_group) if getattr(self.storage, component) == "sharded" else 1

    def needs_gather(self) -> bool:
        return self.storage_shards("weights") > 1

    def gradient_reduction(self) -> str:
        """``reduce_scatter`` when gradients are stored sharded, ``all_reduce`` when
        they are replicated over more than one rank, else ``none``."""
        if len(self.storage_group) <= 1:
            return "none"
        return "reduce_scatter" if self.storage.gradients == "sharded" else "all_reduce"


_DEFAULT_STORAGE = ParameterStorage("all_ranks", "sharded", "sharded", "sharded")


@dataclass(frozen=True)
class Parallelism:
    ranks_per_replica: int = 1
    num_replicas: int = 1
    groups: Mapping[str, Sequence[Sequence[int]]] = field(default_factory=dict)
    default_parameter_placement: Placement = field(default_factory=Replicated)
    parameter_placements: Mapping[str, Placement] = field(default_factory=dict)
    default_parameter_storage: ParameterStorage = _DEFAULT_STORAGE
    parameter_storage: Mapping[str, ParameterStorage] = field(default_factory=dict)
    min_shard_bytes: int = MIN_SHARD_BYTES
    inputs: str = "per_rank"            # per_rank | split_microbatches

    def __post_init__(self) -> None:
        for n in ("ranks_per_replica", "num_replicas"):
            v = getattr(self, n)
            if type(v) is not int or v < 1:
                raise ValueError(f"{n} must be a positive integer")
        groups = dict(self.groups) or {"all_ranks": (tuple(range(self.ranks_per_replica)),)}
        frozen: dict[str, GroupRef] = {}
        for name, members in groups.items():
            ref = GroupRef(name, tuple(tuple(int(r) for r in g) for g in members))
            if sorted(r for g in ref.groups for r in g) != list(range(self.ranks_per_replica)):
                raise ValueError(f"{name}: groups must cover exactly one replica")
            frozen[name] = ref
        object.__setattr__(self, "groups", frozen)
        if not isinstance(self.default_parameter_placement, (Replicated, Sharded)):
            raise TypeError("default_parameter_placement must be Replicated or Sharded")
        if not isinstance(self.default_parameter_storage, ParameterStorage):
            raise TypeError("default_parameter_storage must be ParameterStorage")
        if not self.default_parameter_storage.complete:
            raise ValueError("the default storage must set the group and every component")
        for field_name, kinds in (("parameter_placements", (Replicated, Sharded)),
                                  ("parameter_storage", (ParameterStorage,))):
            table = dict(getattr(self, field_name))
            for sel, v in table.items():
                if not isinstance(sel, str) or not sel:
                    raise ValueError(f"{field_name}: selectors must be non-empty names")
                if not isinstance(v, kinds):
                    raise TypeError(f"{field_name}[{sel!r}]: invalid declaration")
            object.__setattr__(self, field_name, table)
        named = [self.default_parameter_placement.group, self.default_parameter_storage.group]
        named += [p.group for p in self.parameter_placements.values()]
        named += [s.group for s in self.parameter_storage.values() if s.group is not None]
        for g in named:
            if g not in self.groups:
                raise ValueError(f"unknown group {g!r}")
        if self.inputs not in ("per_rank", "split_microbatches"):
            raise ValueError("inputs must be 'per_rank' or 'split_microbatches'")

    # ------------------------------------------------------------------ geometry
    @property
    def world_size(self) -> int:
        return self.ranks_per_replica * self.num_replicas

    def replica_of(self, rank: int) -> tuple[int, int]:
        """``(replica index, rank within the replica)``."""
        if not 0 <= rank < self.world_size:
            raise ValueError(f"rank {rank} outside a world of {self.world_size}")
        return divmod(rank, self.ranks_per_replica)

    # ------------------------------------------------------------------ selection
    @staticmethod
    def _pick(table: Mapping[str, Any], name: str):
        if name in table:
            return table[name]
        hits = [s for s in table if fnmatch.fnmatchcase(name, s)]
        return table[max(hits, key=len)] if hits else None

    def resolve(self, name: str, rank: int, nbytes: int | None = None) -> ResolvedParameter:
        """Ownership of parameter ``name`` on global ``rank``. Tensors smaller than
        ``min_shard_bytes`` keep their storage whole on every rank."""
        replica, local = self.replica_of(rank)
        base = replica * self.ranks_per_replica
        placement = self._pick(self.parameter_placements, name) or self.default_parameter_placement
        override = self._pick(self.parameter_storage, name)
        storage = override.over(self.default_parameter_storage) if override \
            else self.default_parameter_storage
        if nbytes is not None and nbytes < self.min_shard_bytes:
            storage = replace(storage, weights="replicated", gradients="replicated",
                              optimizer="replicated")
        cg = self.groups[placement.group].group_of(local)
        sg = self.groups[storage.group].group_of(local)
        if isinstance(placement, Sharded) and placement.stored == "local":
            # a locally stored slice belongs to this rank alone: its stored components
            # are not divided further and its gradients need no reduction
            sg = (local,)
        return ResolvedParameter(name, placement, storage, tuple(base + r for r in cg),
                                 tuple(base + r for r in sg),
                                 cg.index(local) if isinstance(placement, Sharded) else 0,
                                 sg.index(local))

    # ------------------------------------------------------------------ records
    def to_json(self) -> dict[str, Any]:
        def place(p: Placement) -> dict[str, Any]:
            if isinstance(p, Sharded):
                return {"sharded": p.group, "dim": p.dim, "stored": p.stored}
            return {"replicated": p.group}

        def store(s: ParameterStorage) -> dict[str, Any]:
            return {k: getattr(s, k) for k in ("group", "weights", "gradients", "optimizer")
                    if getattr(s, k) is not None}
        return {"ranks_per_replica": self.ranks_per_replica, "num_replicas": self.num_replicas,
                "groups": {n: [list(g) for g in r.groups] for n, r in self.groups.items()},
                "default_parameter_placement": place(self.default_parameter_placement),
                "parameter_placements": {k: place(v) for k, v in self.parameter_placements.items()},
                "default_parameter_storage": store(self.default_parameter_storage),
                "parameter_storage": {k: store(v) for k, v in self.parameter_storage.items()},
                "min_shard_bytes": self.min_shard_bytes, "inputs": self.inputs}

    @staticmethod
    def from_json(d: Mapping[str, Any]) -> "Parallelism":
        def place(r: Mapping[str, Any]) -> Placement:
            if "sharded" in r:
                return Sharded(r["sharded"], int(r.get("dim", 0)), r.get("stored", "local"))
            return Replicated(r.get("replicated", "all_ranks"))
        return Parallelism(
            int(d.get("ranks_per_replica", 1)), int(d.get("num_replicas", 1)),
            {k: tuple(tuple(g) for g in v) for k, v in d.get("groups", {}).items()},
            place(d.get("default_parameter_placement", {})),
            {k: place(v) for k, v in d.get("parameter_placements", {}).items()},
            ParameterStorage(**d.get("default_parameter_storage",
                                     {"group": "all_ranks", "weights": "sharded",
                                      "gradients": "sharded", "optimizer": "sharded"})),
            {k: ParameterStorage(**v) for k, v in d.get("parameter_storage", {}).items()},
            int(d.get("min_shard_bytes", MIN_SHARD_BYTES)), d.get("inputs", "per_rank"))


def data_parallel(ranks: int, *, weights: str = "sharded", gradients: str = "sharded",
                  optimizer: str = "sharded", replicas: int = 1,
                  min_shard_bytes: int = MIN_SHARD_BYTES) -> Parallelism:
    """All state divided over (or copied on) every rank of a replica; batches split
    by microbatch. Sharded weights or gradients imply sharded optimizer state."""
    if "sharded" in (weights, gradients) and optimizer != "sharded":
        raise ValueError("optimizer state must shard with sharded weights or gradients")
    return Parallelism(ranks, replicas,
                       default_parameter_storage=ParameterStorage("all_ranks", weights, gradients,
                                                                  optimizer),
                       min_shard_bytes=min_shard_bytes, inputs="split_microbatches")


def expert_parallel(ranks: int, *, n_experts: int, top_k: int,
                    expert_selector: str = "*.experts.*",
                    min_shard_bytes: int = MIN_SHARD_BYTES) -> Parallelism:
    """Expert banks sharded on dimension 0 and stored locally; everything else
    replicated for compute with sharded optimizer state
    (packages/client/src/shadowspill_client/parallelism.py:60-120)."""
    if not 2 <= ranks <= 128:
        raise ValueError("expert parallelism needs 2 to 128 ranks")
    if n_experts % ranks:
        raise ValueError("n_experts must be divisible by the number of ranks")
    if not 1 <= top_k <= 32:
        raise ValueError("top_k must be between 1 and 32")
    return Parallelism(ranks, 1,
                       parameter_placements={expert_selector: Sharded("all_ranks", 0, "local")},
                       default_parameter_storage=ParameterStorage("all_ranks", "replicated",
                                                                  "replicated", "sharded"),
                       min_shard_bytes=min_shard_bytes, inputs="per_rank")


def from_client_record(record: Mapping[str, Any]) -> Parallelism:
    """Turns the client's plain-dict declaration (``client.parallelism``) into a spec."""
    kind = record.get("kind")
    if kind == "data_parallel":
        st = record.get("storage", {})
        return data_parallel(int(record["ranks_per_replica"]), weights=st.get("weights", "sharded"),
                             gradients=st.get("gradients", "sharded"),
                             optimizer=st.get("optimizer", "sharded"),
                             replicas=int(record.get("num_replicas", 1)),
                             min_shard_bytes=int(record.get("min_shard_bytes", MIN_SHARD_BYTES)))
    if kind == "expert_parallel":
        ranks = int(record["ranks_per_replica"])
        return expert_parallel(ranks, n_experts=int(record["experts_per_rank"]) * ranks, top_k=1,
                               min_shard_bytes=int(record.get("min_shard_bytes", MIN_SHARD_BYTES)))
    return Parallelism.from_json(record)
