"""Training settings: ``Model``, ``Weights``, ``LoRA``, ``Objective``, ``Optimizer``,
``BatchConfig``, ``Memory``, ``Execution``, ``Preparation`` and friends.

The names and meanings follow the reference client
(packages/client/src/shadowspill_client/config/{model,batch,execution,preparation,
resources,operations}.py); every record is frozen, validated and serialises to
plain JSON.
"""
from __future__ import annotations

from typing import Any

from ._records import record, require


@record
class Weights:
    source: str = "random"          # random | checkpoint | artifact
    seed: int = 0
    location: str = ""              # checkpoint directory or artifact id

    @staticmethod
    def random(seed: int = 0) -> "Weights":
        return Weights("random", seed)

    @staticmethod
    def checkpoint(location: str) -> "Weights":
        return Weights("checkpoint", 0, location)

    @staticmethod
    def artifact(artifact_id: str) -> "Weights":
        return Weights("artifact", 0, artifact_id)

    def validate(self):
        require(self.source in ("random", "checkpoint", "artifact"), f"unknown weights source {self.source!r}")
        require(self.source == "random" or bool(self.location), "weights location is required")


@record
class LoRA:
    rank: int = 16
    alpha: float = 32.0
    targets: tuple = ("attention", "experts")

    def validate(self):
        require(self.rank > 0, "LoRA rank must be positive")


@record
class Model:
    name: str = "llama3-8b"                   # catalog name <family>-<size>
    config: dict | None = None                # explicit architecture (overrides the catalog)
    weights: Weights = Weights()
    lora: LoRA | None = None
    dtype: str = "bfloat16"

    @staticmethod
    def from_pretrained(location: str, name: str) -> "Model":
        return Model(name=name, weights=Weights.checkpoint(location))

    def validate(self):
        require(bool(self.name) or self.config is not None, "a model needs a name or a config")
        require(self.dtype in ("bfloat16", "float32"), f"unsupported dtype {self.dtype!r}")


@record
class Objective:
    id: str = "shadowspill/cross_entropy@1"
    config: dict | None = None
    terms: tuple = ()

    @staticmethod
    def sum(*terms: "Objective") -> "Objective":
        return Objective("shadowspill/sum@1", None, tuple(terms))

    def validate(self):
        require("@" in self.id, "objective ids are versioned: name@version")


@record
class Optimizer:
    id: str = "adamw@1"
    lr: float = 1e-4
    beta1: float = 0.9
    beta2: float = 0.95
    eps: float = 1e-8
    weight_decay: float = 0.0
    gradient_dtype: str = "bfloat16"
    opt_state_dtype: str = "bfloat16"
    master_dtype: str = "bfloat16"
    parameter_rounding: str = "stochastic"    # nearest | stochastic
    opt_state_rounding: str = "stochastic"
    # first match wins: ({"match": ["*norm*"], "weight_decay": 0.0}, {"match": ["embed.*"], "lr_scale": 0.1})
    parameter_groups: tuple = ()

    def validate(self):
        require(self.lr >= 0 and 0 <= self.beta1 < 1 and 0 <= self.beta2 < 1, "bad AdamW hyperparameters")
        require(self.parameter_rounding in ("nearest", "stochastic"), "bad parameter_rounding")
        require(self.opt_state_rounding in ("nearest", "stochastic"), "bad opt_state_rounding")
        for g in self.parameter_groups:
            require(isinstance(g, dict) and g.get("match") and all(isinstance(m, str) for m in g["match"]),
                    "a parameter group needs 'match': a list of name patterns")
            require(set(g) <= {"match", "lr_scale", "weight_decay"}, "parameter group keys: match, lr_scale, weight_decay")


@record
class BatchConfig:
    tokens_per_step: int = 65536              # per worker
    microbatch_tokens: int = 8192
    max_datums: int = 0                       # 0 = derived from the microbatch size
    packing: str = "best_fit"                 # best_fit | balanced

    def validate(self):
        require(self.microbatch_tokens > 0 and self.tokens_per_step % self.microbatch_tokens == 0,
                "tokens_per_step must be a positive multiple of microbatch_tokens")
        require(self.packing in ("best_fit", "balanced"), "unknown packing policy")

    @property
    def microbatches(self) -> int:
        return self.tokens_per_step // self.microbatch_tokens


@record
class Memory:
    device_gib: float = 0.0                   # 0 = automatic: 90 % of the device
    spill_gib: float = 0.0                    # 0 = automatic: 90 % of free host memory
    # where spilled state lives: "host" (pinned memory), "file" (a direct-I/O file on a local
    # drive of the worker's node) or "remote" (memory of an ss_memory_daemon); the last two are
    # staged through small pinned rings
    spill_pool: str = "host"
    spill_address: str = ""                   # "remote": host:port of the memory daemon
    spill_directory: str = ""                 # "file": existing directory for the scratch file
    spill_chunk_bytes: int = 2 << 20          # "file": staged piece of a transfer, multiple of 4096
    spill_queue_depth: int = 16               # "file": chunks staged at once per direction

    def validate(self):
        require(self.device_gib >= 0 and self.spill_gib >= 0, "memory budgets are non-negative")
        require(self.spill_pool in ("host", "file", "remote"), "spill_pool is 'host', 'file' or 'remote'")
        if self.spill_pool == "remote":
            require(":" in self.spill_address, "a remote spill pool needs spill_address = host:port")
        if self.spill_pool == "file":
            require(bool(self.spill_directory), "a file spill pool needs spill_directory")
        if self.spill_pool != "host":
            require(self.spill_gib > 0, "a file or remote spill pool needs an explicit spill_gib")
            require(self.spill_chunk_bytes > 0 and self.spill_chunk_bytes % 4096 == 0
                    and self.spill_chunk_bytes <= 1 << 30, "spill_chunk_bytes: multiple of 4096, at most 1 GiB")
            require(1 <= self.spill_queue_depth <= 1024, "spill_queue_depth is between 1 and 1024")


@record
class Execution:
    seed: int = 0
    max_staging_bytes: int = 1 << 30
    max_pending_requests: int = 8
    idle_timeout_seconds: float = 0.0         # 0 = never
    runtime_trace: bool = False
    profiler_annotations: bool = False
    reject_overbudget: bool = True
    nsys: dict | None = None                  # {start_step, steps, gpu_metrics}: Nsight capture of a few
                                              # steps where the node has nsys (orchestration/capture.py)
    collectives: str = "auto"                 # peer | dist | auto
    observe_norms: bool = False               # every update's result carries grad_norm and param_norm (one worker)


@record
class Policy:
    id: str
    config: dict | None = None


@record
class BuildOptions:
    walks: tuple = ("breadth",)
    recompute_shares: tuple = (100,)
    saved_variant: str = "save_attention"
    projection_chunks: tuple = ()
    moe_chunks: tuple = ()
    # "stages": the hand-written stage classes; "graph": torch.export -> partition -> AOT graph pairs
    frontend: str = "stages"


@record
class ProfilingOptions:
    enabled: bool = True
    min_samples: int = 3
    max_samples: int = 8
    tolerance: float = 0.03


@record
class PlanningOptions:
    strategies: tuple = ("stall", "traffic")
    fetch_rules: tuple = ("demand", "latest-safe", "packed-fifo", "packed-fit")
    workers: int = 0
    max_repairs: int = 16
    minimum_object_bytes_evict_eligible: int = 1 << 20
    deterministic: bool = False
    collective_overhead_us: float = 0.0       # planned cost added to every communication-stream task


@record
class Preparation:
    build: BuildOptions = BuildOptions()
    profiling: ProfilingOptions = ProfilingOptions()
    planning: PlanningOptions = PlanningOptions()
    policies: tuple = ()
    calibrate: bool = True
    # run build / profile / communicate / plan as four fresh processes before the workers start
    separate_processes: bool = False


@record
class Resources:
    gpus: int = 1
    node: str = ""                            # "" = the service's own node
    backend: str = "cuda"                     # cuda | cpu (mock backend, functional runs)


@record
class Operation:
    name: str                                 # step | forward_backward | forward | optim_step
    enabled: bool = True


def training_setup(model: Model, optimizer: Optimizer = Optimizer(), objective: Objective = Objective(),
                   batch: BatchConfig = BatchConfig(), memory: Memory = Memory(),
                   execution: Execution = Execution(), preparation: Preparation = Preparation(),
                   resources: Resources = Resources(), parallelism: dict | None = None,
                   operations: tuple = ("step",)) -> dict[str, Any]:
    """The JSON body of a run-creation request."""
    return {"model": model.to_json(), "optimizer": optimizer.to_json(),
            "objective": objective.to_json(), "batch": batch.to_json(), "memory": memory.to_json(),
            "execution": execution.to_json(), "preparation": preparation.to_json(),
            "resources": resources.to_json(), "parallelism": parallelism or {},
            "operations": list(operations)}
