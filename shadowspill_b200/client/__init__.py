"""Client package: NumPy-only API to a training service.

    from shadowspill_b200.client import ServiceClient, Model, Optimizer, Memory, BatchConfig
    with ServiceClient("http://127.0.0.1:8765") as svc:
        trainer = svc.create_training_client(Model("llama3-8b"), Optimizer(lr=1e-4),
                                             memory=Memory(24, 128)).result()
        result = trainer.step(text_batch(sequences)).result()
"""
from .config import (BatchConfig, BuildOptions, Execution, LoRA, Memory, Model, Objective,  # noqa: F401
                     Operation, Optimizer, PlanningOptions, Policy, Preparation, ProfilingOptions,
                     Resources, Weights)
from .display import BatchStatistics, CommandTable, LengthStatistics  # noqa: F401
from .metrics import MetricPage, MetricQueries  # noqa: F401
from .packing import (Assignment, BatchError, BatchValidation, BatchValidator, CoverageBound,  # noqa: F401
                      assign_bins, pack_batch)
from .parallelism import MIN_SHARD_BYTES, data_parallel, expert_parallel  # noqa: F401
from .schedules import Constant, WarmupCosine  # noqa: F401
from .service import ServiceClient  # noqa: F401
from .transport import SSH, SSHTunnel, TransportError  # noqa: F401
from .text import (Datum, build_candidates, policy_datum, tensor_datum, text_batch,  # noqa: F401
                   text_batch_statistics, text_datum)
from .training import OperationFailed, TrainingClient, TrainingResult  # noqa: F401
