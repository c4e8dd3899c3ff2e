"""B200-native memory-budgeted training runtime.

Public phase API (lazy): ``build_step``, ``measure_program``, ``plan_program``,
``Executor``, ``save_checkpoint`` / ``load_checkpoint``, ``write_report`` and the
client/server entry points. Importing the package itself is cheap and needs no GPU.
"""
from __future__ import annotations

import importlib

__version__ = "0.1.0"

_PUBLIC = {
    # models / ops
    "preset": ("shadowspill_b200.models.config", "preset"),
    "DecoderConfig": ("shadowspill_b200.models.config", "DecoderConfig"),
    "build_stages": ("shadowspill_b200.models.decoder", "build_stages"),
    # phase API
    "build_step": ("shadowspill_b200.frontend.capture", "build_step"),
    "build_forward": ("shadowspill_b200.frontend.capture", "build_forward"),
    "build_forward_backward": ("shadowspill_b200.frontend.capture", "build_forward_backward"),
    "measure_program": ("shadowspill_b200.profiling.measure", "measure_program"),
    "apply_profiles": ("shadowspill_b200.profiling.measure", "apply_profiles"),
    "measure_communication": ("shadowspill_b200.communication.measure", "measure_communication"),
    "CommunicationInfo": ("shadowspill_b200.communication.info", "CommunicationInfo"),
    "plan_program": ("shadowspill_b200.planning.plan", "plan_program"),
    "sweep_programs": ("shadowspill_b200.planning.plan", "sweep_programs"),
    "SearchOptions": ("shadowspill_b200.planning.plan", "SearchOptions"),
    "PlanningInputs": ("shadowspill_b200.planning.offline", "PlanningInputs"),
    "simulate": ("shadowspill_b200.simulator.api", "simulate"),
    "Executor": ("shadowspill_b200.execution.executor", "Executor"),
    "ResidentTrainer": ("shadowspill_b200.execution.resident", "ResidentTrainer"),
    "save_checkpoint": ("shadowspill_b200.checkpoint.save", "save_checkpoint"),
    "load_checkpoint": ("shadowspill_b200.checkpoint.load", "load_checkpoint"),
    "write_report": ("shadowspill_b200.reporting.write", "write_report"),
    "Parallelism": ("shadowspill_b200.parallelism.spec", "Parallelism"),
    "Sharded": ("shadowspill_b200.parallelism.spec", "Sharded"),
    "Replicated": ("shadowspill_b200.parallelism.spec", "Replicated"),
    "Program": ("shadowspill_b200.ir.program", "Program"),
    "Plan": ("shadowspill_b200.ir.plan", "Plan"),
    # service
    "Server": ("shadowspill_b200.server.service", "Server"),
    "ServiceClient": ("shadowspill_b200.client.service", "ServiceClient"),
}


def __getattr__(name: str):
    try:
        module, attr = _PUBLIC[name]
    except KeyError:
        raise AttributeError(f"module {__name__!r} has no attribute {name!r}") from None
    value = getattr(importlib.import_module(module), attr)
    globals()[name] = value
    return value


def __dir__():
    return sorted(list(globals()) + list(_PUBLIC))
