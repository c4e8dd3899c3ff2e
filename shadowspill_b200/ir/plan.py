"""Memory schedule and execution plan.

``MemorySchedule`` is the ordered list of fetch / evict / release actions, each
issued when its trigger task completes (the reference's ``MemorySchedule`` /
``MemoryAction``, packages/engine/src/shadowspill/ir/schedule.py:55-277).
``Plan`` binds a program and a schedule to a physical layout: one fixed device
offset per device stay, one spill offset per object that ever lives in the
spill pool, and the reuse dependencies the layout implies (the reference's
``ExecutionPlan`` + fixed-layout certificate, ir/execution.py:345).
"""
from __future__ import annotations

import ctypes as C
from dataclasses import asdict, dataclass, field
from typing import Any

import numpy as np

from .. import native
from .program import Program

ACTION_KINDS = ("fetch", "evict", "release")


@dataclass
class MemoryAction:
    kind: str
    object: int
    trigger_task: int      # -1 = step start


@dataclass
class Stay:
    """One residency of an object in the device pool."""
    object: int
    begin_action: int      # fetch index, or -1 when a task creates it
    begin_task: int
    end_action: int
    bytes: int
    start_ns: int
    end_ns: int
    offset: int


@dataclass
class MemorySchedule:
    actions: list[MemoryAction] = field(default_factory=list)

    def to_native(self):
        arr = (native.Action * max(1, len(self.actions)))()
        for i, a in enumerate(self.actions):
            arr[i] = native.Action(ACTION_KINDS.index(a.kind), a.object, a.trigger_task, 0)
        return arr

    def bytes_moved(self, program: Program) -> tuple[int, int]:
        f = sum(program.objects[a.object].bytes for a in self.actions if a.kind == "fetch")
        e = sum(program.objects[a.object].bytes for a in self.actions if a.kind == "evict")
        return f, e


@dataclass
class PlanSummary:
    duration_seconds: float = 0.0
    compute_seconds: float = 0.0
    input_wait_seconds: float = 0.0
    capacity_wait_seconds: float = 0.0
    execution_peak_bytes: int = 0
    layout_span_bytes: int = 0
    workspace_bytes: int = 0
    fixed_device_bytes: int = 0
    spill_peak_bytes: int = 0
    fetch_bytes: int = 0
    evict_bytes: int = 0
    tokens: int = 0
    tokens_per_second: float = 0.0
    strategy: str = ""
    fetch_rule: str = ""
    selection: str = ""
    ordering: str = ""
    candidates_evaluated: int = 0
    candidates_feasible: int = 0
    repairs_applied: int = 0
    logical_capacity_bytes: int = 0
    simulation_only: bool = False
    logical_ranks: int = 1


@dataclass
class Plan:
    program: Program
    schedule: MemorySchedule
    stays: list[Stay]
    spill_offsets: list[int]                 # per object, -1 = never in spill
    reuse_pred_begin: list[int]
    reuse_pred_index: list[int]
    task_start_ns: list[int]
    task_end_ns: list[int]
    action_start_ns: list[int]
    action_end_ns: list[int]
    device_bytes: int                        # pool extent the layout needs (span)
    spill_bytes: int
    budgets: dict[str, int] = field(default_factory=dict)
    summary: PlanSummary = field(default_factory=PlanSummary)
    communication: dict[str, Any] = field(default_factory=dict)
    # homes in the file-backed pool (per object, -1 = not there); empty = no file pool.
    # An object has one home: a non-negative entry here means spill_offsets[o] == -1.
    file_offsets: list[int] = field(default_factory=list)
    file_bytes: int = 0

    def home_pool(self, obj: int) -> str:
        """``"file"``, ``"host"`` or ``""`` (the object never leaves the device)."""
        if self.file_offsets and self.file_offsets[obj] >= 0:
            return "file"
        return "host" if self.spill_offsets[obj] >= 0 else ""

    def to_json(self) -> dict[str, Any]:
        return {"format": "ss-b200.plan", "version": 1, "program": self.program.to_json(),
                "actions": [asdict(a) for a in self.schedule.actions],
                "stays": [asdict(s) for s in self.stays], "spill_offsets": self.spill_offsets,
                "reuse_pred_begin": self.reuse_pred_begin,
                "reuse_pred_index": self.reuse_pred_index,
                "task_start_ns": self.task_start_ns, "task_end_ns": self.task_end_ns,
                "action_start_ns": self.action_start_ns, "action_end_ns": self.action_end_ns,
                "device_bytes": self.device_bytes, "spill_bytes": self.spill_bytes,
                "budgets": self.budgets, "summary": asdict(self.summary),
                "communication": self.communication, "file_offsets": self.file_offsets,
                "file_bytes": self.file_bytes}

    @staticmethod
    def from_json(d: dict[str, Any]) -> "Plan":
        if d.get("format") != "ss-b200.plan" or d.get("version") != 1:
            raise ValueError("not a version-1 plan")
        return Plan(Program.from_json(d["program"]),
                    MemorySchedule([MemoryAction(**a) for a in d["actions"]]),
                    [Stay(**s) for s in d["stays"]], list(d["spill_offsets"]),
                    list(d["reuse_pred_begin"]), list(d["reuse_pred_index"]),
                    list(d["task_start_ns"]), list(d["task_end_ns"]),
                    list(d["action_start_ns"]), list(d["action_end_ns"]),
                    int(d["device_bytes"]), int(d["spill_bytes"]), dict(d.get("budgets", {})),
                    PlanSummary(**d.get("summary", {})), dict(d.get("communication", {})),
                    list(d.get("file_offsets", [])), int(d.get("file_bytes", 0)))

    def to_native_desc(self):
        """``(native.PlanDesc, keepalive)`` for ``ss_plan_admit``."""
        prog, keep = self.program.to_native()
        acts = self.schedule.to_native()
        ivs = (native.Interval * max(1, len(self.stays)))()
        for i, s in enumerate(self.stays):
            ivs[i] = native.Interval(s.object, s.begin_action, s.begin_task, s.end_action, s.bytes,
                                     s.start_ns, s.end_ns, s.offset)
        ob = native.as_i64([o.bytes for o in self.program.objects])
        so = native.as_i64(self.spill_offsets)
        pb, pi = native.as_i32(self.reuse_pred_begin), native.as_i32(self.reuse_pred_index or [0])
        fo = native.as_i64(self.file_offsets) if self.file_offsets else None
        desc = native.PlanDesc(prog.n_tasks, prog.n_objects, native.ptr64(ob), native.ptr64(so),
                               len(self.schedule.actions), acts, len(self.stays), ivs,
                               native.ptr32(pb), native.ptr32(pi), prog.n_uses, prog.use_task,
                               prog.use_object, prog.use_mode,
                               native.ptr64(fo) if fo is not None else None)
        return desc, (keep, acts, ivs, ob, so, pb, pi, fo)
