"""Framework-neutral program IR: objects, tasks, uses and alternatives.

A *Program* is one training (or forward) invocation unrolled over stages and
microbatches in a fixed order. Objects are byte ranges with a home (the spill
pool for persistent state, nowhere for transients); tasks are opaque stage
executions with measured durations; a *use* says how a task touches an object.
The structure follows the reference's ``ShadowSpillProgram`` / ``ObjectSpec`` /
``TaskSpec`` (packages/engine/src/shadowspill/ir/program/specs.py:37-652),
reduced to what one CUDA backend with stage-granular tasks needs.
"""
from __future__ import annotations

import hashlib
import json
from dataclasses import asdict, dataclass, field
from typing import Any

import numpy as np

from .. import native

OBJECT_KINDS = ("weight", "optimizer_state", "gradient", "activation", "saved", "input",
                "activation_gradient", "output")
TASK_KINDS = ("forward", "backward", "head", "optimizer", "control", "collective")
USE_MODES = {"read": native.USE_READ, "create": native.USE_CREATE, "mutate": native.USE_MUTATE}


@dataclass
class ObjectSpec:
    name: str
    bytes: int
    kind: str
    persistent: bool = False         # home is the spill pool at invocation boundaries
    pinned_resident: bool = False    # never cut by the planner
    stage: int = -1
    microbatch: int = -1
    dtype: str = "uint8"
    shape: tuple[int, ...] = ()
    sharding: str = "whole"          # whole | sharded | replicated (data-parallel storage)

    def __post_init__(self):
        if self.kind not in OBJECT_KINDS:
            raise ValueError(f"unknown object kind {self.kind!r}")
        if self.bytes < 0:
            raise ValueError("object bytes must be non-negative")
        self.shape = tuple(self.shape)


@dataclass
class UseSpec:
    object: int
    mode: str                        # read | create | mutate
    role: str = ""                   # how the task refers to it (e.g. "params", "x", "dy")


@dataclass
class TaskSpec:
    name: str
    kind: str
    stage: int = -1
    microbatch: int = -1
    uses: list[UseSpec] = field(default_factory=list)
    duration_ns: int = 0
    workspace_bytes: int = 0
    variant: str = ""                # e.g. "save" / "recompute" / "save_attention"
    group: int = -1                  # alternative group (forward/backward pair), -1 = none
    flops: float = 0.0
    tokens: int = 0
    profile_key: str = ""            # tasks with the same key share one measured profile
    # the task's allocation contract: sizes of the tensor allocations it makes, in order, as
    # recorded when it was profiled under the allocation adapter (empty = not recorded)
    allocations: list[int] = field(default_factory=list)

    def __post_init__(self):
        if self.kind not in TASK_KINDS:
            raise ValueError(f"unknown task kind {self.kind!r}")
        self.uses = [u if isinstance(u, UseSpec) else UseSpec(**u) for u in self.uses]


@dataclass
class Program:
    objects: list[ObjectSpec] = field(default_factory=list)
    tasks: list[TaskSpec] = field(default_factory=list)
    metadata: dict[str, Any] = field(default_factory=dict)

    # ---- construction helpers
    def add_object(self, spec: ObjectSpec) -> int:
        self.objects.append(spec)
        return len(self.objects) - 1

    def add_task(self, spec: TaskSpec) -> int:
        self.tasks.append(spec)
        return len(self.tasks) - 1

    def object_index(self, name: str) -> int:
        for i, o in enumerate(self.objects):
            if o.name == name:
                return i
        raise KeyError(name)

    # ---- validation
    def validate(self) -> None:
        created: set[int] = set()
        names = set()
        for o in self.objects:
            if o.name in names:
                raise ValueError(f"duplicate object name {o.name!r}")
            names.add(o.name)
        for ti, t in enumerate(self.tasks):
            seen = set()
            for u in t.uses:
                if not 0 <= u.object < len(self.objects):
                    raise ValueError(f"task {t.name}: object index {u.object} out of range")
                if u.object in seen:
                    raise ValueError(f"task {t.name}: object used twice")
                seen.add(u.object)
                if u.mode not in USE_MODES:
                    raise ValueError(f"task {t.name}: unknown use mode {u.mode!r}")
                obj = self.objects[u.object]
                if u.mode == "create":
                    if obj.persistent:
                        raise ValueError(f"task {t.name}: persistent object {obj.name} created")
                    if u.object in created:
                        raise ValueError(f"task {t.name}: {obj.name} created twice")
                    created.add(u.object)
                elif not obj.persistent and u.object not in created:
                    raise ValueError(f"task {t.name} (#{ti}): {obj.name} used before creation")

    # ---- flat arrays for the native core
    def to_native(self):
        """Returns ``(native.Program, keepalive)``; keep ``keepalive`` referenced
        for as long as the structure is in use."""
        dur = native.as_i64([t.duration_ns for t in self.tasks])
        ws = native.as_i64([t.workspace_bytes for t in self.tasks])
        ob = native.as_i64([o.bytes for o in self.objects])
        fl = native.as_i32([(native.OBJ_PERSISTENT if o.persistent else 0)
                            | (native.OBJ_PINNED_RESIDENT if o.pinned_resident else 0)
                            for o in self.objects])
        ut, uo, um = [], [], []
        for ti, t in enumerate(self.tasks):
            for u in sorted(t.uses, key=lambda u: u.object):
                ut.append(ti); uo.append(u.object); um.append(USE_MODES[u.mode])
        ut, uo, um = native.as_i32(ut), native.as_i32(uo), native.as_i32(um)
        p = native.Program(len(self.tasks), native.ptr64(dur), native.ptr64(ws), len(self.objects),
                           native.ptr64(ob), native.ptr32(fl), len(ut), native.ptr32(ut),
                           native.ptr32(uo), native.ptr32(um))
        return p, (dur, ws, ob, fl, ut, uo, um)

    def sorted_uses(self, task: int) -> list[UseSpec]:
        """Uses of a task in the order the native runtime reports device pointers."""
        return sorted(self.tasks[task].uses, key=lambda u: u.object)

    # ---- serialisation
    def to_json(self) -> dict[str, Any]:
        return {"format": "ss-b200.program", "version": 1,
                "objects": [asdict(o) for o in self.objects],
                "tasks": [asdict(t) for t in self.tasks], "metadata": self.metadata}

    @staticmethod
    def from_json(d: dict[str, Any]) -> "Program":
        if d.get("format") != "ss-b200.program" or d.get("version") != 1:
            raise ValueError("not a version-1 program")
        return Program([ObjectSpec(**o) for o in d["objects"]],
                       [TaskSpec(**t) for t in d["tasks"]], dict(d.get("metadata", {})))

    def digest(self) -> str:
        blob = json.dumps(self.to_json(), sort_keys=True, default=str).encode()
        return hashlib.sha256(blob).hexdigest()

    # ---- summaries
    def total_compute_ns(self) -> int:
        return sum(t.duration_ns for t in self.tasks)

    def persistent_bytes(self) -> int:
        return sum(o.bytes for o in self.objects if o.persistent)
