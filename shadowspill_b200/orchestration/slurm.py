"""Read-only facts about the Slurm job this process runs in; an allocation is never made.

``detect()`` reads the job's environment (``SLURM_JOB_ID`` and friends); ``parse_job`` reads
the JSON that ``scontrol show job <id> --json`` prints, bounded in size and checked against
the job and owner it was asked for. ``device_inventory`` uses the result to offer a run only
what the job was given: a node of a 4-GPU, 200 GB allocation is not an 8-GPU, 2 TB node.

Reference: packages/engine/src/shadowspill/orchestration/launch/slurm_job.py:1-120
("bounded read-only facts for an existing Slurm job").
"""
from __future__ import annotations

import json
import os
import re
from dataclasses import dataclass, field
from typing import Mapping

MAX_RESPONSE_BYTES = 4 << 20
MAX_NODES = 4096
_NAME = re.compile(r"^[A-Za-z0-9][A-Za-z0-9._-]{0,254}$")


@dataclass(frozen=True)
class SlurmNode:
    name: str
    cpus: int = 0
    memory_mib: int = 0
    gpus: int = 0

    def __post_init__(self):
        if not _NAME.match(self.name):
            raise ValueError(f"bad Slurm node name {self.name!r}")


@dataclass(frozen=True)
class SlurmJob:
    job_id: int
    user_id: int
    nodes: Mapping[str, SlurmNode] = field(default_factory=dict)

    def __post_init__(self):
        if self.job_id < 1:
            raise ValueError("an existing Slurm job has a positive id")
        if not self.nodes or len(self.nodes) > MAX_NODES:
            raise ValueError("a Slurm job has a bounded, non-empty node allocation")
        if any(name != node.name for name, node in self.nodes.items()):
            raise ValueError("Slurm node records differ from their names")


def expand_hostlist(expr: str) -> list[str]:
    """``node[01-03,07],gpu5`` -> ``[node01, node02, node03, node07, gpu5]``."""
    out, depth, cur = [], 0, ""
    parts = []
    for ch in expr:
        if ch == "," and depth == 0:
            parts.append(cur); cur = ""
            continue
        depth += ch == "["
        depth -= ch == "]"
        cur += ch
    if cur:
        parts.append(cur)
    for part in parts:
        m = re.match(r"^([^\[\]]*)\[([^\]]+)\](.*)$", part)
        if not m:
            out.append(part)
            continue
        head, body, tail = m.groups()
        for piece in body.split(","):
            if "-" in piece:
                lo, hi = piece.split("-", 1)
                if int(hi) - int(lo) >= MAX_NODES:
                    raise ValueError("host range too large")
                out += [f"{head}{str(i).zfill(len(lo))}{tail}" for i in range(int(lo), int(hi) + 1)]
            else:
                out.append(f"{head}{piece}{tail}")
        if len(out) > MAX_NODES:
            raise ValueError("host list too large")
    return out


def _gpu_count(value: str) -> int:
    """``4``, ``gpu:4``, ``gpu:b200:4`` or an index list ``0,1,2,3``."""
    value = value.strip()
    if not value:
        return 0
    if re.fullmatch(r"\d+(,\d+)+", value):
        return len(value.split(","))
    tail = value.split(":")[-1].split("(")[0]
    return int(tail) if tail.isdigit() else 0


def detect(env: Mapping[str, str] | None = None) -> SlurmJob | None:
    """The job of this process from its environment, or ``None`` outside Slurm."""
    env = os.environ if env is None else env
    if not env.get("SLURM_JOB_ID", "").isdigit():
        return None
    names = expand_hostlist(env.get("SLURM_JOB_NODELIST", env.get("SLURM_NODELIST", ""))) \
        or [env.get("SLURMD_NODENAME", "localhost")]
    cpus = int(env.get("SLURM_CPUS_ON_NODE", "0") or 0)
    mem = int(env.get("SLURM_MEM_PER_NODE", "0") or 0)
    gpus = _gpu_count(env.get("SLURM_GPUS_ON_NODE", "") or env.get("SLURM_JOB_GPUS", "")
                      or env.get("SLURM_STEP_GPUS", ""))
    nodes = {n: SlurmNode(n, cpus, mem, gpus) for n in names}
    uid = int(env.get("SLURM_JOB_UID", str(os.getuid())) or os.getuid())
    return SlurmJob(int(env["SLURM_JOB_ID"]), uid, nodes)


def parse_job(data: bytes, *, job_id: int, user_id: int) -> SlurmJob:
    """``scontrol show job <job_id> --json`` -> ``SlurmJob``; anything unexpected is an error."""
    if len(data) > MAX_RESPONSE_BYTES:
        raise ValueError("Slurm job response exceeds its byte bound")
    doc = json.loads(data)
    if doc.get("errors"):
        raise ValueError("Slurm returned scheduler errors")
    jobs = doc.get("jobs") or []
    if len(jobs) != 1:
        raise ValueError("the Slurm query must identify exactly one existing job")
    job = jobs[0]
    if int(job.get("job_id", -1)) != job_id:
        raise ValueError("the Slurm response belongs to a different job")
    if int(job.get("user_id", -1)) != user_id:
        raise ValueError("the Slurm job belongs to a different user")
    res = job.get("job_resources") or {}
    alloc = res.get("nodes")
    alloc = alloc.get("allocation", []) if isinstance(alloc, dict) else (res.get("allocated_nodes") or [])
    gres = str(job.get("gres_detail", [""])[0] if isinstance(job.get("gres_detail"), list) and job.get("gres_detail")
               else job.get("tres_per_node", ""))
    nodes = {}
    for n in alloc:
        name = n.get("name") or n.get("nodename")
        cpus = n.get("cpus", {}).get("count", 0) if isinstance(n.get("cpus"), dict) else int(n.get("cpus_used", 0) or 0)
        mem = n.get("memory", {}).get("allocated", 0) if isinstance(n.get("memory"), dict) else int(n.get("memory_allocated", 0) or 0)
        nodes[name] = SlurmNode(name, int(cpus), int(mem), _gpu_count(gres))
    if not nodes:
        nodes = {n: SlurmNode(n) for n in expand_hostlist(str(job.get("nodes", "")))}
    return SlurmJob(job_id, user_id, nodes)


def clamp_inventory(inventory: dict, job: SlurmJob | None, node_name: str | None = None) -> dict:
    """What this node offers a run inside ``job``: never more than the job was given."""
    if job is None:
        return inventory
    node = job.nodes.get(node_name or "") or next(iter(job.nodes.values()))
    out = dict(inventory, slurm_job=str(job.job_id), slurm_nodes=sorted(job.nodes))
    if node.gpus:
        out["gpus"] = min(inventory.get("gpus", 0), node.gpus)
        out["gpu_names"] = list(inventory.get("gpu_names", []))[:out["gpus"]]
    if node.cpus:
        out["cpus"] = min(inventory.get("cpus", node.cpus), node.cpus)
    if node.memory_mib:
        gib = node.memory_mib / 1024.0
        out["host_total_gib"] = min(inventory.get("host_total_gib", gib), gib)
        out["host_free_gib"] = min(inventory.get("host_free_gib", gib), gib)
    return out
