"""Preparation as four fresh processes: build, profile, communicate, plan.

    python -m shadowspill_b200.training.phases prepare --setup setup.json --directory prep/
    python -m shadowspill_b200.training.phases <build|profile|communicate|plan> --setup ... --directory ...

Each phase is its own Python process, so nothing one phase leaves behind (a CUDA context with the
profiler's allocations, cached kernels' workspaces, pinned calibration buffers) is alive in the next
one or in the worker that will execute the plan:

  build        the candidate programs (walk orders x save/recompute resolutions) and the programs
               of the further operations; records their digests, so that later phases prove they
               rebuilt the same programs                                   -> build.json
  profile      every distinct task timed in isolation, with its workspace and (under the
               allocation adapter) its allocation contract                 -> profiles.json
  communicate  host-link lanes (all ranks streaming at once when the job has several), and the
               burst-to-sustained scale of task times                      -> communication.json
  plan         no GPU: profiles applied, every candidate planned, the fastest kept; the plans of
               the further operations share its state layout (the plan family) -> training.ssp

``prepare_job`` runs the four in order and returns the bundle; a ``TrainingSetup`` with that
``bundle`` then opens its executor directly. A phase that fails stops the job with that phase's
output; phases whose result file exists are skipped unless ``force`` is set, so a job resumes
where it stopped.

Reference: packages/engine/src/shadowspill/training/preparation/phases/operations.py:39,91,127,197
(``build`` / ``profile`` / ``communicate`` / ``plan``), phases/job.py:86 (``prepare_job``).
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import time
from dataclasses import asdict, fields
from pathlib import Path

PHASES = ("build", "profile", "communicate", "plan")
RESULT = {"build": "build.json", "profile": "profiles.json", "communicate": "communication.json",
          "plan": "training.ssp"}


def setup_to_json(setup) -> dict:
    if hasattr(setup.optimizer_rule, "apply"):
        raise ValueError("a captured optimizer is a graph in this process; separate preparation processes "
                         "take the named rules (adamw, sgd, lion)")
    d = asdict(setup)
    d["model"] = setup.model if isinstance(setup.model, str) else setup.model.to_json()
    return d


def setup_from_json(d: dict):
    from ..models.config import DecoderConfig
    from ..planning.plan import SearchOptions
    from .session import TrainingSetup
    d = dict(d)
    if isinstance(d.get("model"), dict):
        d["model"] = DecoderConfig.from_json(d["model"])
    if isinstance(d.get("search"), dict):
        s = dict(d["search"])
        for k in ("strategies", "fetch_rules"):
            if k in s:
                s[k] = tuple(s[k])
        d["search"] = SearchOptions(**s)
    known = {f.name for f in fields(TrainingSetup)}
    for k, v in list(d.items()):
        if k not in known:
            del d[k]
        elif isinstance(v, list):
            d[k] = tuple(v)
    return TrainingSetup(**d)


def run_phase(phase: str, setup, directory: str | Path, log=None) -> dict:
    """Runs one phase in THIS process (the command line gives each its own)."""
    from dataclasses import replace
    from .session import TrainingSession
    directory = Path(directory)
    t0 = time.perf_counter()
    kw = dict(stop_after=phase, phase_directory=str(directory))
    if phase == "plan":
        kw["bundle"] = str(directory / RESULT["plan"])
        kw["allocator"] = "caching"       # planning never touches a GPU: nothing to install
    if phase in ("build", "profile"):
        kw["calibrate"] = False
    session = TrainingSession(replace(setup, **kw), log=log)
    session.close()
    return {"phase": phase, "seconds": time.perf_counter() - t0, "result": str(directory / RESULT[phase])}


def prepare_job(setup, directory: str | Path, force: bool = False, timeout: float = 3600.0, log=None) -> Path:
    """The four phases as four fresh processes; returns the path of the prepared bundle."""
    directory = Path(directory)
    directory.mkdir(parents=True, exist_ok=True)
    (directory / "setup.json").write_text(json.dumps(setup_to_json(setup), default=str))
    record = []
    for phase in PHASES:
        target = directory / RESULT[phase]
        if target.exists() and not force:
            record.append({"phase": phase, "skipped": True})
            continue
        cmd = [sys.executable, "-m", "shadowspill_b200.training.phases", phase, "--setup",
               str(directory / "setup.json"), "--directory", str(directory)]
        if phase == "communicate" and setup.world_size > 1 and setup.device == "cuda":
            # every rank streams at once: the ranks share the host's memory system
            cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1",
                   f"--nproc-per-node={setup.world_size}", "--master-addr", "127.0.0.1",
                   "--master-port", str(29500 + os.getpid() % 2000), "-m", "shadowspill_b200.training.phases",
                   phase, "--setup", str(directory / "setup.json"), "--directory", str(directory)]
        t0 = time.perf_counter()
        proc = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout)
        (directory / f"{phase}.log").write_text(proc.stdout + proc.stderr)
        if proc.returncode != 0 or not target.exists():
            tail = "\n".join((proc.stderr or proc.stdout).splitlines()[-12:])
            raise RuntimeError(f"preparation phase {phase!r} failed (exit {proc.returncode}):\n{tail}")
        record.append({"phase": phase, "seconds": round(time.perf_counter() - t0, 3), "pid_was_fresh": True})
        if log:
            log(f"phase {phase}: {record[-1]['seconds']:.1f} s")
    (directory / "job.json").write_text(json.dumps({"phases": record}))
    return directory / RESULT["plan"]


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("phase", choices=PHASES + ("prepare",))
    ap.add_argument("--setup", required=True, help="JSON of the TrainingSetup fields")
    ap.add_argument("--directory", required=True)
    ap.add_argument("--force", action="store_true")
    a = ap.parse_args(argv)
    fields_json = json.load(open(a.setup))
    rank = int(os.environ.get("RANK", 0))
    if a.phase == "communicate" and int(os.environ.get("WORLD_SIZE", 1)) > 1:
        import torch
        import torch.distributed as dist
        local = int(os.environ.get("LOCAL_RANK", rank))
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        fields_json.update(rank=rank, device_index=local, world_size=int(os.environ["WORLD_SIZE"]))
    elif a.phase != "prepare":
        fields_json.update(rank=0)
    setup = setup_from_json(fields_json)
    log = (lambda m: print(f"[{a.phase}] {m}", file=sys.stderr, flush=True)) if rank == 0 else None
    if a.phase == "prepare":
        print(prepare_job(setup, a.directory, force=a.force, log=log))
        return 0
    rec = run_phase(a.phase, setup, a.directory, log)
    if rank == 0:
        print(json.dumps(rec))
    return 0


if __name__ == "__main__":
    sys.exit(main())
