"""Nsight Systems capture of worker processes.

``Execution(nsys={"start_step": 3, "steps": 2, "gpu_metrics": False})`` asks for a capture
of a few steps of every worker. Where the ``nsys`` executable exists on the worker's node,
the worker command is wrapped so that recording is controlled by the CUDA profiler range:
the worker calls ``cudaProfilerStart`` before step ``start_step`` and ``cudaProfilerStop``
after ``steps`` steps (``StepWindow``), and one report per rank lands in the run's
directory. Where it does not exist the request is recorded as unavailable and the run goes
on unprofiled. Ranks enter and leave the window together: a barrier on both sides keeps a
collective from straddling the boundary.

Reference: packages/engine/src/shadowspill/orchestration/capture/{nsys.py:13,
nsys_worker.py, _nsys_runtime.py:18-21}.
"""
from __future__ import annotations

import shutil
from dataclasses import dataclass
from pathlib import Path


@dataclass(frozen=True)
class NsysOptions:
    start_step: int = 3          # first captured step (1-based count of executed steps)
    steps: int = 2
    gpu_metrics: bool = False    # sample GPU hardware counters as well (needs privileges)
    cuda_memory: bool = False
    executable: str = "nsys"

    @staticmethod
    def from_json(d: dict | None) -> "NsysOptions | None":
        if not d:
            return None
        known = {k: d[k] for k in ("start_step", "steps", "gpu_metrics", "cuda_memory", "executable") if k in d}
        o = NsysOptions(**known)
        if o.start_step < 1 or o.steps < 1:
            raise ValueError("nsys: start_step and steps are positive")
        return o


def available(options: NsysOptions | None = None) -> str | None:
    """Path of the ``nsys`` executable, or ``None``."""
    return shutil.which((options or NsysOptions()).executable)


def report_path(directory: str | Path, rank: int) -> Path:
    return Path(directory) / f"worker{rank}.nsys-rep"


def wrap_command(command: list[str], rank: int, directory: str | Path, options: NsysOptions) -> list[str]:
    """``command`` run under ``nsys profile``, recording only between the profiler range calls."""
    exe = available(options)
    if exe is None:
        raise FileNotFoundError(f"{options.executable} is not installed on this node")
    out = report_path(directory, rank)
    args = [exe, "profile", "--capture-range=cudaProfilerApi", "--capture-range-end=stop",
            "--trace=cuda,nvtx,osrt", "--sample=none", "--cpuctxsw=none", "--force-overwrite=true",
            f"--output={out.with_suffix('')}"]
    if options.gpu_metrics:
        args.append("--gpu-metrics-devices=cuda-visible")
    if options.cuda_memory:
        args.append("--cuda-memory-usage=true")
    return args + list(command)


class StepWindow:
    """Opens the profiler range before step ``start_step`` and closes it ``steps`` steps later.
    ``start`` / ``stop`` default to ``torch.cuda.profiler``; ``barrier`` to a no-op."""

    def __init__(self, options: NsysOptions, start=None, stop=None, barrier=None):
        self.options = options
        self.executed = 0
        self.state = "waiting"           # waiting -> recording -> done
        self._start, self._stop = start, stop
        self._barrier = barrier or (lambda: None)

    def before_step(self) -> None:
        if self.state == "waiting" and self.executed + 1 == self.options.start_step:
            self._barrier()
            (self._start or _cuda_profiler("start"))()
            self.state = "recording"

    def after_step(self) -> None:
        self.executed += 1
        if self.state == "recording" and self.executed >= self.options.start_step + self.options.steps - 1:
            self._barrier()
            (self._stop or _cuda_profiler("stop"))()
            self.state = "done"


def _cuda_profiler(which: str):
    import torch

    def call():
        if torch.cuda.is_available():
            torch.cuda.synchronize()
            getattr(torch.cuda.profiler, which)()
    return call


def status(directory: str | Path, rank: int, requested: NsysOptions | None) -> dict:
    """What ``GET .../nsys?rank=`` reports."""
    if requested is None:
        return {"requested": False, "available": available() is not None}
    exe = available(requested)
    if exe is None:
        return {"requested": True, "available": False,
                "reason": f"{requested.executable} is not installed on this node"}
    rep = report_path(directory, rank)
    return {"requested": True, "available": True, "executable": exe, "report": str(rep),
            "complete": rep.exists(), "bytes": rep.stat().st_size if rep.exists() else 0}
