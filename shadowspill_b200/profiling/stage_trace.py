"""Run one task of a training program in isolation, for a profiler to look at.

    python -m shadowspill_b200.profiling.stage_trace --model llama3-8b --task B.layer1.0 \\
        --selection 1:save_attention --microbatch 2048 --repeats 3

The program is built as a session would build it, the named task gets freshly allocated operands
with valid synthetic contents (the same ones task profiling uses), runs ``--warmup`` times, and then
``--repeats`` times between ``cudaProfilerStart`` / ``cudaProfilerStop`` with one NVTX range per
repeat (``stage_trace/<task>/<i>``), so that a capture started with the profiler-range trigger of
Nsight Systems or with ``ncu --nvtx --nvtx-include`` holds exactly these launches and nothing of
the set-up. Keep the microbatch small when every launch is replayed: the point of a single task is
that the capture ends by itself. Without a profiler the tool prints what it measured: the task's
time by CUDA events, its workspace, and the number of kernel-library launches by entry point.

Reference: tools/stage_traces (a compiled stage run under Nsight with a profiler-range window).
"""
from __future__ import annotations

import argparse
import json
import sys

import torch

from ..data.synthetic import make_batch
from ..execution.executor import Hyperparameters, TaskRunner
from ..frontend.capture import BatchGeometry, StepDataOrdering, build_step
from ..models.config import preset
from .measure import _fill_inputs


def parse_selection(text: str) -> dict[int, str]:
    """``"1:save,2:save_attention"`` -> {1: "save", 2: "save_attention"} (stage index: variant)."""
    out = {}
    for part in filter(None, text.split(",")):
        stage, variant = part.split(":")
        out[int(stage)] = variant
    return out


def trace_task(model: str, task: str, microbatch_tokens: int = 2048, microbatches: int = 2,
               selection: dict[int, str] | None = None, frontend: str = "stages", device: str = "cuda",
               warmup: int = 2, repeats: int = 3, dtype=torch.bfloat16) -> dict:
    cfg = preset(model) if isinstance(model, str) else model
    geo = BatchGeometry(microbatch_tokens=microbatch_tokens, n_microbatches=microbatches,
                        slots=microbatch_tokens // 32 + 1, mean_seqlen=min(1200, microbatch_tokens // 2))
    program, desc = build_step(cfg, geo, StepDataOrdering(), dtype=dtype, selection=selection or {},
                               frontend=frontend)
    names = [t.name for t in program.tasks]
    if task not in names:
        close = [n for n in names if n.split(".")[0] == task.split(".")[0]][:12]
        raise KeyError(f"no task {task!r} in the program; tasks of that kind: {close}")
    ti = names.index(task)
    dev = torch.device(device)
    cuda = dev.type == "cuda"
    runner = TaskRunner(program, desc, Hyperparameters(lr=0.0), seed=0, stochastic_rounding=True)
    host = make_batch(0, vocab=cfg.vocab_size, tokens_per_step=runner.T * runner.n_mb, microbatch_tokens=runner.T,
                      slots=runner.slots, max_len=min(8192, runner.T), median=min(1200.0, runner.T / 4),
                      min_len=min(32, runner.T // 4))
    flats = [torch.empty(program.objects[u.object].bytes, dtype=torch.uint8, device=dev) for u in runner.uses[ti]]
    _fill_inputs(runner, ti, flats, host)
    bound = runner.bind(ti, flats)
    launches_before = _launch_counts()
    for _ in range(warmup):
        runner.grad_seen = set()
        runner.run_task(ti, bound)
    workspace = 0
    if cuda:
        torch.cuda.synchronize(dev)
        torch.cuda.reset_peak_memory_stats(dev)
        base = torch.cuda.memory_allocated(dev)
        torch.cuda.cudart().cudaProfilerStart()
    times = []
    for i in range(repeats):
        runner.grad_seen = set()
        if cuda:
            torch.cuda.nvtx.range_push(f"stage_trace/{task}/{i}")
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            runner.run_task(ti, bound)
            b.record()
            torch.cuda.synchronize(dev)
            torch.cuda.nvtx.range_pop()
            times.append(a.elapsed_time(b) * 1e-3)
        else:
            import time
            t0 = time.perf_counter()
            runner.run_task(ti, bound)
            times.append(time.perf_counter() - t0)
    if cuda:
        torch.cuda.cudart().cudaProfilerStop()
        workspace = torch.cuda.max_memory_allocated(dev) - base
    after = _launch_counts()
    per_run = {k: (after[k] - launches_before.get(k, 0)) // max(1, warmup + repeats)
               for k in after if after[k] != launches_before.get(k, 0)}
    t = program.tasks[ti]
    return {"task": task, "kind": t.kind, "variant": t.variant, "profile_key": t.profile_key,
            "microbatch_tokens": microbatch_tokens, "seconds": times, "workspace_bytes": int(workspace),
            "operand_bytes": sum(f.numel() for f in flats), "library_launches_per_run": per_run}


def _launch_counts() -> dict[str, int]:
    try:
        from ..ops import _lib
        return dict(_lib.launch_counts())
    except (ImportError, AttributeError, OSError):
        return {}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", default="llama3-8b")
    ap.add_argument("--task", required=True, help="task name as the program lists it, e.g. F.layer1.0, B.layer1.0, H.head.0")
    ap.add_argument("--microbatch", type=int, default=2048)
    ap.add_argument("--selection", default="", help="stage:variant pairs, e.g. 1:save_attention")
    ap.add_argument("--frontend", default="stages", choices=["stages", "graph"])
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--warmup", type=int, default=2)
    ap.add_argument("--repeats", type=int, default=3)
    a = ap.parse_args(argv)
    rec = trace_task(a.model, a.task, a.microbatch, selection=parse_selection(a.selection), frontend=a.frontend,
                     device=a.device, warmup=a.warmup, repeats=a.repeats,
                     dtype=torch.bfloat16 if a.device != "cpu" else torch.float32)
    print(json.dumps(rec))
    return 0


if __name__ == "__main__":
    sys.exit(main())
