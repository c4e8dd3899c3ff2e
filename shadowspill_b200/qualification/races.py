"""Race detection for the native core: the runtime's threads under ThreadSanitizer.

    python -m shadowspill_b200.qualification.races [--keep DIR]

The C++ core is rebuilt with ``-fsanitize=thread`` into a scratch directory and a workload
that exercises every thread the runtime owns is run against it in a child process: planned
training steps on the mock backend (dispatcher + worker thread + two stream threads), the
same through the file pool and the remote pool (plus disk threads and staged lanes), lane calibration from the
calling thread, and a step that ends in an injected copy failure (latch + drain). The child
runs with ``libtsan`` preloaded because the interpreter itself is not instrumented.

Only reports whose racing access is inside ``libss_core`` count. PyTorch's OpenMP workers
are not instrumented, so ThreadSanitizer cannot see their barriers and reports their
hand-offs as races; those reports never have a core frame on top and are dropped.

The reference keeps helgrind suppressions and runs its C core under the race detectors in
CI (tools/helgrind suppressions; packages/engine/csrc tests); this is the same check for
this tree's runtime.
"""
from __future__ import annotations

import argparse
import glob
import os
import re
import subprocess
import sys
import tempfile
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]

WORKLOAD = r"""
import copy, sys, tempfile, torch
from shadowspill_b200.communication.info import CommunicationInfo
from shadowspill_b200.data.synthetic import make_batch
from shadowspill_b200.execution.executor import Executor
from shadowspill_b200.frontend.capture import BatchGeometry, StepDataOrdering, build_step
from shadowspill_b200.models.config import preset
from shadowspill_b200.planning.plan import (MemoryBudgets, PlanningError, SearchOptions,
                                            move_homes_to_file, plan_program)
from shadowspill_b200.runtime.core import Runtime, RuntimeFailure

torch.set_num_threads(1)          # keep uninstrumented OpenMP workers out of the picture
cfg = preset("llama3-tiny")
geo = BatchGeometry(microbatch_tokens=256, n_microbatches=2, slots=16, mean_seqlen=64)
prog, desc = build_step(cfg, geo, StepDataOrdering(), dtype=torch.float32)
total = sum(o.bytes for o in prog.objects)
ws = max(t.workspace_bytes for t in prog.tasks)
plan = None
for pct in range(30, 101, 5):
    try:
        plan = plan_program(prog, MemoryBudgets(ws + total * pct // 100, 64 << 20, headroom_bytes=0),
                            CommunicationInfo(), SearchOptions(minimum_object_bytes_evict_eligible=1024, workers=2))
        break
    except PlanningError:
        pass
batch = lambda s: make_batch(s, vocab=cfg.vocab_size, tokens_per_step=512, microbatch_tokens=256,
                             median=60, min_len=8, max_len=128, slots=16)
ex = Executor(copy.deepcopy(plan), desc, device="cpu", seed=1, trace_capacity=4096)
ex.initialize()
want = [ex.run(batch(s), trace=(s == 1)).loss for s in range(2)]
ex.rt.mock_fail("copy", 5)
try:
    ex.run(batch(2))
    raise SystemExit("the injected failure did not surface")
except RuntimeFailure:
    pass
ex.closed = True
ex.rt.close()
with tempfile.TemporaryDirectory() as d:
    ex = Executor(move_homes_to_file(copy.deepcopy(plan)), desc, device="cpu", seed=1,
                  file_pool={"directory": d, "chunk_bytes": 16 << 10, "queue_depth": 3})
    ex.initialize()
    got = [ex.run(batch(s)).loss for s in range(2)]
    ex.close()
    assert got == want, (got, want)
    rt = Runtime(8 << 20, 4096, backend="mock", file_bytes=8 << 20, file_directory=d,
                 file_chunk_bytes=64 << 10, file_queue_depth=3)
    rt.calibrate_file(1 << 20, repeats=1)
    rt.close()
# the remote pool: chunks over sockets borrowed by several disk threads at once
import subprocess
from shadowspill_b200 import build
build.build_core()
daemon = subprocess.Popen([str(build.MEMORY_DAEMON), "--port", "0"], stdout=subprocess.PIPE, text=True)
try:
    address = "127.0.0.1:" + daemon.stdout.readline().split()[1]
    ex = Executor(move_homes_to_file(copy.deepcopy(plan)), desc, device="cpu", seed=1,
                  file_pool={"remote": address, "chunk_bytes": 16 << 10, "queue_depth": 3})
    ex.initialize()
    got = [ex.run(batch(s)).loss for s in range(2)]
    ex.close()
    assert got == want, (got, want)
finally:
    daemon.kill()
    daemon.wait()
print("workload ok")
"""


def build_instrumented(directory: Path) -> Path:
    src = sorted(p for p in (ROOT / "csrc" / "src").glob("*.cpp") if "backend_cuda" not in p.name)
    out = directory / "libss_core.so"
    cmd = ["g++", "-O1", "-g", "-std=c++17", "-fPIC", "-fsanitize=thread", "-pthread", "-shared",
           "-I", str(ROOT / "csrc" / "include"), "-o", str(out), *map(str, src), "-ldl"]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"instrumented build failed:\n{proc.stderr}")
    return out


def tsan_runtime() -> str | None:
    path = subprocess.run(["g++", "-print-file-name=libtsan.so"], capture_output=True, text=True).stdout.strip()
    return path if path and os.path.isabs(path) and os.path.exists(path) else None


def core_reports(log_text: str) -> list[str]:
    """The reports whose racing access (the top frame of an access stack) is in the core."""
    out = []
    for rep in log_text.split("WARNING: ThreadSanitizer:")[1:]:
        tops = []
        for section in re.split(r"\n\s*\n", rep):
            if re.search(r"(Write|Read|Previous \w+|Atomic \w+) of size", section):
                m = re.search(r"#0 (.*)", section)
                tops.append(m.group(1) if m else "")
        if any("libss_core" in t for t in tops) or "lock-order-inversion" in rep.split("\n", 1)[0]:
            out.append("WARNING: ThreadSanitizer:" + rep)
    return out


def run(keep: str | None = None, timeout: float = 1500.0) -> dict:
    runtime = tsan_runtime()
    if runtime is None:
        return {"available": False, "reason": "libtsan.so not found next to g++"}
    ctx = tempfile.TemporaryDirectory() if keep is None else None
    directory = Path(keep) if keep else Path(ctx.name)
    directory.mkdir(parents=True, exist_ok=True)
    try:
        lib = build_instrumented(directory)
        env = dict(os.environ, LD_PRELOAD=runtime, SS_CORE_LIB=str(lib), OMP_NUM_THREADS="1",
                   PYTHONPATH=str(ROOT.parent) + os.pathsep + os.environ.get("PYTHONPATH", ""),
                   TSAN_OPTIONS=f"exitcode=0 halt_on_error=0 report_signal_unsafe=0 log_path={directory / 'tsan'}")
        proc = subprocess.run([sys.executable, "-c", WORKLOAD], env=env, capture_output=True, text=True,
                              timeout=timeout, cwd=str(ROOT.parent))
        logs = "".join(open(f).read() for f in sorted(glob.glob(str(directory / "tsan.*"))))
        reports = core_reports(logs)
        return {"available": True, "workload_ok": proc.returncode == 0 and "workload ok" in proc.stdout,
                "stderr_tail": proc.stderr[-2000:], "all_reports": logs.count("WARNING: ThreadSanitizer:"),
                "core_reports": reports}
    finally:
        if ctx is not None:
            ctx.cleanup()


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--keep", default=None, help="directory for the instrumented library and the logs")
    a = ap.parse_args(argv)
    res = run(a.keep)
    if not res["available"]:
        print(f"race detection unavailable: {res['reason']}")
        return 0
    print(f"workload {'ok' if res['workload_ok'] else 'FAILED'}; {res['all_reports']} reports in all, "
          f"{len(res['core_reports'])} with a racing access inside the core")
    for rep in res["core_reports"]:
        print(rep[:3000])
    if not res["workload_ok"]:
        print(res["stderr_tail"])
    return 0 if res["workload_ok"] and not res["core_reports"] else 1


if __name__ == "__main__":
    raise SystemExit(main())
