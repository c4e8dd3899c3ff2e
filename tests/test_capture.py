"""Nsight capture plumbing, with a stand-in ``nsys`` executable (none is installed here)."""
import os
import stat
import sys

import numpy as np
import pytest

from shadowspill_b200.orchestration import capture


def _fake_nsys(directory):
    """A script that behaves like ``nsys profile <options> <command>``: writes the report file
    named by --output and runs the command."""
    path = directory / "nsys"
    path.write_text("#!/bin/sh\nshift\nout=\nwhile [ $# -gt 0 ]; do case \"$1\" in\n"
                    "  --output=*) out=\"${1#--output=}\"; shift;;\n  --*) shift;;\n  *) break;;\nesac; done\n"
                    "echo report > \"$out.nsys-rep\"\nexec \"$@\"\n")
    path.chmod(path.stat().st_mode | stat.S_IEXEC)
    return path


def test_step_window_opens_and_closes_once_with_barriers():
    calls = []
    w = capture.StepWindow(capture.NsysOptions(start_step=3, steps=2), start=lambda: calls.append("start"),
                           stop=lambda: calls.append("stop"), barrier=lambda: calls.append("barrier"))
    for step in range(1, 8):
        w.before_step()
        calls.append(f"step{step}")
        w.after_step()
    assert calls == ["step1", "step2", "barrier", "start", "step3", "step4", "barrier", "stop",
                     "step5", "step6", "step7"]
    assert w.state == "done"
    with pytest.raises(ValueError):
        capture.NsysOptions.from_json({"start_step": 0})


def test_wrap_command_and_status(tmp_path, monkeypatch):
    opts = capture.NsysOptions(start_step=2, steps=1, gpu_metrics=True)
    monkeypatch.setenv("PATH", str(tmp_path / "empty"))
    assert capture.available(opts) is None
    assert capture.status(tmp_path, 0, opts) == {"requested": True, "available": False,
                                                 "reason": "nsys is not installed on this node"}
    with pytest.raises(FileNotFoundError):
        capture.wrap_command(["python", "x.py"], 0, tmp_path, opts)
    fake = _fake_nsys(tmp_path)
    monkeypatch.setenv("PATH", f"{tmp_path}{os.pathsep}/usr/bin{os.pathsep}/bin")
    cmd = capture.wrap_command(["python", "x.py"], 1, tmp_path, opts)
    assert cmd[0] == str(fake) and cmd[1] == "profile" and cmd[-2:] == ["python", "x.py"]
    assert "--capture-range=cudaProfilerApi" in cmd and "--gpu-metrics-devices=cuda-visible" in cmd
    assert f"--output={tmp_path / 'worker1'}" in cmd
    assert capture.status(tmp_path, 1, opts)["complete"] is False
    assert capture.status(tmp_path, 1, None) == {"requested": False, "available": True}


def test_workers_run_under_the_wrapper_and_the_service_reports_it(tmp_path, monkeypatch):
    from shadowspill_b200.client import (BatchConfig, Memory, Model, Optimizer, Preparation,
                                         ProfilingOptions, Resources, ServiceClient, text_batch)
    from shadowspill_b200.client.config import Execution, PlanningOptions
    from shadowspill_b200.server.service import Server
    bin_dir = tmp_path / "bin"
    bin_dir.mkdir()
    _fake_nsys(bin_dir)
    monkeypatch.setenv("PATH", f"{bin_dir}{os.pathsep}{os.path.dirname(sys.executable)}{os.pathsep}/usr/bin{os.pathsep}/bin")
    rng = np.random.default_rng(0)
    seqs = [rng.integers(0, 512, size=40) for _ in range(8)]
    with Server(tmp_path / "svc", token="t") as srv, ServiceClient(srv.url, token="t") as svc:
        trainer = svc.create_training_client(
            Model("llama3-tiny", dtype="float32"), Optimizer(lr=3e-3, parameter_rounding="nearest"),
            batch=BatchConfig(tokens_per_step=512, microbatch_tokens=256),
            memory=Memory(device_gib=0.53, spill_gib=0.25), resources=Resources(gpus=1, backend="cpu"),
            execution=Execution(nsys={"start_step": 1, "steps": 1}, runtime_trace=True),
            preparation=Preparation(profiling=ProfilingOptions(enabled=False), calibrate=False,
                                    planning=PlanningOptions(minimum_object_bytes_evict_eligible=1024, workers=1)),
            timeout=300).result()
        assert trainer.step(text_batch(seqs)).result().loss > 0
        info = svc.get_nsys(trainer.run).result() if hasattr(trainer, "run") else None
        # a traced step: the runtime report of the worker comes back with the result
        res, where = trainer.traced_step(text_batch(seqs), tmp_path / "trace_dl").result()
        assert res.loss > 0 and (where / "rank0" / "runtime.html").exists()
        assert (where / "rank0" / "runtime.json").exists()
        trainer.close()
    reports = list((tmp_path / "svc").rglob("worker0.nsys-rep"))
    assert len(reports) == 1
    if info is not None:
        assert info["requested"] and info["available"] and info["report"].endswith("worker0.nsys-rep")


def test_stage_trace_runs_one_task_in_isolation():
    """The single-task tool builds the program, binds the named task to synthetic operands and
    times it; an unknown task name lists the tasks of that kind."""
    import pytest
    from shadowspill_b200.profiling.stage_trace import parse_selection, trace_task
    import torch
    assert parse_selection("1:save,2:save_attention") == {1: "save", 2: "save_attention"}
    rec = trace_task("llama3-tiny", "B.layer0.1", microbatch_tokens=256, selection={1: "save_attention"},
                     device="cpu", warmup=1, repeats=2, dtype=torch.float32)
    assert rec["variant"] == "save_attention" and len(rec["seconds"]) == 2 and rec["operand_bytes"] > 0
    graph = trace_task("llama3-tiny", "F.layer1.0", microbatch_tokens=256, frontend="graph", device="cpu",
                       warmup=1, repeats=1, dtype=torch.float32)
    assert graph["kind"] == "forward"
    with pytest.raises(KeyError, match="B.layer0.0"):
        trace_task("llama3-tiny", "B.layer9.0", microbatch_tokens=256, device="cpu", dtype=torch.float32)


def test_gap_report_separates_lanes_waits_and_interference(tmp_path):
    """Two lanes built by hand: a backward task that starts exactly when a reduce-scatter ends
    waited for it; compute tasks that ran beside a collective are slower than those that ran alone."""
    from shadowspill_b200.qualification.gap_report import Row, build, from_directory
    rows = [Row(0, "F.layer0.0", "forward", 0.010, 0.010, 0.000, 0.010),
            Row(1, "B.layer1.0", "backward", 0.010, 0.010, 0.010, 0.010),            # alone, on profile
            Row(2, "RS.layer1.g0", "collective", 0.001, 0.001, 0.020, 0.006),
            Row(3, "B.layer0.1", "backward", 0.010, 0.010, 0.026, 0.010),            # waited for the RS
            Row(4, "AG.layer0.fwd.g1", "collective", 0.001, 0.001, 0.036, 0.008),
            Row(5, "F.layer0.1", "forward", 0.010, 0.010, 0.036, 0.014),             # beside the AG: slower
            Row(6, "O.layer0", "optimizer", 0.001, 0.001, 0.050, 0.002)]
    rep = build(rows, simulated_s=0.045)
    assert rep.lanes["compute"]["tasks"] == 4 and rep.lanes["communication"]["tasks"] == 3
    assert abs(rep.lanes["compute"]["gap_s"] - 0.006) < 1e-9
    (why, gap), = rep.waits.items()
    assert "RS task" in why and gap["count"] == 1 and abs(gap["seconds"] - 0.006) < 1e-9
    assert rep.interference["beside"]["tasks"] == 1 and abs(rep.interference["beside"]["ratio"] - 1.4) < 1e-9
    assert rep.interference["alone"]["tasks"] == 3 and abs(rep.interference["alone"]["ratio"] - 1.0) < 1e-9
    assert abs(rep.makespan_s - 0.052) < 1e-9 and "measured 52.0 ms, simulated 45.0 ms" in rep.text()
    # the communication lane cost the compute lane the 6 ms gap and the 4 ms by which the task beside the
    # gather ran over its profile: 10 ms over 3 tasks, planned with 1 ms each
    assert abs(rep.exposure["seconds"] - 0.010) < 1e-9 and rep.exposure["tasks"] == 3
    assert abs(rep.exposure["suggested_overhead_us"] - (0.010 - 0.003) / 3 * 1e6) < 1e-3
    assert "collective_overhead_us = 2333" in rep.text()
    # without collectives the update belongs to the compute lane
    solo = build([Row(0, "B.layer0.0", "backward", 0.01, 0.01, 0.0, 0.01), Row(1, "O.layer0", "optimizer", 0.001, 0.001, 0.012, 0.001)])
    assert "communication" not in solo.lanes and solo.waits["host (frontend late)"]["count"] == 1
    # the files a traced step writes
    import csv
    with open(tmp_path / "runtime_tasks.csv", "w", newline="") as f:
        w = csv.writer(f)
        w.writerow(["index", "name", "kind", "stage", "microbatch", "profiled_s", "simulated_start_s", "simulated_s",
                    "real_start_s", "real_s", "gap_before_s", "simulated_gap_s", "waited_inputs", "waited_reuse"])
        for r in rows:
            w.writerow([r.index, r.name, r.kind, 0, 0, r.profiled_s, 0, r.simulated_s, r.start_s, r.real_s, 0, 0, 0, 0])
    assert from_directory(tmp_path).waits == rep.waits


def test_collective_overhead_is_added_to_communication_stream_tasks_only():
    import torch
    from shadowspill_b200.frontend.capture import (BatchGeometry, StepDataOrdering, add_collective_overhead,
                                                   build_step)
    from shadowspill_b200.models.config import preset
    geo = BatchGeometry(256, 4, 16, 64)
    prog, _ = build_step(preset("llama3-tiny"), geo, StepDataOrdering(microbatch_groups=2), dtype=torch.float32,
                         world_size=2, rank=0)
    before = {t.name: t.duration_ns for t in prog.tasks}
    side = [t for t in prog.tasks if t.kind == "collective" or t.variant == "adamw_dp"]
    assert {t.name.split(".")[0] for t in side} == {"AG", "RS", "O"}
    assert add_collective_overhead(prog, 250.0) == len(side)
    for t in prog.tasks:
        assert t.duration_ns - before[t.name] == (250_000 if t in side else 0)
    assert add_collective_overhead(prog, 0.0) == 0
    solo, _ = build_step(preset("llama3-tiny"), geo, StepDataOrdering(), dtype=torch.float32)
    assert add_collective_overhead(solo, 250.0) == 0              # one worker: nothing runs on that stream


def test_worker_logs_are_bounded(tmp_path):
    """A worker's output is copied into its log up to the limit, a note marks the cut, and the pipe
    keeps being drained so that the writer never blocks."""
    import subprocess
    import sys
    from shadowspill_b200.training.group import BoundedLog
    chatty = ("import sys\n"
              "for i in range(20000):\n"
              "    sys.stdout.write('line %06d of worker output\\n' % i)\n"
              "sys.stdout.flush()\n"
              "print('done')\n")
    proc = subprocess.Popen([sys.executable, "-c", chatty], stdout=subprocess.PIPE, stderr=subprocess.STDOUT)
    log = BoundedLog(proc.stdout, tmp_path / "worker0.log", 4096)
    log.start()
    assert proc.wait(timeout=60) == 0                     # 540 kB of output never blocked on the pipe
    log.join(timeout=30)
    text = (tmp_path / "worker0.log").read_bytes()
    assert text.startswith(b"line 000000") and b"log limit of 4096 bytes reached" in text
    assert len(text) < 4096 + 200 and log.dropped > 500_000
    quiet = subprocess.Popen([sys.executable, "-c", "print('short')"], stdout=subprocess.PIPE, stderr=subprocess.STDOUT)
    small = BoundedLog(quiet.stdout, tmp_path / "worker1.log", 4096)
    small.start(); quiet.wait(timeout=60); small.join(timeout=30)
    assert (tmp_path / "worker1.log").read_text() == "short\n" and small.dropped == 0
