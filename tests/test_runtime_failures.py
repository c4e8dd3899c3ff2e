"""Failure detection without touching a GPU: the mock backend fails the n-th
operation, host-side waits run out, and the first failure is latched."""
import sys

import pytest
import torch

sys.path.insert(0, __file__.rsplit("/", 1)[0])
from test_executor_cpu import _batches, _setup  # noqa: E402

from shadowspill_b200 import native
from shadowspill_b200.execution.executor import Executor
from shadowspill_b200.orchestration.nodes import AdmissionError, Membership, NodeAdmission
from shadowspill_b200.runtime.core import Runtime, RuntimeFailure
from shadowspill_b200.server.journal import Journal, JournalCorrupt
from shadowspill_b200.training.controller import OperationState, Rejected, RunController


def test_failed_copy_latches_and_refuses_further_work():
    cfg, plan, desc = _setup()
    ex = Executor(plan, desc, device="cpu", seed=1)
    ex.initialize()
    ex.run(_batches(cfg))                                   # a clean step first
    ex.rt.mock_fail("copy", 5)                              # the 5th copy from now fails
    with pytest.raises(RuntimeFailure) as e:
        ex.run(_batches(cfg, 1))
    info = e.value.info
    assert info["status"] == native.BACKEND_FAILURE and info["action"] >= 0 and info["object"] >= 0
    assert "failed to enqueue" in info["message"]
    # first writer wins: a later failure does not overwrite the record
    ex.rt.latch_failure("second failure")
    assert ex.rt.failure()["message"] == info["message"]
    with pytest.raises(RuntimeFailure):
        ex.run(_batches(cfg, 2))                            # latched: nothing starts
    ex.closed = True
    ex.rt.close()


def test_failed_event_record_is_attributed_to_the_task():
    cfg, plan, desc = _setup()
    ex = Executor(plan, desc, device="cpu", seed=1)
    ex.initialize()
    ex.rt.mock_fail("event_record", 3)
    with pytest.raises(RuntimeFailure) as e:
        ex.run(_batches(cfg))
    assert e.value.info["status"] == native.BACKEND_FAILURE
    ex.closed = True
    ex.rt.close()


def test_pool_allocation_failure_is_reported_at_creation():
    lib = native.core()
    backend = lib.ss_mock_backend_create(0.0, 0)
    lib.ss_mock_fail_operation(backend, native.OP_KINDS.index("device_alloc"), 1)
    import ctypes as C
    cfg = native.RuntimeConfig(1 << 20, 1 << 20, -1, 0, 1000, 0, 0, None)
    handle = native.vp()
    assert lib.ss_runtime_create(backend, C.byref(cfg), C.byref(handle)) == native.OOM


def test_trace_ring_records_the_step():
    cfg, plan, desc = _setup()
    ex = Executor(plan, desc, device="cpu", seed=1, trace_capacity=4096)
    ex.initialize()
    res = ex.run(_batches(cfg), trace=True, time_tasks=True)
    kinds = {e["kind"] for e in res.trace}
    assert {"step_begin", "task_begin", "task_end", "fetch_issue", "step_end"} <= kinds
    assert sum(e["kind"] == "task_end" for e in res.trace) == len(plan.program.tasks)
    assert len(res.task_seconds) == len(plan.program.tasks)
    ex.close()


def test_membership_lease_expiry_fences_permanently():
    now = [0.0]
    m = Membership(lease_seconds=10.0, clock=lambda: now[0])
    inc = m.join("node-a")
    now[0] = 5.0
    assert m.heartbeat("node-a", inc) and m.live() == ["node-a"]
    now[0] = 30.0
    assert m.reconcile() == ["node-a"] and m.live() == []
    assert not m.heartbeat("node-a", inc)                    # a late heartbeat is refused
    inc2 = m.join("node-a")
    assert inc2 != inc and m.heartbeat("node-a", inc2)
    assert not m.heartbeat("node-a", inc)                    # the old incarnation stays fenced


def test_node_commands_are_delivered_until_acknowledged():
    now = [0.0]
    m = Membership(lease_seconds=10.0, clock=lambda: now[0])
    inc = m.join("node-a")
    cid = m.enqueue("node-a", {"kind": "drain"})
    assert [c["id"] for c in m.poll("node-a", inc)] == [cid]
    assert [c["id"] for c in m.poll("node-a", inc)] == [cid]          # not acknowledged: again
    assert m.receipt("node-a", inc, cid, {"state": "done"}) and m.poll("node-a", inc) == []
    assert not m.receipt("node-a", inc, cid)                          # only once
    now[0] = 8.0
    assert m.poll("node-a", inc) == []                                # a poll renews the lease
    now[0] = 17.0
    assert m.live() == ["node-a"]
    now[0] = 40.0
    assert m.poll("node-a", inc) is None                              # expired: fenced
    with pytest.raises(KeyError):
        m.enqueue("node-a", {"kind": "drain"})
    new = m.join("node-a")
    assert m.poll("node-a", inc) is None and m.poll("node-a", new) == []


def test_node_admission_never_oversubscribes():
    adm = NodeAdmission(gpus=4, host_bytes=100)
    a, devs = adm.lease(3, 60)
    assert devs == (0, 1, 2)
    with pytest.raises(AdmissionError):
        adm.lease(2, 10)
    with pytest.raises(AdmissionError):
        adm.lease(1, 50)
    adm.release(a)
    assert adm.lease(4, 100)[1] == (0, 1, 2, 3)


def test_journal_chain_detects_tampering(tmp_path):
    j = Journal(tmp_path)
    for i in range(5):
        j.append("receipt", {"i": i})
    assert [r["data"]["i"] for r in Journal(tmp_path).records("receipt")] == list(range(5))
    victim = tmp_path / "000000000002.json"
    victim.write_text(victim.read_text().replace('"i": 2', '"i": 9'))
    with pytest.raises(JournalCorrupt):
        Journal(tmp_path)


def test_operation_state_machine():
    s = OperationState()
    s.admit("forward_backward"); s.complete("forward_backward")
    for op in ("step", "save", "restore"):
        with pytest.raises(Rejected):
            s.admit(op)
    s.admit("optim_step"); s.complete("optim_step")
    assert s.b.completed_updates == 1 and s.b.accumulation == 0
    with pytest.raises(Rejected):
        s.admit("optim_step")                                # nothing accumulated
    s.fail("unknown")
    with pytest.raises(Rejected):
        s.admit("step")
    s.admit("close")                                         # the only thing still accepted


def test_controller_never_replays_and_propagates_failed_dependencies():
    calls = []

    def execute(req, payload):
        calls.append(req["request_id"])
        if req["operation"] == "forward_backward":
            err = RuntimeError("worker lost"); err.effect = "unknown"
            raise err
        return {"loss": 1.0}
    c = RunController(execute)
    a = {"request_id": "a", "operation": "step", "dependencies": [], "digest": "d1"}
    c.register(a)
    assert c.wait("a", 5).state == "completed"
    assert c.register(a).state == "completed" and calls == ["a"]          # idempotent, not replayed
    with pytest.raises(Rejected):
        c.register(dict(a, digest="other"))
    c.register({"request_id": "b", "operation": "forward_backward", "dependencies": ["a"], "digest": "d2"})
    rb = c.wait("b", 5)
    assert rb.state == "failed" and rb.effect == "unknown"
    c.register({"request_id": "c", "operation": "step", "dependencies": ["b"], "digest": "d3"})
    assert c.wait("c", 5).state == "rejected" and calls == ["a", "b"]
    c.stop()


def test_invalid_worker_group_still_accepts_close():
    from shadowspill_b200.training.group import WorkerFailure, WorkerGroup
    import pytest
    g = WorkerGroup.__new__(WorkerGroup)
    g.valid, g.chans, g.procs = False, [object()], []
    with pytest.raises(WorkerFailure):
        g.execute("r1", "step", {})
    assert g.execute("r2", "close", {})[0]["state"] == "completed"


@pytest.mark.parametrize("bad", [1, -1])
def test_host_agreement_stops_every_rank_before_the_collectives(bad):
    """Three gloo ranks; one raises while preparing the invocation. Every rank learns of it over
    the control group and none enters the collective; with no failure they all proceed, and a
    mismatch of the selected operation is refused too."""
    import os
    import subprocess
    from pathlib import Path
    worker = Path(__file__).with_name("_coord_worker.py")
    env = dict(os.environ, MASTER_ADDR="127.0.0.1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=3",
           "--master-addr", "127.0.0.1", "--master-port", "29683" if bad >= 0 else "29685", str(worker), str(bad)]
    out = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-2000:]
    assert out.stdout.count(" OK refused" if bad >= 0 else " OK ran") == 3, out.stdout[-2000:]
