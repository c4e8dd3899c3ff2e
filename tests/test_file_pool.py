"""File-backed spill pool and its staged lanes, on the mock backend.

The file lives in a temporary directory; copies are host memcpys on ordered stream
threads, so the whole path (disk threads, pinned rings, slot events, durable evicts,
reuse dependencies) runs as it does with a GPU.
"""
import copy
import sys

import pytest
import torch

sys.path.insert(0, __file__.rsplit("/", 1)[0])
from test_executor_cpu import _batches, _setup  # noqa: E402

from shadowspill_b200 import native
from shadowspill_b200.execution.executor import Executor
from shadowspill_b200.ir.plan import Plan
from shadowspill_b200.planning.plan import move_homes_to_file
from shadowspill_b200.runtime.core import Runtime, RuntimeFailure


def test_whole_object_io_and_lane_calibration(tmp_path):
    rt = Runtime(8 << 20, 1 << 20, backend="mock", file_bytes=8 << 20, file_directory=str(tmp_path),
                 file_chunk_bytes=64 << 10, file_queue_depth=3)
    info = rt.file_info()
    assert info["ring_bytes"] == 3 * (64 << 10) and info["bytes"] == 8 << 20
    data = torch.arange(100_000, dtype=torch.int32)
    rt.file_write(4096 + 12, data)                       # unaligned offset and length
    back = rt.file_read(4096 + 12, data.numel() * 4).view(torch.int32)
    assert torch.equal(back, data)
    rates = rt.calibrate_file(2 << 20, repeats=2)
    assert rates.fetch_solo_bps > 0 and rates.evict_solo_bps > 0
    assert rates.fetch_concurrent_bps <= rates.fetch_solo_bps
    with pytest.raises(native.NativeError):
        rt.file_read(8 << 20, 16)                        # outside the pool
    rt.close()
    assert list(tmp_path.iterdir()) == []                # the scratch file was never linked


def test_runtime_refuses_a_file_home_without_a_file_pool():
    cfg, plan, desc = _setup()
    move_homes_to_file(plan)
    with pytest.raises(ValueError):
        Executor(plan, desc, device="cpu", seed=1)


def _train(plan, desc, cfg, steps=4, **kw):
    ex = Executor(plan, desc, device="cpu", seed=1, **kw)
    ex.initialize()
    losses = [ex.run(_batches(cfg, s)).loss for s in range(steps)]
    state = ex.state_dict()
    stats = ex.rt.stats()
    ex.close()
    return losses, state, stats


@pytest.mark.parametrize("chunk,depth,io", [(4096, 2, 0), (16 << 10, 3, 0), (1 << 20, 16, 0),
                                            (8192, 1, 1), (64 << 10, 5, 8)])
def test_training_through_the_file_pool_is_bit_identical(tmp_path, chunk, depth, io):
    cfg, plan, desc = _setup()
    host_losses, host_state, host_stats = _train(copy.deepcopy(plan), desc, cfg)
    filed = move_homes_to_file(copy.deepcopy(plan))
    assert filed.file_bytes >= plan.spill_bytes and filed.spill_bytes < plan.spill_bytes
    n_file = sum(o >= 0 for o in filed.file_offsets)
    assert n_file > 0 and all(filed.spill_offsets[i] < 0 for i, o in enumerate(filed.file_offsets) if o >= 0)
    assert filed.home_pool(filed.program.objects.index(
        next(o for o in filed.program.objects if o.name == "batch.0"))) == "host"
    # the record survives its JSON form
    again = Plan.from_json(filed.to_json())
    assert again.file_offsets == filed.file_offsets and again.file_bytes == filed.file_bytes
    losses, state, stats = _train(again, desc, cfg, file_pool={
        "directory": str(tmp_path), "chunk_bytes": chunk, "queue_depth": depth, "io_threads": io})
    assert losses == host_losses
    assert set(state) == set(host_state)
    for k in state:
        assert torch.equal(state[k], host_state[k]), k
    assert stats["fetch_bytes"] == host_stats["fetch_bytes"]
    assert stats["evict_bytes"] == host_stats["evict_bytes"]
    # everything except the pinned batches and the loss word went through the rings, chunk by chunk
    assert 0 < stats["staged_read_bytes"] <= stats["fetch_bytes"]
    assert 0 < stats["staged_write_bytes"] <= stats["evict_bytes"]
    assert stats["staged_read_chunks"] >= stats["staged_read_bytes"] // chunk
    assert host_stats["staged_read_bytes"] == 0 and host_stats["staged_write_chunks"] == 0


def test_a_kept_image_carries_state_to_the_next_run(tmp_path):
    cfg, plan, desc = _setup()
    filed = move_homes_to_file(plan)
    image = tmp_path / "pool.img"
    ex = Executor(copy.deepcopy(filed), desc, device="cpu", seed=1,
                  file_pool={"image": str(image), "create_image": True})
    ex.initialize()
    first = [ex.run(_batches(cfg, s)).loss for s in range(2)]
    state = ex.state_dict()
    done = ex.runner.completed_updates
    ex.close()
    assert image.stat().st_size >= filed.file_bytes
    with pytest.raises(native.NativeError):                 # creating over an existing image is refused
        Executor(copy.deepcopy(filed), desc, device="cpu", seed=1,
                 file_pool={"image": str(image), "create_image": True})
    ex = Executor(copy.deepcopy(filed), desc, device="cpu", seed=1, file_pool={"image": str(image)})
    ex.runner.completed_updates = done
    for k, v in ex.state_dict().items():
        assert torch.equal(v, state[k]), k
    more = ex.run(_batches(cfg, 2)).loss
    ex.close()
    # the same three steps in one run
    ref = Executor(copy.deepcopy(plan), desc, device="cpu", seed=1, file_pool={"directory": str(tmp_path)})
    ref.initialize()
    ref_losses = [ref.run(_batches(cfg, s)).loss for s in range(3)]
    ref.close()
    assert first + [more] == ref_losses


def test_an_adopted_image_is_read_in_place_and_never_written(tmp_path):
    cfg, plan, desc = _setup()
    filed = move_homes_to_file(plan)
    image = tmp_path / "pool.img"
    ex = Executor(copy.deepcopy(filed), desc, device="cpu", seed=1,
                  file_pool={"image": str(image), "create_image": True})
    ex.initialize()
    ex.run(_batches(cfg))
    state = ex.state_dict()
    ex.close()
    size = image.stat().st_size
    digest = __import__("hashlib").sha256(image.read_bytes()).hexdigest()
    scratch = tmp_path / "scratch"
    scratch.mkdir()
    ex = Executor(copy.deepcopy(filed), desc, device="cpu", seed=1,
                  file_pool={"image": str(image), "adopt_image": True, "directory": str(scratch)})
    for k, v in ex.state_dict().items():            # the imported state is readable in place
        assert torch.equal(v, state[k]), k
    with pytest.raises((RuntimeFailure, native.NativeError)):
        ex.run(_batches(cfg, 1))                    # training writes its state back: refused
    info = ex.rt.failure()
    assert info is not None and info["pool"] == 2
    ex.closed = True
    ex.rt.close()
    assert image.stat().st_size == size and __import__("hashlib").sha256(image.read_bytes()).hexdigest() == digest
    # a pool larger than the image: the part beyond it is scratch and writable
    rt = Runtime(1 << 20, 4096, backend="mock", file_bytes=size + (1 << 20), file_image=str(image),
                 file_adopt_image=True, file_directory=str(scratch))
    blob = torch.arange(5000, dtype=torch.int32)
    rt.file_write(size + 4096, blob)
    assert torch.equal(rt.file_read(size + 4096, 20000).view(torch.int32), blob)
    straddle = rt.file_read(size - 8, 16)           # a read across the boundary comes from both files
    assert straddle.numel() == 16
    with pytest.raises(native.NativeError):
        rt.file_write(size - 8, blob)               # touches the image: refused
    rt.close()
    with pytest.raises(ValueError):
        Runtime(1 << 20, 4096, backend="mock", file_bytes=size, file_image=str(image), file_adopt_image=True)


def test_a_failed_host_copy_in_a_staged_lane_latches(tmp_path):
    cfg, plan, desc = _setup()
    ex = Executor(move_homes_to_file(plan), desc, device="cpu", seed=1,
                  file_pool={"directory": str(tmp_path), "chunk_bytes": 16 << 10, "queue_depth": 2})
    ex.initialize()
    ex.run(_batches(cfg))
    ex.rt.mock_fail("copy", 7)
    with pytest.raises(RuntimeFailure) as e:
        ex.run(_batches(cfg, 1))
    assert e.value.info["pool"] == 2 and "staged" in e.value.info["message"]
    ex.closed = True
    ex.rt.close()


def test_session_with_a_file_spill_pool_matches_the_pinned_one(tmp_path):
    from shadowspill_b200.planning.plan import SearchOptions
    from shadowspill_b200.training.session import TrainingSession, TrainingSetup
    common = dict(model="llama3-tiny", device_gib=0.53, spill_gib=0.25, tokens_per_step=512,
                  microbatch_tokens=256, dtype="float32", stochastic_rounding=False, device="cpu",
                  profile=False, calibrate=False, seed=3, lr=3e-3,
                  search=SearchOptions(minimum_object_bytes_evict_eligible=1024, workers=1))
    losses = {}
    for pool in ("host", "file"):
        extra = dict(spill_pool="file", spill_directory=str(tmp_path), spill_chunk_bytes=8192,
                     spill_queue_depth=4) if pool == "file" else {}
        s = TrainingSession(TrainingSetup(**common, **extra))
        cfg = s.cfg
        losses[pool] = [s.step(_batches(cfg, i)).loss for i in range(3)]
        if pool == "file":
            assert s.plan.file_bytes > 0 and s.plan.spill_bytes < 1 << 20
            s.save(tmp_path / "ckpt")
            more = s.step(_batches(cfg, 3)).loss
            s.restore(tmp_path / "ckpt")
            assert s.step(_batches(cfg, 3)).loss == more
        s.close()
    assert losses["file"] == losses["host"]
    with pytest.raises(ValueError):
        TrainingSession(TrainingSetup(**common, spill_pool="file"))


def test_client_memory_record_validates_the_file_pool(tmp_path):
    from shadowspill_b200.client import Memory
    Memory(device_gib=1, spill_gib=2, spill_pool="file", spill_directory=str(tmp_path))
    for bad in (dict(spill_pool="tape"), dict(spill_pool="file", spill_gib=1),
                dict(spill_pool="file", spill_gib=1, spill_directory="x", spill_chunk_bytes=1000)):
        with pytest.raises(ValueError):
            Memory(**bad)


@pytest.mark.gpu
def test_file_pool_with_the_cuda_backend_matches_the_pinned_pool(tmp_path):
    """Real pinned rings, CUDA events on the slots and copies on the lane streams: the same
    plan run from a file and from pinned memory gives the same losses and state."""
    from shadowspill_b200.communication.info import CommunicationInfo
    from shadowspill_b200.data.synthetic import make_batch
    from shadowspill_b200.execution.executor import Hyperparameters
    from shadowspill_b200.frontend.capture import BatchGeometry, StepDataOrdering, build_step
    from shadowspill_b200.models.config import DecoderConfig
    from shadowspill_b200.planning.plan import MemoryBudgets, PlanningError, SearchOptions, plan_program
    cfg = DecoderConfig("llama3", 3, 512, 4, 2, 128, 1024, 4096)
    geo = BatchGeometry(1024, 3, slots=32, mean_seqlen=200)
    prog, desc = build_step(cfg, geo, StepDataOrdering())
    total = sum(o.bytes for o in prog.objects)
    ws = max(t.workspace_bytes for t in prog.tasks)
    plan = None
    for pct in range(25, 101, 5):
        try:
            plan = plan_program(prog, MemoryBudgets(2 * ws + total * pct // 100, 1 << 30, headroom_bytes=0),
                                CommunicationInfo(), SearchOptions(minimum_object_bytes_evict_eligible=4096))
            break
        except PlanningError:
            continue
    assert plan is not None and plan.summary.fetch_bytes > 0

    def run(p, **kw):
        ex = Executor(p, desc, device="cuda", seed=3, hyper=Hyperparameters(lr=1e-3),
                      stochastic_rounding=False, **kw)
        ex.initialize(on_device=False)
        losses = []
        for step in range(3):
            host = make_batch(step, vocab=cfg.vocab_size, tokens_per_step=3072, microbatch_tokens=1024,
                              median=200, min_len=16, max_len=512, slots=32)
            losses.append(ex.run(host).loss)
        state = ex.state_dict()
        info = ex.rt.file_info() if p.file_bytes else None
        ex.close()
        return losses, state, info

    host_losses, host_state, _ = run(copy.deepcopy(plan))
    filed = move_homes_to_file(copy.deepcopy(plan))
    losses, state, info = run(filed, file_pool={"directory": str(tmp_path), "chunk_bytes": 256 << 10,
                                                "queue_depth": 4})
    assert info["ring_bytes"] == 1 << 20
    # the only run-to-run difference is the atomic order of embedding gradients
    for a, b in zip(losses, host_losses):
        assert abs(a - b) < 1e-3 * abs(b)
    for k, v in host_state.items():
        a, b = state[k].float().reshape(-1), v.float().reshape(-1)
        assert float((a - b).norm() / (b.norm() + 1e-12)) < 2.5e-2, k
    rt = Runtime(64 << 20, 4096, backend="cuda", file_bytes=64 << 20, file_directory=str(tmp_path))
    rates = rt.calibrate_file(16 << 20, repeats=2)
    assert rates.fetch_solo_bps > 0 and rates.evict_solo_bps > 0
    rt.close()


# ---------------------------------------------------------------------------- remote pool
@pytest.fixture()
def memory_daemon():
    """A real ``ss_memory_daemon`` on a free loopback port."""
    import subprocess
    from shadowspill_b200 import build
    build.build_core()
    proc = subprocess.Popen([str(build.MEMORY_DAEMON), "--port", "0", "--capacity-gib", "0.25"],
                            stdout=subprocess.PIPE, text=True)
    line = proc.stdout.readline().split()
    assert line[0] == "listening"
    yield f"127.0.0.1:{line[1]}"
    proc.kill()
    proc.wait()


def _daemon_stat(address):
    import socket
    host, port = address.rsplit(":", 1)
    with socket.create_connection((host, int(port)), timeout=5) as s:
        s.sendall(b"STAT\n")
        reply = s.makefile().readline().split()
    assert reply[0] == "OK"
    return int(reply[1]), int(reply[2])


def test_training_from_a_memory_daemon_is_bit_identical(memory_daemon):
    cfg, plan, desc = _setup()
    host_losses, host_state, _ = _train(copy.deepcopy(plan), desc, cfg)
    filed = move_homes_to_file(copy.deepcopy(plan))
    ex = Executor(filed, desc, device="cpu", seed=1,
                  file_pool={"remote": memory_daemon, "chunk_bytes": 32 << 10, "queue_depth": 4})
    assert _daemon_stat(memory_daemon) == (1, filed.file_bytes)
    ex.initialize()
    losses = [ex.run(_batches(cfg, s)).loss for s in range(4)]
    state = ex.state_dict()
    ex.close()
    assert losses == host_losses
    for k in state:
        assert torch.equal(state[k], host_state[k]), k
    assert _daemon_stat(memory_daemon) == (0, 0)            # closing the run freed its region


def test_the_daemon_enforces_its_capacity_and_leases(memory_daemon):
    with pytest.raises(native.NativeError):
        Runtime(1 << 20, 4096, backend="mock", file_bytes=1 << 30, remote_address=memory_daemon)
    rt = Runtime(1 << 20, 4096, backend="mock", file_bytes=64 << 20, remote_address=memory_daemon)
    data = torch.arange(50_000, dtype=torch.int64)
    rt.file_write(12345, data)
    assert torch.equal(rt.file_read(12345, data.numel() * 8).view(torch.int64), data)
    assert rt.file_info()["direct_io"] is False
    rt.close()
    assert _daemon_stat(memory_daemon) == (0, 0)
    # a client that dies without FREE: the region's lease ends with its connection
    import socket
    import time
    host, port = memory_daemon.rsplit(":", 1)
    s = socket.create_connection((host, int(port)), timeout=5)
    s.sendall(b"ALLOCATE 1048576\n")
    assert s.makefile().readline().split()[0] == "OK"
    assert _daemon_stat(memory_daemon) == (1, 1 << 20)
    s.close()
    deadline = time.time() + 5
    while time.time() < deadline and _daemon_stat(memory_daemon)[0]:
        time.sleep(0.05)
    assert _daemon_stat(memory_daemon) == (0, 0)


def test_an_unreachable_daemon_is_an_error_not_a_hang():
    with pytest.raises(native.NativeError):
        Runtime(1 << 20, 4096, backend="mock", file_bytes=1 << 20, remote_address="127.0.0.1:1")


def test_session_with_a_remote_spill_pool(memory_daemon):
    from shadowspill_b200.planning.plan import SearchOptions
    from shadowspill_b200.training.session import TrainingSession, TrainingSetup
    common = dict(model="llama3-tiny", device_gib=0.53, spill_gib=0.1, tokens_per_step=512,
                  microbatch_tokens=256, dtype="float32", stochastic_rounding=False, device="cpu",
                  profile=False, calibrate=False, seed=3, lr=3e-3,
                  search=SearchOptions(minimum_object_bytes_evict_eligible=1024, workers=1))
    host = TrainingSession(TrainingSetup(**common))
    want = [host.step(_batches(host.cfg, i)).loss for i in range(3)]
    host.close()
    s = TrainingSession(TrainingSetup(**common, spill_pool="remote", spill_address=memory_daemon))
    assert [s.step(_batches(s.cfg, i)).loss for i in range(3)] == want
    s.close()
    with pytest.raises(ValueError):
        TrainingSession(TrainingSetup(**common, spill_pool="remote"))


def test_a_daemon_that_dies_between_steps_latches_an_io_failure():
    """The far side of the remote pool goes away: the next step ends with the runtime's failure
    latch set (pool 2, an I/O status), never with a hang, and the run refuses further steps."""
    import subprocess
    import time
    from shadowspill_b200 import build
    build.build_core()
    proc = subprocess.Popen([str(build.MEMORY_DAEMON), "--port", "0"], stdout=subprocess.PIPE, text=True)
    address = f"127.0.0.1:{proc.stdout.readline().split()[1]}"
    cfg, plan, desc = _setup()
    ex = Executor(move_homes_to_file(plan), desc, device="cpu", seed=1,
                  file_pool={"remote": address, "chunk_bytes": 32 << 10, "queue_depth": 2})
    ex.initialize()
    assert ex.run(_batches(cfg)).loss > 0
    proc.kill()
    proc.wait()
    t0 = time.time()
    with pytest.raises((RuntimeFailure, native.NativeError)) as e:
        ex.run(_batches(cfg, 1))
    assert time.time() - t0 < 20
    info = ex.rt.failure()
    assert info is not None and info["pool"] == 2 and info["status"] == native.IO_ERROR
    with pytest.raises((RuntimeFailure, native.NativeError)):
        ex.run(_batches(cfg, 2))
    ex.closed = True
    ex.rt.close()
