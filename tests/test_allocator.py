"""The allocation adapter's slice, task scopes and contract, on its host build (no GPU): the carve
logic is pointer arithmetic, so a fake base address exercises all of it."""
import ctypes as C

import pytest

from shadowspill_b200.runtime import allocator as al


@pytest.fixture()
def adapter():
    a = al.Adapter(al.HOST_LIB)
    a.lib.ss_alloc_take_error(None, 0)
    yield a
    a.configure(0, 0)


def test_tasks_carve_the_slice_and_driver_serves_the_rest(adapter):
    base, size = 1 << 40, 1 << 20
    adapter.configure(base, size, None)
    outside = adapter.lib.ss_alloc(1000, 0, None)                 # no task: a driver block
    assert not (base <= outside < base + size)
    with adapter.task("F.layer0.0", al.RECORD) as seq:
        a = adapter.lib.ss_alloc(1000, 0, None)
        b = adapter.lib.ss_alloc(4096, 0, None)
        other_stream = adapter.lib.ss_alloc(512, 0, C.c_void_p(0x10))   # a side stream: not the slice
        assert base <= a < base + size and base <= b < base + size and b - a == 1024   # 512-byte grain
        assert not (base <= other_stream < base + size)
        adapter.lib.ss_free(a, 1000, 0, None)
        c = adapter.lib.ss_alloc(700, 0, None)
        assert c == a                                             # first fit reuses the freed range
        adapter.lib.ss_free(b, 0, 0, None), adapter.lib.ss_free(c, 0, 0, None)
        adapter.lib.ss_free(other_stream, 0, 0, C.c_void_p(0x10))
    assert seq == [1000, 4096, 512, 700]
    st = adapter.stats()
    assert st["in_use"] == 0 and st["peak"] == 1024 + 4096 and st["slice_allocations"] == 3
    adapter.lib.ss_free(outside, 0, 0, None)
    again = adapter.lib.ss_alloc(900, 0, None)                    # the freed driver block is cached
    assert again == outside and adapter.stats()["cache_hits"] == 1
    adapter.lib.ss_free(again, 0, 0, None)
    adapter.trim()
    assert adapter.stats()["driver_cached"] == 0


def test_contract_is_checked_and_names_the_task(adapter):
    adapter.configure(1 << 40, 1 << 20, None)
    with adapter.task("B.layer3.1", al.CHECK, [256, 512]):
        p = adapter.lib.ss_alloc(256, 0, None)
        q = adapter.lib.ss_alloc(512, 0, None)
        adapter.lib.ss_free(p, 0, 0, None), adapter.lib.ss_free(q, 0, 0, None)
    with pytest.raises(al.AllocationContractViolation, match=r"B\.layer3\.1.*request 1 asks for 640"):
        with adapter.task("B.layer3.1", al.CHECK, [256, 512]):
            p = adapter.lib.ss_alloc(256, 0, None)
            q = adapter.lib.ss_alloc(640, 0, None)
            adapter.lib.ss_free(p, 0, 0, None), adapter.lib.ss_free(q, 0, 0, None)
    with pytest.raises(al.AllocationContractViolation, match="1 requests made, 2 recorded"):
        with adapter.task("B.layer3.1", al.CHECK, [256, 512]):
            adapter.lib.ss_free(adapter.lib.ss_alloc(256, 0, None), 0, 0, None)


def test_exhaustion_is_an_out_of_memory_error_that_names_the_task(adapter):
    import torch
    base, size = 1 << 40, 8192
    adapter.configure(base, size, None)
    with pytest.raises(torch.OutOfMemoryError, match=r"task H\.head\.0: workspace exhausted: 8000 bytes"):
        with adapter.task("H.head.0"):
            a = adapter.lib.ss_alloc(4096, 0, None)
            b = adapter.lib.ss_alloc(8000, 0, None)       # does not fit: served by the driver, latched
            assert base <= a < base + size and b and not (base <= b < base + size)
            adapter.lib.ss_free(a, 0, 0, None), adapter.lib.ss_free(b, 0, 0, None)
    # live tensors pin the slice
    with adapter.task("x"):
        a = adapter.lib.ss_alloc(512, 0, None)
    with pytest.raises(RuntimeError, match="live tensors"):
        adapter.configure(base, size, None)
    adapter.lib.ss_free(a, 0, 0, None)


@pytest.mark.gpu
@pytest.mark.parametrize("mode,expect", [("run", "OK ran"), ("graph", "OK ran"), ("violate", "OK violation"),
                                         ("oom", "OK oom")])
def test_adapter_in_a_fresh_worker_process(mode, expect):
    """Installed before the first CUDA use, the adapter serves every task tensor of a planned
    training step from the workspace slice; a broken contract and an exhausted workspace surface
    as errors that name the task. Nothing faults: an over-budget request is served by the driver."""
    import subprocess
    import sys
    from pathlib import Path
    worker = Path(__file__).with_name("_alloc_worker.py")
    out = subprocess.run([sys.executable, str(worker), mode], capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-3000:]
    assert expect in out.stdout, out.stdout[-2000:]
