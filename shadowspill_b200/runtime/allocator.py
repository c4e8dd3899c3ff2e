"""Python side of the allocation adapter (``csrc/adapter/allocator.cpp``).

``install()`` makes the adapter PyTorch's CUDA allocator for this process; it has to run before
the process allocates any CUDA tensor, which is why execution happens in a fresh worker process
(reference: packages/engine/src/shadowspill/runtime/bootstrap.py:122 ``install_runtime``). After
that, ``configure`` hands it the workspace slice of the runtime's device pool, and every task
runs inside ``task(name, ...)``: its tensors come out of the slice, its sequence of requests is
recorded (profiling) or checked against the recorded contract (execution), and a slice that
runs out or a contract that is broken surfaces as ``torch.OutOfMemoryError`` /
``AllocationContractViolation`` naming the task
(packages/engine/src/shadowspill/pytorch/runtime_adapter/boundaries.py:32-55,
docs/architecture/task-boundaries.md:147-151).
"""
from __future__ import annotations

import ctypes as C
from contextlib import contextmanager
from pathlib import Path

_DIR = Path(__file__).resolve().parents[1] / "csrc"
CUDA_LIB = _DIR / "libss_allocator.so"
HOST_LIB = _DIR / "libss_allocator_host.so"

OFF, RECORD, CHECK = 0, 1, 2


class AllocationContractViolation(RuntimeError):
    """A task asked the allocator for something else than it did when it was profiled."""


class Adapter:
    """ctypes view of one loaded adapter library (the CUDA build, or the host build in tests)."""

    def __init__(self, path: Path):
        self.path = Path(path)
        lib = C.CDLL(str(self.path))
        lib.ss_alloc.restype = C.c_void_p
        lib.ss_alloc.argtypes = [C.c_int64, C.c_int, C.c_void_p]
        lib.ss_free.restype = None
        lib.ss_free.argtypes = [C.c_void_p, C.c_int64, C.c_int, C.c_void_p]
        lib.ss_alloc_configure.argtypes = [C.c_void_p, C.c_int64, C.c_void_p]
        lib.ss_alloc_begin_task.argtypes = [C.c_char_p, C.c_int, C.POINTER(C.c_int64), C.c_int64]
        lib.ss_alloc_end_task.restype = C.c_int64
        lib.ss_alloc_sequence.restype = C.c_int64
        lib.ss_alloc_sequence.argtypes = [C.POINTER(C.c_int64), C.c_int64]
        lib.ss_alloc_take_error.argtypes = [C.c_char_p, C.c_int64]
        lib.ss_alloc_stats.argtypes = [C.POINTER(C.c_int64)]
        lib.ss_alloc_stats.restype = None
        lib.ss_alloc_reset_peak.restype = None
        lib.ss_alloc_trim.restype = None
        self.lib = lib

    def configure(self, base: int, nbytes: int, stream: int | None = None) -> None:
        if self.lib.ss_alloc_configure(base, nbytes, stream) != 0:
            raise RuntimeError("the workspace slice still holds live tensors")

    def begin_task(self, name: str, mode: int = OFF, expected: list[int] | None = None) -> None:
        arr = (C.c_int64 * len(expected))(*expected) if expected else None
        if self.lib.ss_alloc_begin_task(name.encode(), mode, arr, len(expected) if expected else 0) != 0:
            raise RuntimeError("a task scope is already open")

    def end_task(self) -> list[int]:
        n = self.lib.ss_alloc_end_task()
        if n < 0:
            raise RuntimeError("no task scope is open")
        buf = (C.c_int64 * max(1, n))()
        self.lib.ss_alloc_sequence(buf, n)
        return list(buf[:n])

    def raise_if_failed(self) -> None:
        buf = C.create_string_buffer(1024)
        kind = self.lib.ss_alloc_take_error(buf, len(buf))
        if kind == 1:
            import torch
            raise torch.OutOfMemoryError(buf.value.decode())
        if kind == 2:
            raise AllocationContractViolation(buf.value.decode())

    @contextmanager
    def task(self, name: str, mode: int = OFF, expected: list[int] | None = None):
        """Scope of one task; yields a list that holds the recorded request sizes afterwards."""
        record: list[int] = []
        self.begin_task(name, mode, expected)
        try:
            yield record
        finally:
            record.extend(self.end_task())
        self.raise_if_failed()

    def stats(self) -> dict[str, int]:
        buf = (C.c_int64 * 9)()
        self.lib.ss_alloc_stats(buf)
        keys = ("slice_bytes", "in_use", "peak", "task_peak", "driver_bytes", "driver_cached",
                "slice_allocations", "driver_allocations", "cache_hits")
        return dict(zip(keys, buf))

    def reset_peak(self) -> None:
        self.lib.ss_alloc_reset_peak()

    def trim(self) -> None:
        self.lib.ss_alloc_trim()


_installed: Adapter | None = None


def installed() -> Adapter | None:
    return _installed


def install() -> Adapter:
    """Makes the adapter this process's CUDA allocator. Must precede every CUDA allocation."""
    global _installed
    if _installed is not None:
        return _installed
    import torch
    if not CUDA_LIB.exists():
        raise RuntimeError(f"{CUDA_LIB} is not built; run `python -m shadowspill_b200.build`")
    if torch.cuda.is_initialized() and torch.cuda.memory_allocated() > 0:
        raise RuntimeError("the allocation adapter must be installed before the first CUDA allocation "
                           "(run execution in a fresh process)")
    alloc = torch.cuda.memory.CUDAPluggableAllocator(str(CUDA_LIB), "ss_alloc", "ss_free")
    torch.cuda.memory.change_current_allocator(alloc)
    adapter = Adapter(CUDA_LIB)          # the same loaded library: dlopen returns one instance per path
    adapter.torch_allocator = alloc
    _installed = adapter
    return adapter
