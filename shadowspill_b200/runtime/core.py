"""Python handle of the native execution runtime.

One ``Runtime`` owns one device pool and one pinned spill pool on one backend
(``cuda`` through the dlopened CUDA backend, or ``mock`` = host memory with
real stream threads). It exposes both pools as zero-copy ``torch`` byte tensors,
admits plans, and drives the step protocol. Reference counterparts:
packages/engine/src/shadowspill/runtime/core.py:86 (``Runtime``) and
runtime/bootstrap.py:122 (``install_runtime``).
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import numpy as np
import torch

from .. import native
from ..ir.plan import Plan


class RuntimeFailure(RuntimeError):
    """The runtime's failure latch is set; carries the first recorded failure."""

    def __init__(self, info: dict):
        self.info = info
        super().__init__(f"runtime failure: {info.get('message', '')} "
                         f"(status={native.status_string(info.get('status', 0))}, "
                         f"task={info.get('task')}, object={info.get('object')}, "
                         f"action={info.get('action')})")


class _CudaBuffer:
    """Zero-copy bridge from a raw device pointer to ``torch.as_tensor``."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1",
                                         "data": (ptr, False), "version": 2}


@dataclass
class TransferRates:
    fetch_solo_bps: float
    fetch_concurrent_bps: float
    evict_solo_bps: float
    evict_concurrent_bps: float
    fetch_latency_ns: int
    evict_latency_ns: int


class Runtime:
    def __init__(self, device_bytes: int, spill_bytes: int, backend: str = "cuda",
                 device_index: int = 0, trace_capacity: int = 0, mock_bps: float = 0.0,
                 mock_latency_ns: int = 0, numa_node: int = -1,
                 device_pool: torch.Tensor | None = None, file_bytes: int = 0,
                 file_directory: str = "", file_image: str = "", file_create_image: bool = False,
                 file_chunk_bytes: int = 0, file_queue_depth: int = 0, file_io_threads: int = 0,
                 remote_address: str = "", file_adopt_image: bool = False):
        """``device_pool``: a caller-owned uint8 tensor to use as the device pool
        (a symmetric-memory allocation for multi-GPU plans); it must outlive the runtime.
        ``file_bytes > 0`` adds a file-backed spill pool in ``file_directory`` (an unlinked
        scratch file) or in the kept file ``file_image``; objects homed there move through
        pinned staging rings of ``file_queue_depth`` chunks of ``file_chunk_bytes``.
        ``remote_address`` ("host:port" of an ``ss_memory_daemon``) keeps those bytes in the
        daemon's memory instead of a local file. ``file_adopt_image`` opens an existing
        ``file_image`` read-only as the pool's first bytes (the rest is a scratch file in
        ``file_directory``): state imported into the image can be read by many runs, and any
        transfer that would write into it fails."""
        self.lib = native.core()
        self.backend_name = backend
        self.device_index = device_index
        if backend == "mock":
            self.backend = self.lib.ss_mock_backend_create(float(mock_bps), int(mock_latency_ns))
        elif backend == "cuda":
            if not native.CUDA_BACKEND_PATH.exists():
                from .. import build
                build.build_core()
            err = C.create_string_buffer(256)
            self.backend = self.lib.ss_backend_dlopen(str(native.CUDA_BACKEND_PATH).encode(),
                                                      device_index, err, 256)
            if not self.backend:
                raise RuntimeError(f"cannot open CUDA backend: {err.value.decode()}")
        else:
            raise ValueError(f"unknown backend {backend!r}")
        external = None
        if device_pool is not None:
            if device_pool.numel() < device_bytes:
                raise ValueError("device_pool is smaller than the plan's device bytes")
            external = device_pool.data_ptr()
            self._external_pool = device_pool
        if file_bytes > 0 and not (file_directory or file_image or remote_address):
            raise ValueError("a file pool needs a directory, an image path or a daemon address")
        if file_adopt_image and not (file_image and file_directory):
            raise ValueError("adopting an image needs the image and a directory for the scratch part")
        if file_chunk_bytes % 4096:
            raise ValueError("file_chunk_bytes must be a multiple of 4096")
        cfg = native.RuntimeConfig(int(device_bytes), int(spill_bytes), numa_node,
                                   int(trace_capacity), 1000, 0, 0, external,
                                   int(file_bytes), str(file_directory).encode() or None,
                                   str(file_image).encode() or None,
                                   2 if file_adopt_image else int(bool(file_create_image)),
                                   int(file_queue_depth), int(file_chunk_bytes),
                                   int(file_io_threads), 0, str(remote_address).encode() or None)
        self.file_bytes = int(file_bytes)
        handle = native.vp()
        native.check(self.lib.ss_runtime_create(self.backend, C.byref(cfg), C.byref(handle)),
                     "ss_runtime_create")
        self.handle = handle
        self.device_bytes, self.spill_bytes = int(device_bytes), int(spill_bytes)
        self._closed = False
        dbase = self.lib.ss_runtime_device_base(handle) or 0
        sbase = self.lib.ss_runtime_spill_base(handle) or 0
        self.device_base, self.spill_base = dbase, sbase
        if spill_bytes > 0:
            arr = np.ctypeslib.as_array((C.c_uint8 * int(spill_bytes)).from_address(sbase))
            self.spill = torch.from_numpy(arr)
        else:
            self.spill = torch.empty(0, dtype=torch.uint8)
        if device_pool is not None:
            self.device = device_pool
        elif device_bytes == 0:
            self.device = torch.empty(0, dtype=torch.uint8)
        elif backend == "cuda":
            with torch.cuda.device(device_index):
                self.device = torch.as_tensor(_CudaBuffer(dbase, int(device_bytes)),
                                              device=f"cuda:{device_index}")
        else:
            arr = np.ctypeslib.as_array((C.c_uint8 * int(device_bytes)).from_address(dbase))
            self.device = torch.from_numpy(arr)
        self._plan_keep: dict[int, object] = {}

    # ------------------------------------------------------------------ plans
    def admit(self, plan: Plan) -> int:
        desc, keep = plan.to_native_desc()
        pid = native.i32(0)
        rc = self.lib.ss_plan_admit(self.handle, C.byref(desc), C.byref(pid))
        self._raise(rc, "ss_plan_admit")
        self._plan_keep[pid.value] = keep
        return pid.value

    def close_plan(self, plan_id: int) -> None:
        self._raise(self.lib.ss_plan_close(self.handle, plan_id), "ss_plan_close")
        self._plan_keep.pop(plan_id, None)

    # ------------------------------------------------------------------ step protocol
    def step_begin(self, plan_id: int, compute_stream: int | None) -> None:
        self._raise(self.lib.ss_step_begin(self.handle, plan_id, compute_stream), "ss_step_begin")

    def before_task(self, plan_id: int, task: int, n_uses: int, stream: int | None = None) -> list[int]:
        """``stream``: raw handle of the stream the task runs on when that is not the step's
        compute stream (a collective on the communication stream)."""
        buf = (native.vp * max(1, n_uses))()
        self._raise(self.lib.ss_before_task_on(self.handle, plan_id, task, buf, n_uses, stream),
                    "ss_before_task")
        return [int(buf[i] or 0) for i in range(n_uses)]

    def after_task(self, plan_id: int, task: int, stream: int | None = None) -> None:
        self._raise(self.lib.ss_after_task_on(self.handle, plan_id, task, stream), "ss_after_task")

    def step_end(self, plan_id: int) -> None:
        self._raise(self.lib.ss_step_end(self.handle, plan_id), "ss_step_end")

    def step_abandon(self, plan_id: int, why: str) -> None:
        """Ends a step whose task raised: the failure is latched and the plan can be closed."""
        self.lib.ss_step_abandon(self.handle, plan_id, why.encode()[:200])

    # ------------------------------------------------------------------ diagnostics
    def failure(self) -> dict | None:
        f = native.Failure()
        if self.lib.ss_runtime_failure(self.handle, C.byref(f)) != native.OK:
            return None
        return {"status": f.status, "reason": f.reason, "task": f.task, "object": f.object,
                "action": f.action, "pool": f.pool, "message": f.message.decode(errors="replace")}

    def latch_failure(self, message: str, status: int = native.FAILED, reason: int = 7) -> None:
        self.lib.ss_runtime_latch_failure(self.handle, reason, status, message.encode())

    def stats(self) -> dict[str, int]:
        s = native.RuntimeStats()
        self.lib.ss_runtime_stats_read(self.handle, C.byref(s))
        return {n: getattr(s, n) for n, _ in native.RuntimeStats._fields_}

    def trace_begin(self) -> None:
        native.check(self.lib.ss_trace_begin(self.handle), "ss_trace_begin")

    def trace_end(self) -> list[dict]:
        self.lib.ss_trace_end(self.handle)
        cap = 1 << 16
        buf = (native.TraceEvent * cap)()
        n = self.lib.ss_trace_read(self.handle, buf, cap)
        return [{"kind": native.TRACE_KINDS[buf[i].kind], "id": buf[i].a,
                 "host_ns": buf[i].host_ns, "bytes": buf[i].bytes} for i in range(n)]

    def transfer_times(self, plan_id: int, n_actions: int) -> tuple[list[int], list[int]]:
        """Device-clock ``(begin_ns, end_ns)`` of each action's copy in the plan's last
        step, relative to the step's start; -1 for releases. Needs ``trace_capacity > 0``."""
        b = (native.i64 * max(n_actions, 1))()
        e = (native.i64 * max(n_actions, 1))()
        n = self.lib.ss_plan_transfer_times(self.handle, plan_id, b, e, n_actions)
        if n < 0:
            return [], []
        return list(b[:n_actions]), list(e[:n_actions])

    def calibrate(self, nbytes: int = 256 << 20, repeats: int = 3) -> TransferRates:
        p = native.TransferProfile()
        native.check(self.lib.ss_calibrate_transfers(self.handle, int(nbytes), repeats, C.byref(p)),
                     "ss_calibrate_transfers")
        return TransferRates(p.fetch_solo_bps, p.fetch_concurrent_bps, p.evict_solo_bps,
                             p.evict_concurrent_bps, p.fetch_latency_ns, p.evict_latency_ns)

    def calibrate_file(self, nbytes: int = 256 << 20, repeats: int = 3) -> TransferRates:
        """Rates of the staged lanes between the device pool and the file pool."""
        p = native.TransferProfile()
        self._raise(self.lib.ss_calibrate_file_transfers(self.handle, int(nbytes), repeats, C.byref(p)),
                    "ss_calibrate_file_transfers")
        return TransferRates(p.fetch_solo_bps, p.fetch_concurrent_bps, p.evict_solo_bps,
                             p.evict_concurrent_bps, p.fetch_latency_ns, p.evict_latency_ns)

    def file_write(self, offset: int, data: torch.Tensor) -> None:
        """Writes a contiguous CPU tensor at ``offset`` of the file pool (durable on return)."""
        data = data.contiguous()
        n = data.numel() * data.element_size()
        self._raise(self.lib.ss_file_write(self.handle, int(offset), data.data_ptr(), n), "ss_file_write")

    def file_read(self, offset: int, nbytes: int) -> torch.Tensor:
        out = torch.empty(int(nbytes), dtype=torch.uint8)
        self._raise(self.lib.ss_file_read(self.handle, int(offset), out.data_ptr(), int(nbytes)),
                    "ss_file_read")
        return out

    def file_info(self) -> dict:
        direct, ring = native.i32(0), native.i64(0)
        native.check(self.lib.ss_runtime_file_info(self.handle, C.byref(direct), C.byref(ring)),
                     "ss_runtime_file_info")
        return {"direct_io": bool(direct.value), "ring_bytes": int(ring.value), "bytes": self.file_bytes}

    def mock_fail(self, op: str, nth: int) -> None:
        native.check(self.lib.ss_mock_fail_operation(self.backend, native.OP_KINDS.index(op), nth),
                     "ss_mock_fail_operation")

    def mock_count(self, op: str) -> int:
        return self.lib.ss_mock_operation_count(self.backend, native.OP_KINDS.index(op))

    # ------------------------------------------------------------------ lifecycle
    def close(self) -> None:
        if self._closed:
            return
        self._closed = True
        self.device = self.spill = None
        self.lib.ss_runtime_close(self.handle)
        self.lib.ss_runtime_destroy(self.handle)

    def abandon(self) -> None:
        """Process-exit path: no drain, no synchronisation."""
        if not self._closed:
            self._closed = True
            self.lib.ss_runtime_abandon(self.handle)

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    def _raise(self, rc: int, what: str) -> None:
        if rc == native.OK:
            return
        info = self.failure()
        if info is not None:
            raise RuntimeFailure(info)
        raise native.NativeError(rc, what)
