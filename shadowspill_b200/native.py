"""ctypes projection of the native core (``csrc/libss_core.so``).

Structures mirror ``csrc/include/ss_core.h`` field for field; ``abi_check``
compares their sizes with the compiled ones so that a stale library is caught
at load time rather than by memory corruption. Planning and simulation entry
points release the GIL, so several searches can run from Python threads.
"""
from __future__ import annotations

import ctypes as C
import os
import threading
from pathlib import Path

import numpy as np

_DIR = Path(__file__).resolve().parent / "csrc"
# SS_CORE_LIB selects another build of the core (an instrumented one for race detection)
CORE_PATH = Path(os.environ["SS_CORE_LIB"]) if os.environ.get("SS_CORE_LIB") else _DIR / "libss_core.so"
CUDA_BACKEND_PATH = _DIR / "libss_backend_cuda.so"

i32, i64, f64, vp = C.c_int32, C.c_int64, C.c_double, C.c_void_p
P64, P32 = C.POINTER(i64), C.POINTER(i32)

OK, INVALID, OOM, NO_PROGRESS, BACKEND_FAILURE, CLOSED, FAILED, TIMEOUT, INFEASIBLE = range(9)
INTERNAL, IO_ERROR = 9, 10
USE_READ, USE_CREATE, USE_MUTATE = 0, 1, 2
OBJ_PERSISTENT, OBJ_PINNED_RESIDENT = 1, 2
ACT_FETCH, ACT_EVICT, ACT_RELEASE = 0, 1, 2
FETCH_RULES = ("demand", "latest-safe", "packed-fifo", "packed-fit")
STRATEGIES = ("stall", "traffic")
OP_KINDS = ("device_alloc", "host_alloc", "stream_create", "event_create", "event_record",
            "stream_wait", "copy", "memset", "sync")


class Program(C.Structure):
    _fields_ = [("n_tasks", i32), ("task_duration_ns", P64), ("task_workspace_bytes", P64),
                ("n_objects", i32), ("object_bytes", P64), ("object_flags", P32),
                ("n_uses", i32), ("use_task", P32), ("use_object", P32), ("use_mode", P32)]


class DeviceConfig(C.Structure):
    _fields_ = [("capacity_bytes", i64), ("fetch_solo_bps", f64), ("fetch_concurrent_bps", f64),
                ("evict_solo_bps", f64), ("evict_concurrent_bps", f64), ("fetch_latency_ns", i64),
                ("evict_latency_ns", i64), ("alignment", i64)]


class Action(C.Structure):
    _fields_ = [("kind", i32), ("object", i32), ("trigger_task", i32), ("reserved", i32)]


class Interval(C.Structure):
    _fields_ = [("object", i32), ("begin_action", i32), ("begin_task", i32), ("end_action", i32),
                ("bytes", i64), ("start_ns", i64), ("end_ns", i64), ("offset", i64)]


class SimResult(C.Structure):
    _fields_ = [("status", i32), ("stalled_task", i32), ("makespan_ns", i64), ("compute_ns", i64),
                ("input_wait_ns", i64), ("capacity_wait_ns", i64), ("peak_bytes", i64),
                ("fetch_bytes", i64), ("evict_bytes", i64), ("fetch_busy_ns", i64),
                ("evict_busy_ns", i64)]


class SearchOptions(C.Structure):
    _fields_ = [("workers", i32), ("strategy_mask", i32), ("fetch_rule_mask", i32),
                ("max_repairs", i32), ("minimum_object_bytes_evict_eligible", i64),
                ("capacity_refinement_step", i64), ("deterministic", i32), ("trace", i32),
                ("linear_reduce", i32), ("no_resident_slice", i32)]


class SearchSummary(C.Structure):
    _fields_ = [("status", i32), ("best_strategy", i32), ("best_fetch_rule", i32),
                ("candidates_evaluated", i32), ("candidates_feasible", i32),
                ("repairs_applied", i32), ("n_actions", i32), ("n_intervals", i32),
                ("logical_capacity", i64), ("layout_span", i64), ("sim", SimResult)]


class RuntimeConfig(C.Structure):
    _fields_ = [("device_bytes", i64), ("spill_bytes", i64), ("numa_node", i32),
                ("trace_capacity", i32), ("worker_poll_ns", i64), ("max_objects", i32),
                ("event_pool", i32), ("external_device_base", vp),
                ("file_bytes", i64), ("file_directory", C.c_char_p), ("file_image", C.c_char_p),
                ("file_create_image", i32), ("file_queue_depth", i32), ("file_chunk_bytes", i64),
                ("file_io_threads", i32), ("reserved0", i32), ("remote_address", C.c_char_p)]


class Failure(C.Structure):
    _fields_ = [("status", i32), ("reason", i32), ("task", i32), ("object", i32), ("action", i32),
                ("pool", i32), ("message", C.c_char * 192)]


class TraceEvent(C.Structure):
    _fields_ = [("kind", i32), ("a", i32), ("host_ns", i64), ("bytes", i64)]


class RuntimeStats(C.Structure):
    _fields_ = [(n, i64) for n in ("steps", "tasks", "fetches", "fetch_bytes", "evicts",
                                   "evict_bytes", "releases", "reuse_waits", "events_created",
                                   "host_allocations", "worker_wakeups", "staged_read_chunks",
                                   "staged_read_bytes", "staged_write_chunks", "staged_write_bytes")]


class PlanDesc(C.Structure):
    _fields_ = [("n_tasks", i32), ("n_objects", i32), ("object_bytes", P64), ("spill_offset", P64),
                ("n_actions", i32), ("actions", C.POINTER(Action)), ("n_intervals", i32),
                ("intervals", C.POINTER(Interval)), ("reuse_pred_begin", P32),
                ("reuse_pred_index", P32), ("n_uses", i32), ("use_task", P32),
                ("use_object", P32), ("use_mode", P32), ("file_offset", P64)]


class TransferProfile(C.Structure):
    _fields_ = [("fetch_solo_bps", f64), ("fetch_concurrent_bps", f64), ("evict_solo_bps", f64),
                ("evict_concurrent_bps", f64), ("fetch_latency_ns", i64), ("evict_latency_ns", i64)]


TRACE_KINDS = ("task_begin", "task_end", "fetch_issue", "fetch_done", "evict_issue", "evict_done",
               "release", "reuse_wait", "input_wait", "step_begin", "step_end", "failure",
               "worker_idle", "user")

_STRUCTS = {"ss_program": Program, "ss_device_config": DeviceConfig, "ss_action": Action,
            "ss_interval": Interval, "ss_sim_result": SimResult, "ss_search_options": SearchOptions,
            "ss_search_summary": SearchSummary, "ss_runtime_config": RuntimeConfig,
            "ss_failure": Failure, "ss_trace_event": TraceEvent, "ss_runtime_stats": RuntimeStats,
            "ss_plan_desc": PlanDesc, "ss_transfer_profile": TransferProfile}

_lock = threading.Lock()
_core: C.CDLL | None = None


class NativeError(RuntimeError):
    def __init__(self, status: int, what: str):
        self.status = status
        super().__init__(f"{what}: {status_string(status)} (status {status})")


def core() -> C.CDLL:
    global _core
    if _core is not None:
        return _core
    with _lock:
        if _core is None:
            if not CORE_PATH.exists():
                from . import build
                build.build_core()
            lib = C.CDLL(str(CORE_PATH))
            _declare(lib)
            _core = lib
            abi_check()
    return _core


def _declare(lib: C.CDLL) -> None:
    lib.ss_status_string.restype = C.c_char_p
    lib.ss_status_string.argtypes = [C.c_int]
    lib.ss_struct_size.restype = C.c_size_t
    lib.ss_struct_size.argtypes = [C.c_char_p]
    lib.ss_monotonic_ns.restype = i64
    lib.ss_simulate.argtypes = [C.POINTER(Program), C.POINTER(DeviceConfig), C.POINTER(Action), i32,
                                C.POINTER(SimResult), P64, P64, P64, P64, C.POINTER(Interval), i32,
                                P32]
    lib.ss_check_schedule.argtypes = [C.POINTER(Program), C.POINTER(Action), i32, P32, P32]
    lib.ss_place_lifetimes.argtypes = [i32, P64, P64, P64, i64, P64, P64]
    lib.ss_recover_layout_reuse.argtypes = [i32, P64, P64, P64, P64, P32, P32, i32]
    lib.ss_plan_search.argtypes = [C.POINTER(Program), C.POINTER(DeviceConfig),
                                   C.POINTER(SearchOptions), C.POINTER(vp)]
    lib.ss_plan_reduce_emit.argtypes = [C.POINTER(Program), C.POINTER(DeviceConfig), C.POINTER(SearchOptions),
                                        i64, i32, i32, i32, P32, P32, i32, P32, C.POINTER(Action), i32, P32]
    lib.ss_search_summary_of.restype = C.POINTER(SearchSummary)
    lib.ss_search_summary_of.argtypes = [vp]
    lib.ss_search_actions.restype = C.POINTER(Action)
    lib.ss_search_actions.argtypes = [vp]
    lib.ss_search_intervals.restype = C.POINTER(Interval)
    lib.ss_search_intervals.argtypes = [vp]
    for n in ("task_start", "task_end", "action_start", "action_end"):
        fn = getattr(lib, f"ss_search_{n}")
        fn.restype = P64
        fn.argtypes = [vp]
    lib.ss_search_trace.restype = C.c_char_p
    lib.ss_search_trace.argtypes = [vp]
    lib.ss_search_result_destroy.argtypes = [vp]
    lib.ss_search_result_destroy.restype = None
    lib.ss_mock_backend_create.restype = vp
    lib.ss_mock_backend_create.argtypes = [f64, i64]
    lib.ss_mock_fail_operation.argtypes = [vp, C.c_int, i64]
    lib.ss_mock_operation_count.restype = i64
    lib.ss_mock_operation_count.argtypes = [vp, C.c_int]
    lib.ss_backend_dlopen.restype = vp
    lib.ss_backend_dlopen.argtypes = [C.c_char_p, C.c_int, C.c_char_p, C.c_size_t]
    lib.ss_runtime_create.argtypes = [vp, C.POINTER(RuntimeConfig), C.POINTER(vp)]
    lib.ss_runtime_close.argtypes = [vp]
    lib.ss_runtime_abandon.argtypes = [vp]
    lib.ss_runtime_abandon.restype = None
    lib.ss_runtime_destroy.argtypes = [vp]
    lib.ss_runtime_destroy.restype = None
    lib.ss_runtime_device_base.restype = vp
    lib.ss_runtime_device_base.argtypes = [vp]
    lib.ss_runtime_spill_base.restype = vp
    lib.ss_runtime_spill_base.argtypes = [vp]
    lib.ss_runtime_failure.argtypes = [vp, C.POINTER(Failure)]
    lib.ss_runtime_latch_failure.argtypes = [vp, C.c_int, C.c_int, C.c_char_p]
    lib.ss_runtime_stats_read.argtypes = [vp, C.POINTER(RuntimeStats)]
    lib.ss_trace_begin.argtypes = [vp]
    lib.ss_trace_end.argtypes = [vp]
    lib.ss_trace_read.argtypes = [vp, C.POINTER(TraceEvent), i32]
    lib.ss_plan_transfer_times.argtypes = [vp, i32, C.POINTER(i64), C.POINTER(i64), i32]
    lib.ss_plan_transfer_times.restype = i32
    lib.ss_plan_admit.argtypes = [vp, C.POINTER(PlanDesc), P32]
    lib.ss_plan_close.argtypes = [vp, i32]
    lib.ss_step_begin.argtypes = [vp, i32, vp]
    lib.ss_before_task.argtypes = [vp, i32, i32, C.POINTER(vp), i32]
    lib.ss_after_task.argtypes = [vp, i32, i32]
    lib.ss_before_task_on.argtypes = [vp, i32, i32, C.POINTER(vp), i32, vp]
    lib.ss_after_task_on.argtypes = [vp, i32, i32, vp]
    lib.ss_step_end.argtypes = [vp, i32]
    lib.ss_step_abandon.argtypes = [vp, i32, C.c_char_p]
    lib.ss_runtime_wait_idle.argtypes = [vp]
    lib.ss_spill_write.argtypes = [vp, i64, vp, i64]
    lib.ss_spill_read.argtypes = [vp, i64, vp, i64]
    lib.ss_calibrate_transfers.argtypes = [vp, i64, i32, C.POINTER(TransferProfile)]
    lib.ss_calibrate_file_transfers.argtypes = [vp, i64, i32, C.POINTER(TransferProfile)]
    lib.ss_file_write.argtypes = [vp, i64, vp, i64]
    lib.ss_file_read.argtypes = [vp, i64, vp, i64]
    lib.ss_runtime_file_info.argtypes = [vp, C.POINTER(i32), P64]
    lib.ss_blake3_new.restype = vp
    lib.ss_blake3_update.argtypes = [vp, vp, C.c_size_t]
    lib.ss_blake3_update.restype = None
    lib.ss_blake3_finalize.argtypes = [vp, C.c_char_p]
    lib.ss_blake3_finalize.restype = None
    lib.ss_blake3_free.argtypes = [vp]
    lib.ss_blake3_free.restype = None


def status_string(status: int) -> str:
    return core().ss_status_string(int(status)).decode()


def abi_check() -> None:
    lib = _core or core()
    for name, struct in _STRUCTS.items():
        native = lib.ss_struct_size(name.encode())
        if native != C.sizeof(struct):
            raise ImportError(f"ABI mismatch for {name}: library {native} B, Python "
                              f"{C.sizeof(struct)} B; rebuild libss_core.so")


def check(rc: int, what: str) -> None:
    if rc != OK:
        raise NativeError(rc, what)


def as_i64(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.int64)


def as_i32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.int32)


def ptr64(a: np.ndarray):
    return a.ctypes.data_as(P64)


def ptr32(a: np.ndarray):
    return a.ctypes.data_as(P32)


class Blake3:
    """Streaming BLAKE3 (32-byte digest) backed by the native core."""

    def __init__(self, data: bytes | None = None):
        self._lib = core()
        self._h = self._lib.ss_blake3_new()
        if data:
            self.update(data)

    def update(self, data) -> "Blake3":
        mv = memoryview(data).cast("B")
        if len(mv):
            if mv.readonly:
                buf = bytes(mv)
                self._lib.ss_blake3_update(self._h, C.cast(C.c_char_p(buf), vp), len(buf))
            else:
                arr = (C.c_char * len(mv)).from_buffer(mv)
                self._lib.ss_blake3_update(self._h, C.addressof(arr), len(mv))
        return self

    def digest(self) -> bytes:
        out = C.create_string_buffer(32)
        self._lib.ss_blake3_finalize(self._h, out)
        return out.raw

    def hexdigest(self) -> str:
        return self.digest().hex()

    def __del__(self):
        try:
            self._lib.ss_blake3_free(self._h)
        except Exception:  # noqa: BLE001 - interpreter shutdown
            pass
