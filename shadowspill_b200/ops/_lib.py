"""ctypes binding of ``libss_kernels.so`` (the sm_100a kernel library).

The kernels are exported as plain C launchers that take raw device pointers and
a stream handle, so this module needs no compiled Python extension. On a machine
with a GPU a missing library is an error, never a silent fallback.
"""
from __future__ import annotations

import ctypes
import threading
from pathlib import Path

import torch

_LIB_PATH = Path(__file__).resolve().parent / "libss_kernels.so"
_lock = threading.Lock()
_lib: ctypes.CDLL | None = None

c_int, c_ll, c_ull, c_f, c_p = (ctypes.c_int, ctypes.c_longlong, ctypes.c_ulonglong,
                                ctypes.c_float, ctypes.c_void_p)

_SIGNATURES = {
    "ss_gemm_bf16": [c_p, c_p, c_p, c_int, c_int, c_int, c_ll, c_ll, c_ll, c_int, c_int, c_int,
                     c_int, c_f, c_int, c_int, c_p, c_p],
    "ss_gemm2_bf16": [c_p, c_p, c_p, c_int, c_int, c_int, c_ll, c_ll, c_ll, c_int, c_int, c_int,
                      c_int, c_f, c_int, c_p, c_p],
    "ss_gemm2_gather_bf16": [c_p, c_p, c_p, c_int, c_int, c_int, c_ll, c_ll, c_int, c_int, c_f, c_p, c_ll,
                             c_int, c_int, c_p, c_ull, c_int, c_p, c_p],
    "ss_rmsnorm_fwd": [c_p, c_p, c_p, c_p, c_p, c_int, c_int, c_f, c_int, c_p],
    "ss_rmsnorm_bwd": [c_p, c_p, c_p, c_p, c_p, c_p, c_int, c_int, c_int, c_int, c_p],
    "ss_rope": [c_p, c_p, c_int, c_ll, c_int, c_int, c_int, c_int, c_f, c_int, c_p],
    "ss_swiglu_fwd": [c_p, c_p, c_int, c_int, c_p],
    "ss_swiglu_bwd": [c_p, c_p, c_p, c_int, c_int, c_p],
    "ss_embedding_fwd": [c_p, c_p, c_p, c_int, c_int, c_int, c_p],
    "ss_embedding_bwd": [c_p, c_p, c_p, c_int, c_int, c_int, c_int, c_p],
    "ss_cross_entropy": [c_p, c_p, c_p, c_p, c_p, c_int, c_int, c_ll, c_f, c_int, c_p],
    "ss_token_objective": [c_p, c_p, c_p, c_p, c_p, c_int, c_int, c_ll, c_f, c_int, c_int, c_p, c_p,
                           c_f, c_p, c_f, c_p],
    "ss_adamw_sr": [c_p, c_p, c_p, c_p, c_ll, c_int, c_f, c_f, c_f, c_f, c_f, c_int, c_f, c_ull,
                    c_ull, c_int, c_int, c_p],
    "ss_adamw_f32": [c_p, c_p, c_p, c_p, c_ll, c_f, c_f, c_f, c_f, c_f, c_int, c_f, c_p],
    "ss_sumsq": [c_p, c_ll, c_p, c_p, c_int, c_p],
    "ss_cast_f32_bf16": [c_p, c_p, c_ll, c_f, c_p],
}


class KernelLibraryMissing(RuntimeError):
    pass


def available() -> bool:
    return _LIB_PATH.exists()


def lib() -> ctypes.CDLL:
    """Load (once) and return the kernel library."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is None:
            if not _LIB_PATH.exists():
                raise KernelLibraryMissing(
                    f"{_LIB_PATH} is not built; run `python -m shadowspill_b200.build`")
            handle = ctypes.CDLL(str(_LIB_PATH))
            for name, argtypes in _SIGNATURES.items():
                if not hasattr(handle, name):
                    continue   # optional kernels are probed by their users
                fn = getattr(handle, name)
                fn.argtypes = argtypes
                fn.restype = c_int
            _lib = handle
    return _lib


def register(name: str, argtypes: list) -> None:
    """Declare the signature of another exported launcher (used by sibling modules)."""
    _SIGNATURES[name] = argtypes
    if _lib is not None and hasattr(_lib, name):
        fn = getattr(_lib, name)
        fn.argtypes = argtypes
        fn.restype = c_int


def stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


_status_words: dict[int, torch.Tensor] = {}

STATUS_NAMES = {
    0: "ok", 1: "timeout waiting for a TMA stage", 2: "timeout waiting for a free stage",
    3: "timeout waiting for an accumulator", 4: "timeout waiting for a drained accumulator",
    5: "timeout waiting for a peer flag", 6: "bad argument",
}


def status_word(device: torch.device | int | None = None) -> torch.Tensor:
    """Per-device int32 word that kernels write when a bounded wait gives up."""
    index = torch.cuda.current_device() if device is None else torch.device(device).index
    if index is None:
        index = torch.cuda.current_device()
    word = _status_words.get(index)
    if word is None:
        word = torch.zeros(1, dtype=torch.int32, device=f"cuda:{index}")
        _status_words[index] = word
    return word


def check_status(device: torch.device | int | None = None) -> None:
    """Synchronising read of the status word; raises if any kernel gave up."""
    word = status_word(device)
    code = int(word.item())
    if code != 0:
        word.zero_()
        raise RuntimeError(f"kernel reported: {STATUS_NAMES.get(code, code)} (code {code})")


# kernels launched by one successful call of each launcher (attention backward:
# delta + dQ + dKV; sum of squares: partials + final)
_KERNELS_PER_CALL = {"ss_attn_bwd": 3, "ss_attn_bwd_g": 3, "ss_sumsq": 2}
launch_count = 0
_by_entry: dict[str, int] = {}


def check(rc: int, what: str) -> None:
    """Raises on a failed launcher; counts the kernels a successful one enqueued."""
    global launch_count
    if rc != 0:
        raise RuntimeError(f"{what} failed with code {rc}")
    n = _KERNELS_PER_CALL.get(what, 1)
    launch_count += n
    _by_entry[what] = _by_entry.get(what, 0) + n


def launch_counts() -> dict[str, int]:
    """Kernels enqueued so far, by launcher entry point."""
    return dict(_by_entry)
