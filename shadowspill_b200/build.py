"""In-tree native build: CUDA kernels for sm_100a and the C++ core libraries.

Everything is compiled with explicit ``nvcc`` / ``g++`` commands into shared
objects that sit next to their sources, so a source snapshot that carries the
built ``.so`` files runs without a JIT cache. ``python -m shadowspill_b200.build``
rebuilds what is stale.

The reference builds its C11 core with CMake and no ``nvcc`` at all
(packages/engine/csrc/backends/CMakeLists.txt:74-119); this build has CUDA
sources, so the kernel library is compiled for ``sm_100a`` only.
"""
from __future__ import annotations

import concurrent.futures
import os
import shutil
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent
KERNEL_DIR = ROOT / "ops" / "csrc"
KERNEL_LIB = ROOT / "ops" / "libss_kernels.so"
CORE_DIR = ROOT / "csrc"
CORE_LIB = CORE_DIR / "libss_core.so"
CUDA_BACKEND_LIB = CORE_DIR / "libss_backend_cuda.so"
ALLOCATOR_LIB = CORE_DIR / "libss_allocator.so"           # torch pluggable allocator (links cudart)
ALLOCATOR_HOST_LIB = CORE_DIR / "libss_allocator_host.so"  # the same logic over host memory, for tests
MEMORY_DAEMON = CORE_DIR / "ss_memory_daemon"     # far side of the remote spill pool

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-Wall",
]
CXX_FLAGS = ["-O2", "-g", "-std=c++17", "-fPIC", "-Wall", "-Wextra", "-pthread"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found; set NVCC or install the CUDA toolkit")


def _stale(target: Path, sources: list[Path]) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(s.stat().st_mtime > t for s in sources)


def _run(cmd: list[str], verbose: bool) -> None:
    if verbose:
        print(" ".join(cmd), flush=True)
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"command failed: {' '.join(cmd)}\n{proc.stdout}\n{proc.stderr}")
    if verbose and proc.stderr.strip():
        print(proc.stderr, file=sys.stderr)


def build_kernels(force: bool = False, verbose: bool = False, ptxas_info: bool = False) -> Path:
    """Compile every ``ops/csrc/*.cu`` for sm_100a and link ``libss_kernels.so``."""
    sources = sorted(KERNEL_DIR.glob("*.cu"))
    headers = sorted(KERNEL_DIR.glob("*.cuh")) + sorted(KERNEL_DIR.glob("*.h"))
    if not sources:
        raise RuntimeError(f"no CUDA sources under {KERNEL_DIR}")
    if not force and not _stale(KERNEL_LIB, sources + headers):
        return KERNEL_LIB
    nvcc = _nvcc()
    objdir = KERNEL_DIR / "build"
    objdir.mkdir(exist_ok=True)
    extra = ["-Xptxas", "-v"] if ptxas_info else []

    def compile_one(src: Path) -> Path:
        obj = objdir / (src.stem + ".o")
        if force or _stale(obj, [src] + headers):
            _run([nvcc, *NVCC_FLAGS, *extra, "-c", str(src), "-o", str(obj)], verbose)
        return obj

    with concurrent.futures.ThreadPoolExecutor(max_workers=os.cpu_count() or 4) as pool:
        objs = list(pool.map(compile_one, sources))
    tmp = KERNEL_LIB.with_suffix(".so.tmp")
    _run([nvcc, "-shared", "-o", str(tmp), *map(str, objs), "-lcudart"], verbose)
    os.replace(tmp, KERNEL_LIB)
    return KERNEL_LIB


def _cuda_home() -> Path | None:
    for cand in (os.environ.get("CUDA_HOME"), "/usr/local/cuda"):
        if cand and (Path(cand) / "include" / "cuda_runtime.h").exists():
            return Path(cand)
    return None


def build_core(force: bool = False, verbose: bool = False) -> Path:
    """Compile the C++17 core (simulator, planner, runtime, mock backend)."""
    sources = sorted(p for p in CORE_DIR.rglob("*.cpp") if "backend_cuda" not in p.name
                     and "canary" not in p.name and p.parent.name not in ("daemon", "adapter"))
    headers = sorted(CORE_DIR.rglob("*.h")) + sorted(CORE_DIR.rglob("*.hpp"))
    if not sources:
        return CORE_LIB
    if force or _stale(CORE_LIB, sources + headers):
        tmp = CORE_LIB.with_suffix(".so.tmp")
        _run(["g++", *CXX_FLAGS, "-shared", "-I", str(CORE_DIR / "include"), "-o", str(tmp),
              *map(str, sources), "-ldl"], verbose)
        os.replace(tmp, CORE_LIB)
    daemon_src = sorted((CORE_DIR / "daemon").glob("*.cpp"))
    if daemon_src and (force or _stale(MEMORY_DAEMON, daemon_src)):
        tmp = MEMORY_DAEMON.with_suffix(".tmp")
        _run(["g++", "-O2", "-g", "-std=c++17", "-Wall", "-Wextra", "-pthread", "-o", str(tmp),
              *map(str, daemon_src)], verbose)
        os.replace(tmp, MEMORY_DAEMON)
    cuda_src = sorted(CORE_DIR.rglob("backend_cuda*.cpp"))
    cuda = _cuda_home()
    if cuda_src and cuda is not None and (force or _stale(CUDA_BACKEND_LIB, cuda_src + headers)):
        tmp = CUDA_BACKEND_LIB.with_suffix(".so.tmp")
        _run(["g++", *CXX_FLAGS, "-shared", "-I", str(CORE_DIR / "include"),
              "-I", str(cuda / "include"), "-o", str(tmp), *map(str, cuda_src),
              "-L", str(cuda / "lib64"), "-lcudart", "-ldl"], verbose)
        os.replace(tmp, CUDA_BACKEND_LIB)
    alloc_src = sorted((CORE_DIR / "adapter").glob("allocator*.cpp"))
    if alloc_src and (force or _stale(ALLOCATOR_HOST_LIB, alloc_src)):
        tmp = ALLOCATOR_HOST_LIB.with_suffix(".so.tmp")
        _run(["g++", *CXX_FLAGS, "-shared", "-o", str(tmp), *map(str, alloc_src)], verbose)
        os.replace(tmp, ALLOCATOR_HOST_LIB)
    if alloc_src and cuda is not None and (force or _stale(ALLOCATOR_LIB, alloc_src)):
        tmp = ALLOCATOR_LIB.with_suffix(".so.tmp")
        _run(["g++", *CXX_FLAGS, "-shared", "-DSS_ALLOCATOR_WITH_CUDA", "-I", str(cuda / "include"),
              "-o", str(tmp), *map(str, alloc_src), "-L", str(cuda / "lib64"), "-lcudart"], verbose)
        os.replace(tmp, ALLOCATOR_LIB)
    return CORE_LIB


def build_all(force: bool = False, verbose: bool = False) -> None:
    build_kernels(force=force, verbose=verbose)
    build_core(force=force, verbose=verbose)


def verify() -> dict:
    """What a fresh checkout should check after building (``python -m shadowspill_b200.build
    --verify``): the native core loads and its structs have the sizes the Python binding expects,
    the mock backend runs a plan, the kernel library exports its entry points, the memory daemon
    and the allocation adapter exist, and (on a machine with a GPU) the CUDA backend opens.
    Reference: scripts/setup.sh of the reference (build, then verify backend, ABI and adapter)."""
    import ctypes
    report: dict = {}
    from . import native
    lib = native.core()
    native.abi_check()                                        # raises ImportError on a struct-size mismatch
    report["core"] = {"path": str(CORE_LIB), "abi": int(lib.ss_abi_version())}
    kernels = ctypes.CDLL(str(KERNEL_LIB))
    wanted = ("ss_gemm_bf16", "ss_gemm2_bf16", "ss_attn_fwd", "ss_attn_bwd", "ss_rs_adamw", "ss_rs_accumulate",
              "ss_peer_allgather", "ss_adamw_sr")
    missing = [name for name in wanted if not hasattr(kernels, name)]
    report["kernels"] = {"path": str(KERNEL_LIB), "missing": missing}
    root = Path(CORE_LIB).parent
    report["files"] = {name: (root / name).exists() for name in
                       ("libss_backend_cuda.so", "libss_allocator.so", "ss_memory_daemon")}
    import torch
    report["gpu"] = torch.cuda.is_available()
    report["ok"] = not missing and all(report["files"].values())
    return report


def main(argv=None) -> int:
    argv = sys.argv[1:] if argv is None else list(argv)
    build_all(force="--force" in argv, verbose="-v" in argv or "--verbose" in argv)
    print("built:", KERNEL_LIB, CORE_LIB)
    if "--verify" in argv:
        import json
        outcome = verify()
        print(json.dumps(outcome, indent=1))
        return 0 if outcome["ok"] else 1
    return 0


if __name__ == "__main__":
    sys.exit(main())
