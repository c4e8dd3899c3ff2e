"""Measurements behind ``CommunicationInfo`` and the planner's correction factors.

``measure_communication``  host-link rates of one worker through the runtime's own
                           lanes (each direction alone and both together) and, in a
                           multi-rank job, the cost of the all-gather and
                           reduce-scatter sizes a program uses.
``measure_overlap``        how much slower compute runs while both lanes stream and
                           once the chip has settled at its sustained clocks, as one
                           factor to scale burst-measured task profiles with.
``measure_pool_memory``    how much device and pinned host memory can actually be
                           had, for ``Memory(device_gib=0, spill_gib=0)`` = automatic.

Reference: packages/engine/src/shadowspill/communication/measure.py
(``measure_communication``), overlap.py (``measure_overlap``) and
memory_measurement.py (``measure_pool_memory``).
"""
from __future__ import annotations

import time
from dataclasses import dataclass

import torch

from ..runtime.core import Runtime
from .info import CommunicationInfo


def measure_communication(device_index: int = 0, probe_bytes: int = 256 << 20, repeats: int = 3,
                          backend: str = "cuda", world_size: int = 1,
                          collective_sizes: dict[str, list[int]] | None = None) -> CommunicationInfo:
    """``collective_sizes`` maps ``all_gather`` / ``reduce_scatter`` / ``all_reduce`` to the
    full byte counts to time on the default process group; each is run ``repeats`` times
    and the median kept under ``"op:ranks:bytes"``. Every rank must call this with the
    same arguments."""
    with Runtime(2 * probe_bytes, 2 * probe_bytes, backend, device_index) as rt:
        r = rt.calibrate(probe_bytes, repeats)
    info = CommunicationInfo(r.fetch_solo_bps, r.fetch_concurrent_bps, r.evict_solo_bps,
                             r.evict_concurrent_bps, r.fetch_latency_ns, r.evict_latency_ns,
                             world_size=world_size, source="calibrated")
    if world_size > 1 and collective_sizes:
        import torch.distributed as dist
        dev = torch.device("cuda", device_index) if backend == "cuda" else torch.device("cpu")
        info.collectives.update(_time_collectives(dev, world_size, collective_sizes, repeats))
        info.backend = {"collectives": dist.get_backend()}
    return info


def _time_collectives(device: torch.device, world: int, sizes: dict[str, list[int]],
                      repeats: int) -> dict[str, float]:
    """Times ``torch.distributed`` all-gather / reduce-scatter of the given full byte
    counts on the default process group; the maximum over ranks is kept."""
    import torch.distributed as dist
    out: dict[str, float] = {}
    cuda = device.type == "cuda"
    for op, byte_counts in sizes.items():
        for nbytes in sorted(set(byte_counts)):
            elems = -(-nbytes // 4 // world)
            full = torch.zeros(elems * world, dtype=torch.float32, device=device)
            part = torch.zeros(elems, dtype=torch.float32, device=device)
            samples = []
            for _ in range(repeats + 1):
                dist.barrier()
                if cuda:
                    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    a.record()
                else:
                    t0 = time.perf_counter()
                if op == "all_gather":
                    dist.all_gather_into_tensor(full, part)
                elif op == "reduce_scatter":
                    dist.reduce_scatter_tensor(part, full)
                else:
                    dist.all_reduce(full)
                if cuda:
                    b.record()
                    b.synchronize()
                    samples.append(a.elapsed_time(b) * 1e-3)
                else:
                    samples.append(time.perf_counter() - t0)
            samples = sorted(samples[1:])
            t = torch.tensor([samples[len(samples) // 2]], dtype=torch.float64, device=device)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            out[f"{op}:{world}:{nbytes}"] = float(t.item())
    return out


@dataclass
class OverlapProfile:
    burst_tflops: float          # first burst of a cold GEMM loop
    sustained_tflops: float      # same loop after `settle_seconds`
    streaming_tflops: float      # sustained, with both host lanes busy
    fetch_bps_under_compute: float
    evict_bps_under_compute: float

    @property
    def duration_scale(self) -> float:
        """Factor that turns a burst-measured task time into its time inside a long,
        streaming step."""
        return self.burst_tflops / self.streaming_tflops if self.streaming_tflops > 0 else 1.0


def measure_overlap(device_index: int = 0, settle_seconds: float = 1.5, window_seconds: float = 0.4,
                    copy_bytes: int = 256 << 20, m: int = 8192, n: int = 4096,
                    k: int = 4096) -> OverlapProfile:
    """Runs the framework's own GEMM in a loop: a short cold burst, then a settled
    window, then a settled window with the runtime's two lanes copying
    continuously. Times are CUDA events on the compute stream."""
    from ..ops import functional as F
    dev = torch.device("cuda", device_index)
    a = torch.randn(m, k, device=dev, dtype=torch.bfloat16)
    w = torch.randn(n, k, device=dev, dtype=torch.bfloat16)
    c = torch.empty(m, n, device=dev, dtype=torch.bfloat16)
    flops = 2.0 * m * n * k

    def window(seconds: float) -> float:
        F.linear_fwd(a, w, out=c)
        torch.cuda.synchronize(dev)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        iters = 0
        e0.record()
        t0 = time.perf_counter()
        while time.perf_counter() - t0 < seconds:
            for _ in range(20):
                F.linear_fwd(a, w, out=c)
            iters += 20
            torch.cuda.current_stream(dev).synchronize()
        e1.record()
        e1.synchronize()
        return flops * iters / (e0.elapsed_time(e1) * 1e-3) * 1e-12

    with torch.cuda.device(dev):
        burst = window(0.05)
        window(settle_seconds)
        sustained = window(window_seconds)
        with Runtime(2 * copy_bytes, 2 * copy_bytes, "cuda", device_index) as rt:
            stop = False
            rates = {}

            import threading

            def pump():
                # back-to-back two-way calibration copies keep both lanes full
                while not stop:
                    r = rt.calibrate(copy_bytes, 1)
                    rates["fetch"], rates["evict"] = r.fetch_concurrent_bps, r.evict_concurrent_bps
            th = threading.Thread(target=pump, daemon=True)
            th.start()
            time.sleep(0.05)
            streaming = window(window_seconds)
            stop = True
            th.join()
    return OverlapProfile(burst, sustained, streaming, rates.get("fetch", 0.0), rates.get("evict", 0.0))


@dataclass
class PoolMemoryProfile:
    device_total_bytes: int
    device_free_bytes: int
    device_pool_bytes: int       # what an automatic budget would take
    host_total_bytes: int
    host_available_bytes: int
    spill_pool_bytes: int


def measure_pool_memory(device_index: int = 0, fraction: float = 0.9,
                        ranks_on_host: int = 1) -> PoolMemoryProfile:
    """Automatic budgets: ``fraction`` of the free device memory, and the same fraction
    of this host's available memory divided by the ranks sharing it (the reference's
    ``Memory(0, 0)`` = automatic 90 %, packages/client/src/shadowspill_client/config/batch.py:42)."""
    import psutil
    if torch.cuda.is_available():
        free, total = torch.cuda.mem_get_info(device_index)
    else:
        free = total = 0
    vm = psutil.virtual_memory()
    return PoolMemoryProfile(total, free, int(free * fraction), vm.total, vm.available,
                             int(vm.available * fraction / max(1, ranks_on_host)))
