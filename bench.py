"""Headline benchmark: trained tokens/s of a Llama-3-8B-shaped decoder under a fixed
per-worker memory budget (device 24 GiB, pinned-host spill 128 GiB), full-parameter
AdamW with bf16 parameters, gradients and moments (stochastic rounding), packed
variable-length sequences (<= 8192 tokens, 65,536 tokens per worker per step,
alternating loss-mask spans), synthetic data and random-init weights.

    python bench.py --gpus N --steps K --warmup W         # this framework
    python bench.py --impl reference ...                   # the reference, if installable
    python bench.py --impl library ...                     # same planner/runtime on cuBLAS + flash-attn + NCCL

For N > 1 launch one rank per GPU (torch.distributed.run); per-GPU work is fixed
(weak scaling) and the reported value is the whole-job aggregate. One JSON line
is printed by rank 0. The timed region is bracketed by barrier + synchronize,
timed with CUDA events, and the maximum over ranks is reported.
"""
from __future__ import annotations

import os as _os

# task workspaces come from the caching allocator under a hard cap: expandable segments keep
# fragmentation from turning a fitting plan into an allocation failure
_os.environ.setdefault("PYTORCH_CUDA_ALLOC_CONF", "expandable_segments:True")

import argparse
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

# the reference's published regression floors (tokens/s, 1x RTX 5090; it publishes nothing else)
BASELINE_TOKENS_PER_S = {"llama3-8b": 3423.5, "qwen35-9b": 3026.6, "olmoe-7b-a1b": 13907.1}
GIB = 1 << 30


def reference_arm() -> None:
    reason = ("reference not installable offline: its engine needs torch>=2.13,<2.14 and the "
              "external mlops kernel library cloned from GitHub; neither is on this image "
              "(its pip install fails at metadata generation)")
    ref = ROOT / "baseline" / "_ref"
    if ref.exists() and any(ref.iterdir()):
        try:
            sys.path.insert(0, str(ref))
            import shadowspill  # noqa: F401
            import mlops  # noqa: F401
        except Exception as exc:  # noqa: BLE001
            reason = f"reference import fails: {type(exc).__name__}: {str(exc)[:120]}"
    print(json.dumps({"impl": "reference", "unavailable": reason}))


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi during the timed region."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc, self.lines = index, None, []

    def start(self) -> None:
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "200"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self) -> None:
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        sm, mx, reasons = [], [], set()
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0])); mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown",
                                  "sw_power_cap"), parts[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="native", choices=["native", "reference", "library"],
                    help="library = this repository's planner and runtime over cuBLAS, flash-attn, eager "
                         "elementwise ops and NCCL (the comparison arm; never labelled reference)")
    ap.add_argument("--model", default="llama3-8b")
    ap.add_argument("--device-gib", type=float, default=24.0)
    ap.add_argument("--spill-gib", type=float, default=128.0)
    ap.add_argument("--tokens", type=int, default=65536, help="tokens per worker per step")
    ap.add_argument("--microbatch", type=int, default=8192)
    ap.add_argument("--candidates", default="100,75:save_attention,50:save_attention,25:save_attention,0:save_attention,"
                            "mix:8:save_attention_gu",
                    help="comma list of programs the planner sweeps: <recompute share %%>[:<saved variant>] "
                         "or mix:<K>[:<variant>] (attention saved everywhere, K layers keep <variant>, default save)")
    ap.add_argument("--walks", default="auto",
                    help="comma list of breadth | depth | breadth/<G> (G sweeps over the microbatches, sharded "
                         "runs only); auto: breadth, and with several GPUs also breadth/2 and breadth/4")
    ap.add_argument("--collective-overhead-us", type=float, default=0.0,
                    help="planned cost added to every communication-stream task (see qualification/gap_report.py)")
    ap.add_argument("--lora-rank", type=int, default=0, help="train rank-r adapters on a frozen base")
    ap.add_argument("--expert-parallel", action="store_true",
                    help="multi-GPU runs of routed models: split the experts over the ranks")
    ap.add_argument("--report", default="", help="directory for the plan report")
    ap.add_argument("--spill-pool", default="host", choices=["host", "file", "remote"],
                    help="where spilled state lives: pinned memory, a direct-I/O file, or a memory daemon")
    ap.add_argument("--spill-dir", default="/tmp", help="directory of the file spill pool")
    ap.add_argument("--spill-address", default="", help="host:port of the memory daemon")
    ap.add_argument("--collectives", default="auto", choices=["auto", "peer", "dist"],
                    help="peer = own kernels over NVLink peer memory; dist = NCCL baseline arm")
    ap.add_argument("--fused-gather", action="store_true",
                    help="multi-GPU: the forward weight all-gather runs inside the consuming GEMM")
    ap.add_argument("--allocator", default="caching", choices=["caching", "planned"],
                    help="planned = the allocation adapter: task temporaries from a workspace slice of the "
                         "device pool under a checked contract; caching = torch's allocator under a cap")
    ap.add_argument("--axis-chunk-rows", type=int, default=0,
                    help="graph frontend: run the token-local operators of a layer in row chunks of this size")
    ap.add_argument("--delta-head-groups", type=int, default=1,
                    help="gated delta rule: run each call in this many groups of key heads")
    ap.add_argument("--fixed-len", type=int, default=0,
                    help="sequences of exactly this many tokens (= --microbatch: one long sequence per microbatch)")
    ap.add_argument("--frontend", default="graph", choices=["stages", "graph"],
                    help="graph = torch.export -> partition -> AOT graph pairs; stages = hand-written stage classes")
    args = ap.parse_args()
    if args.impl == "reference":
        reference_arm()
        return
    if args.impl == "library":
        # must be set before the op layer is imported
        os.environ["SS_KERNELS"] = "library"
        os.environ["SS_ATTENTION"] = "library"
        args.collectives = "dist"

    import torch
    import torch.distributed as dist

    if args.allocator == "planned":
        # before anything touches CUDA: the adapter cannot replace an allocator already in use
        from shadowspill_b200.runtime import allocator as _allocator
        _allocator.install()

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        # whatever NCCL logs (a version banner with NCCL_DEBUG=VERSION, more with INFO) goes to
        # stderr: stdout carries the one JSON line and nothing else
        # (NCCL honours NCCL_DEBUG_FILE only above the VERSION level, so VERSION becomes WARN)
        if os.environ.get("NCCL_DEBUG", "").upper() == "VERSION":
            os.environ["NCCL_DEBUG"] = "WARN"
        os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")
        dist.init_process_group("nccl", device_id=torch.device(f"cuda:{local}"))

    from shadowspill_b200.training.session import TrainingSession, TrainingSetup
    from shadowspill_b200.data.synthetic import make_batch
    from shadowspill_b200.ops import _lib

    setup = TrainingSetup(model=args.model, device_gib=args.device_gib, spill_gib=args.spill_gib,
                          tokens_per_step=args.tokens, microbatch_tokens=args.microbatch,
                          lr=1e-5, seed=1234, rank=rank, world_size=world, device_index=local,
                          collectives=args.collectives,
                          candidate_selections=tuple(c for c in args.candidates.split(",") if c),
                          walks=(tuple(args.walks.split(",")) if args.walks != "auto" else
                                 ("breadth",) + tuple(f"breadth/{g}" for g in (2, 4)
                                                      if world > 1 and (args.tokens // args.microbatch) % g == 0)),
                          trace_capacity=(1 << 16) if args.report else 0,
                          lora=({"rank": args.lora_rank, "alpha": 2.0 * args.lora_rank,
                                 "targets": ["wq", "wk", "wv", "wo", "w13", "w2"], "routed_experts": True,
                                 "train_base": False} if args.lora_rank else None),
                          expert_parallel=args.expert_parallel, spill_pool=args.spill_pool,
                          frontend=args.frontend, allocator=args.allocator, fused_gather=args.fused_gather,
                          axis_chunk_rows=args.axis_chunk_rows, profile_sequence_tokens=args.fixed_len,
                          delta_head_groups=args.delta_head_groups,
                          collective_overhead_us=args.collective_overhead_us,
                          spill_directory=args.spill_dir if args.spill_pool == "file" else "",
                          spill_address=args.spill_address)
    log = (lambda m: print(f"[bench] {m}", file=sys.stderr, flush=True)) if rank == 0 else None
    session = TrainingSession(setup, log=log)  # build -> profile -> calibrate -> plan -> executor
    if rank == 0:
        for pl, err in zip(session.sweep.plans, session.sweep.errors):
            if pl is None:
                log(f"candidate infeasible: {err.splitlines()[0] if err else '?'}")
            else:
                sm = pl.summary
                log(f"candidate {sm.ordering} [{sm.selection[:60]}]: simulated "
                    f"{sm.duration_seconds * 1e3:.0f} ms, fetch {sm.fetch_bytes / 1e9:.0f} GB, "
                    f"evict {sm.evict_bytes / 1e9:.0f} GB")
    cfg = session.cfg
    n_batches = args.warmup + args.steps
    batches = [make_batch(1000 * rank + i, vocab=cfg.vocab_size, tokens_per_step=args.tokens,
                          microbatch_tokens=args.microbatch, max_len=8192, median=1200.0,
                          fixed_len=args.fixed_len or None, slots=session.slots) for i in range(n_batches)]
    for b in batches:                 # loss weights are 1/N over the GLOBAL batch
        for mb in b:
            mb.weights /= world
    losses = []
    for i in range(args.warmup):
        losses.append(session.step(batches[i]).loss)

    def fence() -> None:
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(local)
    fence()
    sampler.start()
    launches0 = _lib.launch_count
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    wall0 = time.perf_counter()
    start.record()
    h2d = d2h = 0
    for i in range(args.steps):
        res = session.step(batches[args.warmup + i])   # stages inputs from host, returns host loss
        losses.append(res.loss)
        h2d, d2h = res.h2d_bytes, res.d2h_bytes
    end.record()
    fence()
    wall = time.perf_counter() - wall0
    clocks = sampler.stop()
    dev_s = start.elapsed_time(end) * 1e-3
    launches = _lib.launch_count - launches0
    times = torch.tensor([dev_s, wall], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    dev_s, wall = float(times[0]), float(times[1])
    total_tokens = args.tokens * world * args.steps
    value = total_tokens / dev_s
    if rank == 0:
        plan = session.plan.summary
        out = {
            "metric": "trained tokens/s at fixed device/spill GiB budget",
            "value": round(value, 1), "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": round(dev_s / args.steps * 1e3, 2),
            "higher_is_better": True, "scaling": "weak",
            "vs_baseline": (round(value / BASELINE_TOKENS_PER_S[args.model], 3)
                            if args.model in BASELINE_TOKENS_PER_S else None), "dtype": "bf16",
            "data": ((f"synthetic sequences of exactly {args.fixed_len} tokens, " if args.fixed_len else
                      "synthetic packed varlen (log-normal lengths, median 1200, <=8192), ")
                     + "random-init weights"),
            "config": {"model": args.model, "global_batch": args.tokens * world,
                       "seq_len": args.fixed_len or 8192, "tokens_per_worker_step": args.tokens,
                       "microbatch_tokens": args.microbatch,
                       "parallelism": f"dp{world}" if world > 1 else "single",
                       "memory": {"device_gib": args.device_gib, "spill_gib": args.spill_gib,
                                  "spill_pool": args.spill_pool},
                       "optimizer": "adamw bf16 state, stochastic rounding",
                       "l2": "inputs per step (16+ GB of weights streamed from host) exceed L2",
                       "plan": {"ordering": plan.ordering, "selection": plan.selection,
                                "fetch_rule": plan.fetch_rule, "strategy": plan.strategy,
                                "simulated_ms": round(plan.duration_seconds * 1e3, 1),
                                "device_pool_gib": round(session.plan.device_bytes / GIB, 2),
                                "workspace_gib": round(plan.workspace_bytes / GIB, 2),
                                "spill_gib": round(session.plan.spill_bytes / GIB, 2)},
                       "attention": os.environ.get("SS_ATTENTION", "native"),
                       "frontend": session.desc.frontend, "allocator": args.allocator,
                       "axis_chunk_rows": args.axis_chunk_rows,
                       "collectives": (session.executor.collectives.name
                                       if session.executor.collectives else "none")},
            "e2e": {"value": round(total_tokens / wall, 1), "unit": "tokens/s",
                    "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h),
                    "api": "TrainingSession.step(host numpy batch) -> host loss"},
            "gpu_launches": int(launches), "impl": args.impl, "clocks": clocks,
            "loss_first": round(losses[0], 4), "loss_last": round(losses[-1], 4),
            "peak_device_gib": round(session.peak_device_bytes() / GIB, 2),
        }
        print(json.dumps(out), flush=True)
    if args.report:
        # one more (untimed) step with per-task clocks and the runtime trace on
        extra = make_batch(1000 * rank + n_batches, vocab=cfg.vocab_size, tokens_per_step=args.tokens,
                           microbatch_tokens=args.microbatch, max_len=8192, median=1200.0,
                           fixed_len=args.fixed_len or None, slots=session.slots)
        for mb in extra:
            mb.weights /= world
        _, diag = session.traced_step(extra, args.report if rank == 0 else None)
        if rank == 0:
            session.write_plan_report(args.report)
            log(f"traced step: real {diag.makespan_s * 1e3:.0f} ms vs simulated "
                f"{diag.simulated_makespan_s * 1e3:.0f} ms; tasks real {diag.task_seconds_real * 1e3:.0f} "
                f"/ profiled {diag.task_seconds_profiled * 1e3:.0f} ms; idle {diag.idle_seconds_real * 1e3:.0f} ms "
                f"(inputs {diag.input_readiness_wait_seconds * 1e3:.0f}, reuse "
                f"{diag.allocation_reuse_wait_seconds * 1e3:.0f}, frontend "
                f"{diag.frontend_overhead_seconds * 1e3:.0f})")
    session.close()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
