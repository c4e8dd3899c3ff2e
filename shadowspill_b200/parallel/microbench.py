"""Timing of the peer-memory collectives against the NVLink roofline and the library arm.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        -m shadowspill_b200.parallel.microbench [--mib 416]

Per rank, for a tensor of the given size (default: one Llama-3-8B layer, 416 MiB of bf16):
  all-gather        own pull kernel (`ss_peer_allgather`) vs `dist.all_gather_into_tensor`
  reduce-scatter+AdamW  (with SS_NVLS=1 and a multicast-capable fabric the gradient sum is one
                    multimem.ld_reduce inside the NVSwitch)  own fused kernel (`ss_rs_adamw`: peers' gradient slices are read over
                    NVLink, summed and applied to this rank's shard of weights and moments
                    in one pass) vs `dist.reduce_scatter_tensor` followed by the local AdamW kernel
CUDA-event times, max over ranks, 3 warm-ups; roofline = bytes that must cross NVLink per rank
/ 770 GB/s (measured peer-copy rate per direction) or, for the fused update, the slower of
that and the shard's HBM traffic / measured copy bandwidth.

``--case experts`` times one forward + backward of an expert-parallel routed layer (pull dispatch,
grouped GEMMs, scatter-epilogue combine) beside the same per-rank expert work with nothing crossing
NVLink and beside four library all-to-all exchanges of the row set, which is what a dispatch /
combine built on a collective library moves for one forward + backward.
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

from ..ops import functional as F
from . import collectives as pc

LINK_GBS = 770.0


def _timed(fn, dev, iters=10, warmup=3):
    for _ in range(warmup):
        fn()
    dist.barrier()
    torch.cuda.synchronize(dev)
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(iters):
        fn()
    b.record()
    b.synchronize()
    t = torch.tensor([a.elapsed_time(b) / iters], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t)


def experts_case(a, rank: int, world: int, dev) -> dict:
    from ..ops import moe as moe_ops
    from .expert_parallel import ExpertParallelGroup, experts
    T, D, Fe, E, k = a.tokens, a.d_model, a.d_expert, a.experts, a.top_k
    group = ExpertParallelGroup(T, k, D, E)
    local_experts = E // world
    w13 = (torch.randn(local_experts, 2 * Fe, D, device=dev) * 0.02).bfloat16()
    w2 = (torch.randn(local_experts, D, Fe, device=dev) * 0.02).bfloat16()
    h = torch.randn(T, D, device=dev).bfloat16().requires_grad_(True)
    logits = torch.randn(T, E, device=dev).requires_grad_(True)
    logits_local = torch.randn(T, local_experts, device=dev).requires_grad_(True)
    dout = torch.randn(T, D, device=dev).bfloat16()
    rows_out = torch.empty(T * k, D, device=dev, dtype=torch.bfloat16)
    rows_in = torch.empty_like(rows_out)

    def parallel():
        experts(h, logits, w13, w2, group, True, None).backward(dout)

    def all_local():        # the same expert work per rank on rows that never leave the GPU
        moe_ops.experts(h, logits_local, w13, w2, k, True, None).backward(dout)

    def library_exchange():
        for _ in range(4):
            dist.all_to_all_single(rows_in, rows_out)
    ms = _timed(parallel, dev, iters=5, warmup=2)
    ms_local = _timed(all_local, dev, iters=5, warmup=2)
    ms_a2a = _timed(library_exchange, dev, iters=5, warmup=2)
    flops = 2 * 2 * T * k * (2 * Fe * D + D * Fe)             # per rank: forward + data gradients
    return {"case": "experts_fwd_bwd", "ranks": world, "tokens": T, "d_model": D, "d_expert": Fe,
            "experts": E, "top_k": k, "ms": round(ms, 3), "all_local_ms": round(ms_local, 3),
            "nccl_all_to_all_x4_ms": round(ms_a2a, 3),
            "gemm_floor_ms_at_1.4_pflops": round(flops / 1.4e15 * 1e3, 3)}


def main(argv=None) -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--case", default="collectives", choices=["collectives", "experts"])
    ap.add_argument("--mib", type=float, default=416.0)
    ap.add_argument("--hbm-gbs", type=float, default=6550.0)
    ap.add_argument("--tokens", type=int, default=8192)
    ap.add_argument("--d-model", type=int, default=2048)
    ap.add_argument("--d-expert", type=int, default=1024)
    ap.add_argument("--experts", type=int, default=64)
    ap.add_argument("--top-k", type=int, default=8)
    a = ap.parse_args(argv)
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    if a.case == "experts":
        row = experts_case(a, rank, world, dev)
        if rank == 0:
            print(json.dumps(row), flush=True)
        dist.barrier()
        dist.destroy_process_group()
        return
    n = int(a.mib * (1 << 20)) // 2 // (8 * world) * (8 * world)          # bf16 elements, whole shards
    per = n // world
    pool = pc.allocate_symmetric_pool(2 * n * 2 + (1 << 20), dev)
    peer = pc.PeerCollectives(pool)
    full = pool[:n * 2].view(torch.bfloat16)
    grad = pool[n * 2:n * 4].view(torch.bfloat16)
    full.normal_(0, 0.02)
    grad.normal_(0, 1e-3)
    shard = full[rank * per:(rank + 1) * per]                             # this rank's slice, in the pool
    p = torch.randn(per, device=dev).bfloat16()
    m = torch.zeros(per, device=dev, dtype=torch.bfloat16)
    v = torch.zeros(per, device=dev, dtype=torch.bfloat16)
    out = torch.empty(n, device=dev, dtype=torch.bfloat16)
    hyper = dict(lr=1e-4, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.0, step=1, grad_scale=1.0,
                 seed=1, stochastic_param=True, stochastic_state=True)

    def ag_own():
        peer.barrier_begin()
        peer.all_gather(shard, out)
        peer.barrier_end()

    def ag_lib():
        dist.all_gather_into_tensor(out, shard)

    def rs_own():
        peer.barrier_begin()
        peer.reduce_scatter_adamw(grad, p, m, v, offset=0, **hyper)
        peer.barrier_end()

    gshard = torch.empty(per, device=dev, dtype=torch.bfloat16)

    def rs_lib():
        dist.reduce_scatter_tensor(gshard, grad)
        F.adamw_(p, gshard, m, v, lr=1e-4, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.0, step=1,
                 grad_scale=1.0, seed=1, offset=0, stochastic_param=True, stochastic_state=True)

    rows = []
    link_bytes = (world - 1) * per * 2                                    # what each rank must receive
    rs_name = "rs_adamw_own_nvls" if peer.mc_base else "rs_adamw_own"     # SS_NVLS=1: in-switch sum
    for name, fn, hbm_bytes in (("allgather_own", ag_own, n * 2), ("allgather_nccl", ag_lib, n * 2),
                                (rs_name, rs_own, per * 2 * (world + 6)),
                                ("rs_nccl_then_adamw", rs_lib, per * 2 * (world + 8))):
        ms = _timed(fn, dev)
        floor_ms = max(link_bytes / (LINK_GBS * 1e9), hbm_bytes / (a.hbm_gbs * 1e9)) * 1e3
        rows.append({"case": name, "ranks": world, "mib": round(n * 2 / (1 << 20), 1), "ms": round(ms, 4),
                     "link_gbs": round(link_bytes / ms / 1e6, 1), "roofline_ms": round(floor_ms, 4),
                     "frac_of_roofline": round(floor_ms / ms, 3)})
    if rank == 0:
        for r in rows:
            print(json.dumps(r), flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
