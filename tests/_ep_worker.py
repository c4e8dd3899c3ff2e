"""Child process of the expert-parallel test: one rank of a 2+-GPU job. Every rank
holds the full expert banks (same seed) so that the single-GPU routed-expert op is
the oracle for its own tokens; the expert-parallel op sees only its slice."""
import os
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))

import torch
import torch.distributed as dist

from shadowspill_b200.models.autograd_ops import GradSink
from shadowspill_b200.ops import moe as moe_ops
from shadowspill_b200.parallel.expert_parallel import ExpertParallelGroup, experts


def rel(a, b):
    a, b = a.detach().float(), b.detach().float()
    return float((a - b).norm() / b.norm().clamp_min(1e-6))


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", device_id=dev)
    T, D, Fe, E, k = 512, 256, 128, 8, 2
    g = torch.Generator(device=dev).manual_seed(7)                 # same banks on every rank
    w13 = (torch.randn(E, 2 * Fe, D, device=dev, generator=g) * 0.05).bfloat16()
    w2 = (torch.randn(E, D, Fe, device=dev, generator=g) * 0.05).bfloat16()
    router = torch.randn(E, D, device=dev, generator=g) * 0.1
    gr = torch.Generator(device=dev).manual_seed(100 + rank)       # different tokens per rank
    ep = ExpertParallelGroup(T, k, D, E)
    el, lo = E // world, rank * (E // world)
    for step, renorm in enumerate((True, False)):
        h = torch.randn(T, D, device=dev, generator=gr).bfloat16()
        dout = torch.randn(T, D, device=dev, generator=gr).bfloat16()
        # ---- oracle: every expert local
        h0 = h.clone().requires_grad_(True)
        lg0 = (h.float() @ router.t()).requires_grad_(True)
        G0 = {"w13": torch.zeros(E, 2 * Fe, D, device=dev), "w2": torch.zeros(E, D, Fe, device=dev)}
        y0 = moe_ops.experts(h0, lg0, w13, w2, k, renorm, GradSink(G0, True))
        y0.backward(dout)
        for t in G0.values():                                      # sum over every rank's tokens
            dist.all_reduce(t)
        # ---- expert parallel: this rank's slice of the banks
        h1 = h.clone().requires_grad_(True)
        lg1 = (h.float() @ router.t()).requires_grad_(True)
        G1 = {"w13": torch.zeros(el, 2 * Fe, D, device=dev), "w2": torch.zeros(el, D, Fe, device=dev)}
        y1 = experts(h1, lg1, w13[lo:lo + el].contiguous(), w2[lo:lo + el].contiguous(), ep, renorm,
                     GradSink(G1, True))
        y1.backward(dout)
        torch.cuda.synchronize()
        errs = {"y": rel(y1, y0), "dh": rel(h1.grad, h0.grad), "dlogits": rel(lg1.grad, lg0.grad),
                "dw13": rel(G1["w13"], G0["w13"][lo:lo + el]), "dw2": rel(G1["w2"], G0["w2"][lo:lo + el])}
        bad = {n: e for n, e in errs.items() if not e < 2e-2}
        assert not bad, (rank, step, errs)
    # ---- timing of forward+backward against the all-local op (device events, max over ranks)
    def timed(fn, n=5):
        for _ in range(2):
            fn()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        dist.barrier()
        torch.cuda.synchronize()
        a.record()
        for _ in range(n):
            fn()
        b.record()
        b.synchronize()
        t = torch.tensor([a.elapsed_time(b) / n], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t)
    if os.environ.get("SS_EP_BENCH"):
        T2, D2, F2, E2, k2 = 8192, 2048, 1024, 64, 8
        ep2 = ExpertParallelGroup(T2, k2, D2, E2)
        e2 = E2 // world
        b13 = (torch.randn(e2, 2 * F2, D2, device=dev) * 0.02).bfloat16()
        b2 = (torch.randn(e2, D2, F2, device=dev) * 0.02).bfloat16()
        hh = torch.randn(T2, D2, device=dev).bfloat16().requires_grad_(True)
        lg = torch.randn(T2, E2, device=dev).requires_grad_(True)
        dd = torch.randn(T2, D2, device=dev).bfloat16()

        def run():
            experts(hh, lg, b13, b2, ep2, True, None).backward(dd)
        ms = timed(run)
        # the same per-rank expert work with nothing crossing NVLink (all-local op on E/R experts)
        lg_l = torch.randn(T2, e2, device=dev).requires_grad_(True)

        def run_local():
            moe_ops.experts(hh, lg_l, b13, b2, k2, True, None).backward(dd)
        ms_local = timed(run_local)
        # what a library all-to-all alone would cost for the four row exchanges of one fwd+bwd
        rows_out = torch.empty(T2 * k2, D2, device=dev, dtype=torch.bfloat16)
        rows_in = torch.empty_like(rows_out)

        def run_a2a():
            for _ in range(4):
                dist.all_to_all_single(rows_in, rows_out)
        ms_a2a = timed(run_a2a)
        flops = 2 * 2 * T2 * k2 * (2 * F2 * D2 + D2 * F2)          # per rank: forward + data gradients
        if rank == 0:
            print(f"EP_BENCH world={world} T={T2} D={D2} F={F2} E={E2} k={k2}: {ms:.3f} ms fwd+bwd "
                  f"(no wgrad sink); all-local experts on the same rows {ms_local:.3f} ms; "
                  f"4 x NCCL all_to_all_single of the row set alone {ms_a2a:.3f} ms; "
                  f"GEMM floor {flops / 1.4e15 * 1e3:.3f} ms at 1.4 PFLOP/s sustained")
    print(f"rank {rank} OK ", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
