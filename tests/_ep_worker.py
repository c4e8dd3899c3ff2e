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
    print(f"rank {rank} OK ", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
