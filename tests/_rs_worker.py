"""Child process: one rank of the unit test of the fused reduce-scatter + AdamW kernel.

Fills gradients, parameters and moments with known values on every rank, calls
``PeerCollectives.reduce_scatter_adamw`` (stochastic rounding off) and compares p, m and v of the
owned slice element by element with the plain AdamW definition applied to the fp32 sum of the
ranks' gradients. A kernel that skipped the update, mis-signed it or dropped a rank's
contribution fails by orders of magnitude; the tolerance is one bf16 unit in the last place.
"""
import os
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))

import torch
import torch.distributed as dist

from shadowspill_b200.ops import _lib
from shadowspill_b200.parallel import collectives as pc


def ulp_bf16(x: torch.Tensor) -> torch.Tensor:
    """Spacing of bf16 numbers at |x| (8 significand bits)."""
    return torch.exp2(torch.floor(torch.log2(x.abs().clamp_min(1e-30))) - 7)


def reference(p, g_sum, m, v, *, lr, beta1, beta2, eps, wd, step, grad_scale):
    g = g_sum * grad_scale
    m2 = beta1 * m + (1 - beta1) * g
    v2 = beta2 * v + (1 - beta2) * g * g
    p2 = p * (1 - lr * wd) - lr * (m2 / (1 - beta1 ** step)) / ((v2 / (1 - beta2 ** step)).sqrt() + eps)
    return p2, m2, v2


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", device_id=dev)
    pool = pc.allocate_symmetric_pool(64 << 20, dev)
    coll = pc.PeerCollectives(pool)
    nvls = bool(coll.mc_base)
    hyper = dict(lr=3e-3, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1, step=3, grad_scale=0.5)
    failures = []
    # numel: a multiple of 8 per shard; a ragged tensor whose last shard is short and ends
    # mid-vector; a tensor smaller than one vector per rank
    for case, (numel, g_dtype) in enumerate([(1 << 16, torch.bfloat16), (100_003, torch.bfloat16),
                                             (40_001, torch.float32), (11, torch.bfloat16)]):
        per = -(-(-(-numel // world)) // 8) * 8
        gen = torch.Generator(device=dev).manual_seed(100 + case)       # same stream on every rank
        grads_all = [(torch.randn(numel, generator=gen, device=dev) * (r + 1)).to(g_dtype) for r in range(world)]
        p_full = (torch.randn(numel, generator=gen, device=dev) * 0.5).bfloat16()
        m_full = (torch.randn(numel, generator=gen, device=dev) * 0.1).bfloat16()
        v_full = (torch.rand(numel, generator=gen, device=dev) * 0.01).bfloat16()
        nbytes = numel * grads_all[0].element_size()
        grad = pool[:-(-nbytes // 256) * 256][:nbytes].view(g_dtype)     # inside the symmetric pool
        grad.copy_(grads_all[rank])
        lo, hi = min(numel, rank * per), min(numel, rank * per + per)
        pad = lambda t: torch.cat([t[lo:hi], t.new_zeros(per - (hi - lo))])
        p, m, v = pad(p_full), pad(m_full), pad(v_full)
        coll.barrier_begin()
        coll.reduce_scatter_adamw(grad, p, m, v, offset=0, seed=7, stochastic_param=False,
                                  stochastic_state=False, **hyper)
        coll.barrier_end()
        torch.cuda.synchronize()
        _lib.check_status(dev)
        g_sum = sum(g.float() for g in grads_all)
        sums = [g_sum]
        if nvls and g_dtype == torch.bfloat16:
            # the switch returns the sum as bf16; which neighbour it rounds to is its business, so the
            # result may follow either bf16 neighbour of the exact sum
            near = g_sum.bfloat16().float()
            step_ = ulp_bf16(near)
            # at a power of two the neighbour towards zero is half a step away
            sums = [near, near - step_, near + step_, near - step_ / 2, near + step_ / 2]
            g_sum = near

        def ref_for(gs):
            return reference(p_full.float(), gs, m_full.float(), v_full.float(), lr=hyper["lr"],
                             beta1=hyper["beta1"], beta2=hyper["beta2"], eps=hyper["eps"], wd=hyper["weight_decay"],
                             step=hyper["step"], grad_scale=hyper["grad_scale"])
        wants = [ref_for(gs) for gs in sums]
        want = wants[0]
        for idx, (name, got, ref_full, old) in enumerate((("p", p, want[0], p_full), ("m", m, want[1], m_full),
                                                          ("v", v, want[2], v_full))):
            # one unit in the last place of the result, plus the fp32 rounding of the terms themselves,
            # which matters where they cancel. With the in-switch sum the result may follow any of the
            # candidate sums, each judged against the spacing at ITS result: where the terms cancel, a
            # neighbouring sum gives a result orders of magnitude larger than the nearest one does
            terms = old[lo:hi].float().abs() + (g_sum[lo:hi] * hyper["grad_scale"]).abs() + 1e-3
            good = torch.zeros(hi - lo, dtype=torch.bool, device=dev)
            for w in wants:
                ref = w[idx][lo:hi]
                good |= (got[:hi - lo].float() - ref).abs() <= ulp_bf16(ref) * 1.01 + 4e-7 * terms
            err, tol = (~good).float(), 0.5
            bad = int((err > tol).sum())
            # a slice of a few elements may round back to where it was; a real slice must move
            moved = float((got[:hi - lo].float() - old[lo:hi].float()).abs().max()) if hi - lo >= 64 else 1.0
            if bad or moved == 0.0:
                failures.append(f"case {case} {name}: {bad} elements off, largest change {moved:.3g}")
        if per - (hi - lo) > 0 and float(p[hi - lo:].float().abs().max()) != 0.0:
            failures.append(f"case {case}: padding past the tensor's end was written")
    if failures:
        print(f"rank {rank} FAILED: " + "; ".join(failures), flush=True)
        sys.exit(1)
    print(f"rank {rank} OK nvls={int(nvls)}", flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
