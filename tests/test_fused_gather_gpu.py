"""The all-gather fused into the consuming GEMM, on one GPU: the "ranks" are shards in local
memory, which exercises the whole kernel (gather warps, per-tile counters, the TMA producer's
bounded wait, n-major tile order) except the NVLink hop. No kernel waits on another launch."""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def _shards(W: torch.Tensor, world: int):
    flat = W.reshape(-1)
    per = -(-(-(-flat.numel() // world)) // 8) * 8
    out = []
    for r in range(world):
        s = torch.zeros(per, dtype=W.dtype, device=W.device)
        lo, hi = min(flat.numel(), r * per), min(flat.numel(), r * per + per)
        s[:hi - lo] = flat[lo:hi]
        out.append(s)
    return out, per


@pytest.mark.parametrize("M,N,K,world", [(1024, 768, 512, 2), (512, 1000, 256, 4), (4096, 6144, 1024, 8)])
def test_gather_fused_gemm_matches_plain_gemm_and_fills_the_weight(M, N, K, world):
    from shadowspill_b200.ops import _lib, functional as F
    torch.manual_seed(M + N)
    x = (torch.randn(M, K, device="cuda") * 0.5).bfloat16()
    W = (torch.randn(N, K, device="cuda") * 0.5).bfloat16()
    shards, per = _shards(W, world)
    full = torch.full((N, K), float("nan"), dtype=torch.bfloat16, device="cuda")   # nothing gathered yet
    want = F.gemm(x, W)
    F.register_gather(F.PendingGather(full, [s.data_ptr() for s in shards], per, world, 1,
                                      lambda: pytest.fail("the stand-alone gather ran")))
    before = F.fused_gather_launches
    got = F.linear_fwd(x, full)
    torch.cuda.synchronize()
    _lib.check_status()
    assert F.fused_gather_launches == before + 1
    assert torch.equal(full, W)                        # the weight is local for later GEMMs
    assert torch.equal(got, want)                      # same kernel, same arithmetic
    assert torch.equal(F.linear_fwd(x, full), want)    # nothing pending any more: the plain GEMM


def test_small_row_counts_fall_back_to_the_stand_alone_gather():
    from shadowspill_b200.ops import functional as F
    x = torch.randn(64, 256, device="cuda").bfloat16()
    W = torch.randn(512, 256, device="cuda").bfloat16()
    full = torch.zeros_like(W)
    ran = []
    F.register_gather(F.PendingGather(full, [W.data_ptr()], W.numel(), 1, 0,
                                      lambda: (ran.append(1), full.copy_(W))))
    got = F.linear_fwd(x, full)
    assert ran == [1] and torch.equal(got, F.gemm(x, W))
    assert F.flush_gathers() == 0
