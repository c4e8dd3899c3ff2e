"""Every model family trains on a B200 through the native kernels (bf16)."""
from dataclasses import replace

import pytest
import torch

from shadowspill_b200.data.synthetic import make_batch, to_device
from shadowspill_b200.execution.resident import ResidentTrainer
from shadowspill_b200.models.config import DecoderConfig, preset
from shadowspill_b200.ops import _lib

pytestmark = pytest.mark.gpu


def _gpu_shape(name: str) -> DecoderConfig:
    """The family's tiny preset with head widths the sm_100a attention kernels accept."""
    c = preset(name)
    return replace(c, d_model=256, head_dim=64, dn_head_dim=64 if c.dn_v_heads else c.dn_head_dim,
                   vocab_size=1024)


@pytest.mark.parametrize("name", ["llama3-tiny", "qwen3-tiny", "qwen35-tiny", "olmoe-tiny",
                                  "qwen3moe-tiny", "qwen35moe-tiny"])
def test_family_trains_and_matches_cpu_reference(name):
    cfg = _gpu_shape(name)
    host = make_batch(0, vocab=cfg.vocab_size, tokens_per_step=1024, microbatch_tokens=512,
                      median=100, min_len=16, max_len=300)
    gpu = ResidentTrainer(cfg, device="cuda", seed=3, lr=2e-3, stochastic_rounding=False)
    cpu = ResidentTrainer(cfg, device="cpu", dtype=torch.float32, seed=3, lr=2e-3)
    # same starting point: the bf16 weights, widened
    for (k, a), (_, b) in zip(sorted(gpu.state_dict().items()), sorted(cpu.state_dict().items())):
        b.copy_(a.float().cpu())
    first_gpu = gpu.step([to_device(m, "cuda") for m in host])
    first_cpu = cpu.step([to_device(m, "cpu") for m in host])
    assert abs(first_gpu - first_cpu) < 2e-2 * abs(first_cpu), (first_gpu, first_cpu)
    last = first_gpu
    for _ in range(4):
        last = gpu.step([to_device(m, "cuda") for m in host])
    torch.cuda.synchronize()
    _lib.check_status()
    assert last == last and last < first_gpu


@pytest.mark.parametrize("name", ["llama3-tiny", "olmoe-tiny"])
def test_lora_gradients_on_gpu_match_cpu(name):
    """Adapter gradients from the sm_100a kernels (incl. rank-16 GEMMs and grouped
    per-expert factors) against the fp32 CPU path on the same bf16 weights."""
    from shadowspill_b200.models.lora import LoRAConfig
    cfg = _gpu_shape(name)
    lora = LoRAConfig(rank=16, alpha=32.0, targets=("wq", "wv", "wo", "w13", "w2"))
    host = make_batch(1, vocab=cfg.vocab_size, tokens_per_step=512, microbatch_tokens=512,
                      median=100, min_len=16, max_len=300)
    gpu = ResidentTrainer(cfg, device="cuda", seed=3, lora=lora, stochastic_rounding=False)
    cpu = ResidentTrainer(cfg, device="cpu", dtype=torch.float32, seed=3, lora=lora)
    g = torch.Generator(device="cuda").manual_seed(5)
    for P in gpu.P:
        for n, t in P.items():
            if n.endswith("_lora_b"):
                t.normal_(0.0, 0.05, generator=g)
    for (k, a), (_, b) in zip(sorted(gpu.state_dict().items()), sorted(cpu.state_dict().items())):
        b.copy_(a.float().cpu())
    gpu.forward_backward(to_device(host[0], "cuda"))
    cpu.forward_backward(to_device(host[0], "cpu"))
    torch.cuda.synchronize()
    _lib.check_status()
    assert abs(float(gpu.loss_sum) - float(cpu.loss_sum)) < 2e-2 * abs(float(cpu.loss_sum))
    checked = 0
    for Gg, Gc in zip(gpu.G, cpu.G):
        assert set(Gg) == set(Gc)
        for n in Gg:
            a, b = Gg[n].float().cpu(), Gc[n].float()
            if b.norm() == 0:
                continue
            rel = float((a - b).norm() / b.norm())
            cos = float((a * b).sum() / (a.norm() * b.norm()))
            # routed layers add bf16 routing ties on top of rounding noise
            lim, cmin = (0.15, 0.99) if cfg.is_moe else (0.08, 0.995)
            assert rel < lim and cos > cmin, (n, rel, cos)
            checked += 1
    assert checked >= 4


def test_policy_objective_kernel_matches_reference():
    from shadowspill_b200.ops import functional as F
    from shadowspill_b200.ops import reference as opref
    torch.manual_seed(0)
    R, V = 300, 4096 + 40
    logits = (torch.randn(R, V, device="cuda") * 2).bfloat16()
    tgt = torch.randint(0, V, (R,), device="cuda")
    tgt[::9] = -1
    w = torch.rand(R, device="cuda")
    logp0 = torch.log_softmax(logits.float(), -1).gather(1, tgt.clamp(0)[:, None])[:, 0]
    old = logp0 + 0.3 * torch.randn(R, device="cuda")
    adv = torch.randn(R, device="cuda")
    refp = old + 0.1 * torch.randn(R, device="cuda")
    want_block = logits.clone().float()
    want, want_lp = opref.clipped_policy_(want_block, tgt, w, old, adv, 0.2, refp, 0.05, 1.0, True)
    got = torch.zeros(1, device="cuda")
    lp = torch.empty(R, device="cuda")
    block = logits.clone()
    F.clipped_policy_(block, tgt, w, old, adv, got, clip=0.2, ref_logp=refp, ref_beta=0.05, logp=lp)
    torch.cuda.synchronize()
    assert abs(float(got) - float(want)) < 2e-3 * abs(float(want)) + 1e-3
    ok = tgt >= 0
    assert torch.allclose(lp[ok], want_lp[ok], atol=2e-3)
    err = (block.float() - want_block).norm() / want_block.norm()
    assert float(err) < 1e-2
    only = torch.empty(R, device="cuda")
    F.target_logprobs_(logits, tgt, only)
    assert torch.allclose(only[ok], want_lp[ok], atol=2e-3)
