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
