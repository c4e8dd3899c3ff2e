"""The hand-written stage backward passes against torch.autograd (CPU, fp32)."""
import torch

from shadowspill_b200.data.synthetic import make_batch, to_device
from shadowspill_b200.execution.resident import ResidentTrainer
from shadowspill_b200.models import torch_reference
from shadowspill_b200.models.config import preset


def _grads_match(cfg_name, tol=2e-4):
    cfg = preset(cfg_name)
    tr = ResidentTrainer(cfg, device="cpu", dtype=torch.float32, seed=1)
    mbs = [to_device(m, "cpu") for m in make_batch(3, vocab=cfg.vocab_size, tokens_per_step=512,
                                                   microbatch_tokens=256, median=60, min_len=8,
                                                   max_len=128)]
    tr.loss_sum.zero_()
    for mb in mbs:
        tr.forward_backward(mb)
    params = {k: v.clone().requires_grad_(True) for k, v in tr.state_dict().items()}
    total = sum(torch_reference.loss(cfg, params, mb) for mb in mbs)
    total.backward()
    assert abs(float(total) - float(tr.loss_sum)) < 1e-4 * max(1.0, abs(float(total)))
    for si, st in enumerate(tr.stages):
        for p in st.params:
            ref = params[f"{st.name}.{p.name}"].grad
            got = tr.G[si][p.name].float()
            err = (got - ref).abs().max() / (ref.abs().max() + 1e-12)
            assert err < tol, (st.name, p.name, float(err))


def test_llama_tiny_gradients():
    _grads_match("llama3-tiny")


def test_qwen3_tiny_gradients():
    _grads_match("qwen3-tiny")


def test_training_reduces_loss():
    cfg = preset("llama3-tiny")
    tr = ResidentTrainer(cfg, device="cpu", dtype=torch.float32, seed=0, lr=3e-3)
    mbs = [to_device(m, "cpu") for m in make_batch(0, vocab=cfg.vocab_size, tokens_per_step=512,
                                                   microbatch_tokens=256, median=60, min_len=8,
                                                   max_len=128)]
    losses = [tr.step(mbs) for _ in range(8)]
    assert losses[-1] < losses[0]
