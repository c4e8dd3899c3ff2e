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


def _family_grads_match(cfg_name, tol=5e-4):
    cfg = preset(cfg_name)
    tr = ResidentTrainer(cfg, device="cpu", dtype=torch.float32, seed=2)
    # non-trivial values for parameters that start at zero
    with torch.no_grad():
        for si, st in enumerate(tr.stages):
            for p in st.params:
                if p.name in ("A_log", "dt_bias", "lin_norm", "attn_norm", "mlp_norm", "q_norm", "k_norm"):
                    tr.P[si][p.name].add_(torch.randn(p.shape) * 0.1)
    mbs = [to_device(m, "cpu") for m in make_batch(4, vocab=cfg.vocab_size, tokens_per_step=384,
                                                   microbatch_tokens=192, median=50, min_len=8,
                                                   max_len=100)]
    tr.loss_sum.zero_()
    for mb in mbs:
        tr.forward_backward(mb)
    params = {k: v.clone().requires_grad_(True) for k, v in tr.state_dict().items()}
    total = sum(torch_reference.model_loss(cfg, params, mb) for mb in mbs)
    total.backward()
    assert abs(float(total.detach()) - float(tr.loss_sum)) < 1e-4 * max(1.0, abs(float(total.detach())))
    for si, st in enumerate(tr.stages):
        for p in st.params:
            ref = params[f"{st.name}.{p.name}"].grad
            ref = torch.zeros(p.shape) if ref is None else ref
            got = tr.G[si][p.name].float()
            err = (got - ref).abs().max() / (ref.abs().max() + 1e-9)
            assert err < tol, (st.name, p.name, float(err))


def test_qwen35_hybrid_gradients():
    _family_grads_match("qwen35-tiny")


def test_olmoe_gradients():
    _family_grads_match("olmoe-tiny")


def test_qwen3moe_gradients():
    _family_grads_match("qwen3moe-tiny")


def test_qwen35moe_gradients():
    _family_grads_match("qwen35moe-tiny")


def test_catalog_parameter_counts():
    # the reference's table (MODELS.md:38-59)
    want = {"llama3-tiny": 426_624, "llama3-8b": 8_030_261_248, "qwen3-tiny": 525_184,
            "qwen3-8b": 8_190_735_360, "qwen3-32b": 32_762_123_264}
    for name, n in want.items():
        assert preset(name).parameter_count() == n, name
