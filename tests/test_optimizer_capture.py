"""Any elementwise torch.optim optimizer as the update rule of planned training."""
import pytest
import torch

from shadowspill_b200.data.synthetic import make_batch, to_device
from shadowspill_b200.frontend.optimizer_capture import OptimizerNotCapturable, capture_optimizer_update
from shadowspill_b200.models import torch_reference as twin
from shadowspill_b200.models.config import preset
from shadowspill_b200.planning.plan import SearchOptions
from shadowspill_b200.training.session import TrainingSession, TrainingSetup

FACTORIES = {
    # eps well above the rounding noise of a near-zero gradient: with the default 1e-10 the first
    # steps are lr * g / |g|, which turns that noise into whole steps in either implementation
    "adagrad": lambda ps: torch.optim.Adagrad(ps, lr=1e-2, eps=1e-3),
    "rmsprop_momentum": lambda ps: torch.optim.RMSprop(ps, lr=1e-3, momentum=0.9, alpha=0.95),
    "adamw": lambda ps: torch.optim.AdamW(ps, lr=1e-3, betas=(0.9, 0.95), weight_decay=0.05),
    "radam": lambda ps: torch.optim.RAdam(ps, lr=1e-3),
}


@pytest.mark.parametrize("name", sorted(FACTORIES))
def test_captured_update_trains_like_the_eager_optimizer(name):
    """Three planned, spilling updates with the captured graph as the update rule against eager
    PyTorch stepping the same optimizer on the fp32 twin model: same losses, same weights."""
    factory = FACTORIES[name]
    captured = capture_optimizer_update(factory)
    assert str(captured).startswith("captured:") and 1 <= len(captured.state_names) <= 2
    cfg = preset("llama3-tiny")
    lr = factory([torch.nn.Parameter(torch.zeros(1))]).param_groups[0]["lr"]
    session = TrainingSession(TrainingSetup(
        model=cfg, device_gib=0.53, spill_gib=0.25, tokens_per_step=512, microbatch_tokens=256, lr=lr,
        device="cpu", dtype="float32", profile=False, calibrate=False, seed=3, optimizer_rule=captured,
        stochastic_rounding=False, search=SearchOptions(minimum_object_bytes_evict_eligible=1024, workers=1)))
    assert session.plan.summary.fetch_bytes > 0
    params = {k: v.clone().requires_grad_(True) for k, v in session.executor.state_dict().items()
              if not k.startswith("exp_avg")}
    opt = factory(list(params.values()))
    for step in range(3):
        host = make_batch(step, vocab=cfg.vocab_size, tokens_per_step=512, microbatch_tokens=256, median=60,
                          min_len=8, max_len=128, slots=session.slots)
        got = session.step(host).loss
        opt.zero_grad()
        want = 0.0
        for mb in host:
            loss = twin.model_loss(cfg, params, to_device(mb, "cpu"))
            loss.backward()
            want += float(loss.detach())
        opt.step()
        assert abs(got - want) < 1e-5 * max(1.0, abs(want)), (name, step, got, want)
    state = session.executor.state_dict()
    for k, v in params.items():
        diff = (state[k] - v.detach()).float()
        assert float(diff.norm() / v.detach().float().norm().clamp_min(1e-9)) < 1e-4, (name, k)
    session.close()


def test_what_cannot_be_captured_says_why():
    with pytest.raises(OptimizerNotCapturable, match="closure"):
        capture_optimizer_update(lambda ps: torch.optim.LBFGS(ps))
    with pytest.raises(OptimizerNotCapturable, match="mu_product"):
        capture_optimizer_update(lambda ps: torch.optim.NAdam(ps))

    class Normalised(torch.optim.SGD):                       # mixes the elements of a parameter
        @torch.no_grad()
        def step(self, closure=None):
            for group in self.param_groups:
                for p in group["params"]:
                    p.add_(p.grad / p.grad.norm(), alpha=-group["lr"])
    with pytest.raises(OptimizerNotCapturable, match="elementwise|reproduce"):
        capture_optimizer_update(lambda ps: Normalised(ps, lr=1e-2))
