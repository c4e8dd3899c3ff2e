"""Server-side batch validation."""
import numpy as np
import pytest

from shadowspill_b200.client import text_batch
from shadowspill_b200.client.packing import pack_batch
from shadowspill_b200.training.inputs import InputError, route, validate_microbatches

GEO = {"microbatch_tokens": 256, "microbatches": 2, "workers": 1, "slots": 16, "vocab_size": 512,
       "extra_fields": []}


def _mbs(seed=0):
    rng = np.random.default_rng(seed)
    seqs = [rng.integers(0, 512, size=int(rng.integers(16, 60))) for _ in range(8)]
    return pack_batch(text_batch(seqs), microbatch_tokens=256, microbatches=2, slots=16)


def test_good_batches_pass_and_route():
    mbs = _mbs()
    validate_microbatches(mbs, GEO)
    parts = route(mbs + mbs, 2, 2)
    assert [len(p) for p in parts] == [2, 2] and parts[1][0] is mbs[0]


@pytest.mark.parametrize("damage,needle", [
    (lambda m: m[0].tokens.__setitem__(3, 9999), "token ids"),
    (lambda m: m[1].weights.__setitem__(0, np.nan), "weights"),
    (lambda m: m[0].cu_seqlens.__setitem__(2, 1), "boundaries"),
    (lambda m: m[0].targets.__setitem__(5, 700), "targets"),
    (lambda m: m.pop(), "expected 2"),
    (lambda m: setattr(m[0], "max_seqlen", 1), "max_seqlen"),
])
def test_damaged_batches_are_rejected(damage, needle):
    mbs = _mbs(1)
    damage(mbs)
    with pytest.raises(InputError) as e:
        validate_microbatches(mbs, GEO)
    assert needle in str(e.value)


def test_objective_inputs_are_required():
    geo = dict(GEO, extra_fields=["old_logprobs"])
    with pytest.raises(InputError):
        validate_microbatches(_mbs(), geo)


def test_parameter_groups_travel_from_the_client_record_to_the_worker_setup():
    import pytest
    from shadowspill_b200.client import BatchConfig, Memory, Model, Optimizer, Resources
    from shadowspill_b200.client.config import training_setup
    from shadowspill_b200.training.components import default_registry, resolve_training
    groups = ({"match": ["*norm*"], "weight_decay": 0.0}, {"match": ["embed.*"], "lr_scale": 0.1})
    body = training_setup(Model("llama3-tiny", dtype="float32"), Optimizer(lr=1e-3, weight_decay=0.1, parameter_groups=groups),
                          batch=BatchConfig(tokens_per_step=512, microbatch_tokens=256),
                          memory=Memory(device_gib=0.5, spill_gib=0.25), resources=Resources(gpus=1, backend="cpu"))
    resolved = resolve_training(body, default_registry(), {"gpus": 0, "host_free_gib": 8})
    assert resolved.setups[0]["parameter_groups"] == [dict(g) for g in groups]
    from shadowspill_b200.training.phases import setup_from_json
    setup = setup_from_json(resolved.setups[0])
    assert setup.parameter_groups[1]["lr_scale"] == 0.1 and setup.weight_decay == 0.1
    with pytest.raises(ValueError):
        Optimizer(parameter_groups=({"weight_decay": 0.0},))
    with pytest.raises(ValueError):
        Optimizer(parameter_groups=({"match": ["*"], "momentum": 0.9},))
