"""Prepared bundles: a second session opens from the archive and trains identically."""
from dataclasses import replace

from shadowspill_b200.data.synthetic import make_batch
from shadowspill_b200.planning.plan import SearchOptions
from shadowspill_b200.training.preparation import load_bundle
from shadowspill_b200.training.session import TrainingSession, TrainingSetup


def _setup(bundle):
    return TrainingSetup(model="llama3-tiny", device_gib=0.53, spill_gib=0.25, tokens_per_step=512,
                         microbatch_tokens=256, lr=3e-3, device="cpu", dtype="float32", profile=False,
                         calibrate=False, seed=11, bundle=str(bundle), operations=("step", "forward"),
                         search=SearchOptions(minimum_object_bytes_evict_eligible=1024, workers=1))


def _losses(session, n=3):
    out = []
    for i in range(n):
        batch = make_batch(i, vocab=session.cfg.vocab_size, tokens_per_step=512, microbatch_tokens=256,
                           median=60, min_len=8, max_len=128, slots=session.slots)
        out.append(session.step(batch).loss)
    ev = session.run("forward", make_batch(9, vocab=session.cfg.vocab_size, tokens_per_step=512,
                                           microbatch_tokens=256, median=60, min_len=8, max_len=128,
                                           slots=session.slots)).loss
    session.close()
    return out + [ev]


def test_bundle_round_trip_and_identity(tmp_path):
    path = tmp_path / "training.ssp"
    first = TrainingSession(_setup(path))
    assert not first.prepared_from_bundle and path.exists()
    meta = load_bundle(path)
    assert meta["plan"]["format"] == "ss-b200.plan" and "forward" in meta["extra_plans"]
    want = _losses(first)
    second = TrainingSession(_setup(path))
    assert second.prepared_from_bundle and second.sweep is None
    assert second.plan.to_json() == first.plan.to_json()
    assert _losses(second) == want
    # another budget is another identity: the bundle is ignored and rewritten
    other = TrainingSession(replace(_setup(path), device_gib=0.6))
    assert not other.prepared_from_bundle
    other.close()
    assert load_bundle(path)["identity"] != meta["identity"]
