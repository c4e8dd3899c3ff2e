"""Prepared bundles: a second session opens from the archive and trains identically."""
from dataclasses import replace

import pytest

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


def test_pretrained_weights_and_adapters_through_the_session(tmp_path):
    """A base model exported with Hugging Face names is the starting point of a LoRA run:
    base tensors come from the file, adapters start fresh, only adapters train."""
    import torch
    from shadowspill_b200.checkpoint import hf
    from shadowspill_b200.execution.resident import ResidentTrainer
    from shadowspill_b200.models.config import preset
    from shadowspill_b200.models.lora import LoRAConfig
    cfg = preset("llama3-tiny")
    base = ResidentTrainer(cfg, device="cpu", dtype=torch.float32, seed=123).state_dict()
    hf.save_hf(cfg, base, tmp_path / "base")
    setup = replace(_setup(tmp_path / "lora.ssp"), pretrained=str(tmp_path / "base"), operations=("step",),
                    lora=LoRAConfig(rank=8, alpha=16.0).to_json(), lr=1e-2)
    session = TrainingSession(setup)
    state = session.executor.state_dict()
    q = state["layer0.wq"]
    Hq = cfg.n_heads * cfg.head_dim
    assert torch.equal(q, base["layer0.wqkv"][:Hq])           # fused projection cut back into wq
    assert torch.equal(state["embed.embed"], base["embed.embed"])
    assert float(state["layer0.wq_lora_b"].abs().max()) == 0.0
    losses = []
    for i in range(3):
        batch = make_batch(0, vocab=cfg.vocab_size, tokens_per_step=512, microbatch_tokens=256,
                           median=60, min_len=8, max_len=128, slots=session.slots)
        losses.append(session.step(batch).loss)
    after = session.executor.state_dict()
    assert losses[-1] < losses[0]
    assert torch.equal(after["layer0.wq"], q)                  # the base stayed frozen
    assert float(after["layer0.wq_lora_b"].abs().max()) > 0.0  # the adapter moved
    session.close()


def test_measure_plan_runs_a_prepared_bundle_without_preparing(tmp_path):
    """The plan-measurement tool opens an existing bundle (no build, profile or search), runs
    updates, and writes per-update and summary figures; a bundle of another setup is refused."""
    import json
    from shadowspill_b200.execution.measure_plan import run
    path = tmp_path / "training.ssp"
    TrainingSession(_setup(path)).close()
    out = tmp_path / "measurement"
    report = run(_setup(path), steps=3, warmup_steps=1, output_dir=out)
    s = report["summary"]
    assert s["prepared_from_bundle"] and s["steps"] == 3 and s["tokens_per_second"] > 0
    assert len(report["updates"]) == 4 and report["updates"][0]["warmup"] and not report["updates"][1]["warmup"]
    assert all(u["loss"] > 0 for u in report["updates"])
    assert sum(u["fetch_bytes"] for u in report["updates"]) > 0
    assert json.loads((out / "measurement.json").read_text())["summary"]["unit"] == "tokens"
    assert "measured / simulated" in (out / "measurement.md").read_text()
    with pytest.raises(RuntimeError, match="does not match"):
        run(replace(_setup(path), device_gib=0.61), steps=1, warmup_steps=0)


def test_preparation_as_four_fresh_processes(tmp_path):
    """build, profile, communicate and plan each run as their own process and hand their results
    on through files; the bundle they end in opens a session that trains exactly like one that
    prepared in-process, and a second call finds every phase done."""
    import json
    from shadowspill_b200.training.phases import prepare_job, setup_from_json, setup_to_json
    directory = tmp_path / "prep"
    setup = replace(_setup(""), profile=True)          # profiling on the CPU: wall-clock task times
    assert setup_from_json(json.loads(json.dumps(setup_to_json(setup), default=str))) == setup
    bundle = prepare_job(setup, directory)
    assert bundle.exists() and bundle.name == "training.ssp"
    for name in ("build.json", "profiles.json", "communication.json", "job.json", "build.log", "plan.log"):
        assert (directory / name).exists(), name
    built = json.loads((directory / "build.json").read_text())
    assert len(built["candidates"]) >= 1 and set(built["operations"]) == {"forward"}
    profiles = json.loads((directory / "profiles.json").read_text())["profiles"]["tasks"]
    assert profiles and all(p["seconds"] > 0 for p in profiles.values())
    job = json.loads((directory / "job.json").read_text())["phases"]
    assert [p["phase"] for p in job] == ["build", "profile", "communicate", "plan"]
    assert all(p.get("pid_was_fresh") for p in job)
    opened = TrainingSession(replace(setup, bundle=str(bundle)))
    assert opened.prepared_from_bundle and set(opened.profiles.tasks) == set(profiles)
    direct = TrainingSession(replace(setup, profile=False))
    assert [t.name for t in opened.plan.program.tasks] == [t.name for t in direct.plan.program.tasks]
    assert _losses(opened) == _losses(direct)
    again = prepare_job(setup, directory)               # nothing to do: every result is there
    assert again == bundle
    assert all(p.get("skipped") for p in json.loads((directory / "job.json").read_text())["phases"])
