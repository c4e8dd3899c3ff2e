"""Public client -> HTTP service -> worker process -> planned execution, on CPU.

A real ``Server`` listens on loopback, the run's worker is a real subprocess with
the mock backend, and the client is the NumPy-only package a user imports.
"""
import io

import numpy as np
import time

import pytest

from shadowspill_b200.client import (BatchConfig, BatchError, Memory, Model, Optimizer, TransportError,
                                     OperationFailed, Preparation, ProfilingOptions, Resources,
                                     ServiceClient, text_batch)
from shadowspill_b200.client.config import PlanningOptions
from shadowspill_b200.server.service import Server


def _sequences(seed, n=8, vocab=512):
    rng = np.random.default_rng(seed)
    return [rng.integers(0, vocab, size=int(rng.integers(16, 60))) for _ in range(n)]


@pytest.fixture(scope="module")
def service(tmp_path_factory):
    with Server(tmp_path_factory.mktemp("service"), token="secret") as srv:
        yield srv


def _trainer(svc, operations=("step",)):
    return svc.create_training_client(
        Model("llama3-tiny", dtype="float32"), Optimizer(lr=3e-3, parameter_rounding="nearest"),
        batch=BatchConfig(tokens_per_step=512, microbatch_tokens=256),
        memory=Memory(device_gib=0.53, spill_gib=0.25), resources=Resources(gpus=1, backend="cpu"),
        preparation=Preparation(profiling=ProfilingOptions(enabled=False), calibrate=False,
                                planning=PlanningOptions(minimum_object_bytes_evict_eligible=1024,
                                                         workers=1)),
        operations=operations, timeout=300).result()


def test_auth_is_enforced(service):
    from shadowspill_b200.client.transport import TransportError
    with pytest.raises(TransportError) as e:
        ServiceClient(service.url, token="wrong")
    assert e.value.status == 401


def test_train_checkpoint_resume_through_the_public_api(service, tmp_path_factory):
    with ServiceClient(service.url, token="secret") as svc:
        hw = svc.list_hardware().result()
        assert hw["nodes"][0]["cpus"] >= 1
        desc = svc.describe_training(model=Model("llama3-tiny"),
                                     resources=Resources(backend="cpu")).result()
        assert desc["workers"] == 1 and desc["parameters"] == 426_624
        trainer = _trainer(svc, ("step", "forward_backward", "optim_step", "forward"))
        assert trainer.info["plan_summary"]["fetch_bytes"] > 0
        plans = svc.get_plans(trainer.run).result()["plans"]
        assert [p["operation"] for p in plans] == ["step", "forward", "forward_backward", "optim_step"]
        assert all(p["duration_seconds"] > 0 for p in plans)
        losses = [trainer.step(text_batch(_sequences(0))).result().loss for _ in range(4)]
        assert losses[-1] < losses[0]
        # forward: the loss and, per datum, log p(target) of every position
        probe = text_batch(_sequences(7))
        fwd = trainer.forward(probe).result()
        per = fwd.outputs["per_datum"]
        assert len(per) == len(probe) and all(p.shape == (len(d), 1) for p, d in zip(per, probe))
        rebuilt = sum(float(-(p[:, 0] * d.weights)[d.targets >= 0].sum()) for p, d in zip(per, probe))
        assert abs(rebuilt - fwd.loss) < 1e-4
        # accumulation: two contributions then one update
        f1 = trainer.forward_backward(text_batch(_sequences(1)))
        f2 = trainer.forward_backward(text_batch(_sequences(2)))
        up = trainer.optim_step()
        assert f1.result().loss > 0 and f2.result().loss > 0
        assert up.result().completed_updates == 5
        ev = trainer.forward(text_batch(_sequences(0))).result().loss
        assert 0 < ev < losses[0]
        # a step while gradients are open is rejected, and says why
        trainer.forward_backward(text_batch(_sequences(3))).result()
        with pytest.raises(OperationFailed) as e:
            trainer.step(text_batch(_sequences(0))).result()
        assert "accumulation" in str(e.value)
        trainer.discard_gradients().result()
        saved = trainer.save_checkpoint("after5").result()
        assert saved.outputs["checkpoint"] == "after5"
        # the checkpoint can be fetched: packed on the service, downloaded with ranges, unpacked
        assert trainer.list_checkpoints() == ["after5"]
        listing = trainer.checkpoint_manifest("after5").result()
        assert listing["checkpoint"] == "after5" and len(listing["files"]) == 1
        assert listing["files"][0]["tensors"] > 10 and "embed.embed" in listing["files"][0]["names"]
        assert svc.wait_ready(trainer.run).result()["state"] == "ready"
        local = trainer.download_checkpoint("after5", tmp_path_factory.mktemp("dl"), chunk_bytes=200_000).result()
        from shadowspill_b200.checkpoint.load import checkpoint_files, export_weights
        assert len(checkpoint_files(local)) == 1
        weights = export_weights(local)
        assert weights["embed.embed"].shape == (512, 128) and "exp_avg.embed.embed" not in weights
        report = trainer.download_plan_report(tmp_path_factory.mktemp("report")).result()
        assert (report / "index.html").exists() and (report / "tasks.csv").exists()
        next_loss = trainer.step(text_batch(_sequences(7))).result().loss
        # local validation never reaches the server
        with pytest.raises(BatchError):
            trainer.step(text_batch([np.arange(0, 600) % 512]))
        trainer.log_metrics(6, accuracy=0.5)
        metrics = svc.get_metrics(trainer.run).result()["metrics"]
        assert any(m.get("source") == "caller" for m in metrics) and len(metrics) >= 6
        # ---- the metric journal: one record per finished request of any operation, paged reads
        page = trainer.metrics.query(limit=4).result()
        assert len(page.records) == 4 and page.next_cursor == 4 and page.through >= 10
        records = list(trainer.metrics.snapshot(limit=3))
        assert [r["position"] for r in records] == list(range(1, len(records) + 1))
        assert {"step", "forward", "forward_backward", "optim_step", "save"} <= {r.get("operation") for r in records}
        xs, ys = trainer.metrics.series("loss")
        assert len(ys) >= 6 and xs == sorted(xs)
        assert trainer.metrics.series("accuracy")[1] == [0.5]
        exported = trainer.metrics.export_jsonl(tmp_path_factory.mktemp("metrics") / "run.jsonl").result()
        assert len(exported.read_text().splitlines()) == len(records)
        with pytest.raises(FileExistsError):
            trainer.metrics.export_jsonl(exported).result()
        with pytest.raises(ValueError):
            trainer.metrics.query(limit=1000)
        # ---- local validation reports what it found; a table follows a call without touching it
        import io
        from shadowspill_b200.client.display import CommandTable
        from shadowspill_b200.client.text import text_batch_statistics
        check = trainer.validate_batch(probe, "forward")
        assert check.packing_checked and check.strategy in ("best_fit", "balanced", "repair")
        assert check.capacities["tokens"] == sum(len(d) for d in probe) and check.capacities["sequences"] == len(probe)
        assert check.scheduled_capacities["tokens"] == 512
        plan_seconds = trainer.validate_batch(probe, "step").estimated_seconds
        assert plan_seconds and plan_seconds > 0
        screen = io.StringIO()
        table = CommandTable(stream=screen)
        tracked = table.track("forward", trainer.forward(probe), batch=text_batch_statistics(probe),
                              planned_seconds=plan_seconds)
        assert tracked.result().loss > 0
        for _ in range(100):
            if " done " in screen.getvalue():
                break
            time.sleep(0.02)
        lines = screen.getvalue().splitlines()
        assert any("pending" in ln and "forward()" in ln for ln in lines) and any(" done " in ln for ln in lines)
        assert table.error is None
        progress = svc.get_progress(trainer.run).result()["lines"]
        assert any("ready" in line for line in progress)
        trainer.close()
        # ---- resume from the checkpoint in a fresh run: the same next step
        resumed = svc.create_training_client(
            Model("llama3-tiny", dtype="float32"), Optimizer(lr=3e-3, parameter_rounding="nearest"),
            batch=BatchConfig(tokens_per_step=512, microbatch_tokens=256),
            memory=Memory(device_gib=0.53, spill_gib=0.25), resources=Resources(gpus=1, backend="cpu"),
            preparation=Preparation(profiling=ProfilingOptions(enabled=False), calibrate=False,
                                    planning=PlanningOptions(minimum_object_bytes_evict_eligible=1024,
                                                             workers=1)),
            checkpoint="after5", timeout=300).result()
        r = resumed.step(text_batch(_sequences(7))).result()
        assert abs(r.loss - next_loss) < 1e-6 and r.completed_updates == 6
        resumed.close()


def test_newer_writer_fences_the_older_one(service):
    with ServiceClient(service.url, token="secret") as svc:
        first = _trainer(svc)
        first.step(text_batch(_sequences(0))).result()
        second = svc.get_training_client(first.run).result()
        second.step(text_batch(_sequences(1))).result()
        from shadowspill_b200.client.transport import TransportError
        with pytest.raises(TransportError) as e:
            first.step(text_batch(_sequences(2))).result()
        assert e.value.status == 409 and "fenced" in str(e.value)
        # another process: a new client that adopts the session id reaches the run and takes it over
        with ServiceClient(service.url, token="secret", session=svc.session) as later:
            third = later.get_training_client(first.run).result()
            assert third.step(text_batch(_sequences(3))).result().completed_updates == 3
            with pytest.raises(TransportError):
                second.step(text_batch(_sequences(4))).result()
            third.close()
        with pytest.raises(ValueError):
            ServiceClient(service.url, token="secret", session="../elsewhere")


def test_lora_run_through_the_service(service):
    from shadowspill_b200.client import LoRA
    with ServiceClient(service.url, token="secret") as svc:
        trainer = svc.create_training_client(
            Model("llama3-tiny", dtype="float32", lora=LoRA(rank=8, alpha=16.0)),
            Optimizer(lr=1e-2, parameter_rounding="nearest"),
            batch=BatchConfig(tokens_per_step=512, microbatch_tokens=256),
            memory=Memory(device_gib=0.53, spill_gib=0.25), resources=Resources(gpus=1, backend="cpu"),
            preparation=Preparation(profiling=ProfilingOptions(enabled=False), calibrate=False,
                                    planning=PlanningOptions(minimum_object_bytes_evict_eligible=1024,
                                                             workers=1)),
            timeout=300).result()
        losses = [trainer.step(text_batch(_sequences(0))).result().loss for _ in range(4)]
        assert losses[-1] < losses[0]
        trainer.close()


def test_policy_objective_through_the_service(service):
    """Clipped-policy training end to end: per-token old log-probabilities and advantages travel
    from client datums through packing and the wire to the head kernel."""
    from shadowspill_b200.client import Objective, policy_datum
    rng = np.random.default_rng(5)

    def datums(seed):
        out = []
        for seq in _sequences(seed):
            n = len(seq)
            out.append(policy_datum(seq, np.ones(n), rng.normal(-6.0, 0.1, n), rng.normal(0.0, 1.0, n)))
        return text_batch(out)
    with ServiceClient(service.url, token="secret") as svc:
        trainer = svc.create_training_client(
            Model("llama3-tiny", dtype="float32"), Optimizer(lr=1e-3, parameter_rounding="nearest"),
            objective=Objective("shadowspill/clipped_policy@1", {"clip_ratio": 0.2}),
            batch=BatchConfig(tokens_per_step=512, microbatch_tokens=256),
            memory=Memory(device_gib=0.53, spill_gib=0.25), resources=Resources(gpus=1, backend="cpu"),
            preparation=Preparation(profiling=ProfilingOptions(enabled=False), calibrate=False,
                                    planning=PlanningOptions(minimum_object_bytes_evict_eligible=1024,
                                                             workers=1)),
            timeout=300).result()
        first = trainer.step(datums(0)).result().loss
        second = trainer.step(datums(0)).result().loss
        assert np.isfinite(first) and np.isfinite(second) and first != second
        # a batch without the objective's inputs is refused locally, before anything is sent
        with pytest.raises(BatchError):
            trainer.step(text_batch(_sequences(1)))
        assert np.isfinite(trainer.step(datums(1)).result().loss)
        trainer.close()


def test_two_replicas_of_two_ranks_through_the_service(service):
    """``data_parallel(2, replicas=2)``: four gloo workers, state sharded inside each pair."""
    from shadowspill_b200.client import data_parallel
    with ServiceClient(service.url, token="secret") as svc:
        trainer = svc.create_training_client(
            Model("llama3-tiny", dtype="float32"), Optimizer(lr=3e-3, parameter_rounding="nearest"),
            batch=BatchConfig(tokens_per_step=512, microbatch_tokens=256),
            memory=Memory(device_gib=0.53, spill_gib=0.25), resources=Resources(gpus=4, backend="cpu"),
            parallelism=data_parallel(2, replicas=2),
            preparation=Preparation(profiling=ProfilingOptions(enabled=False), calibrate=False,
                                    planning=PlanningOptions(minimum_object_bytes_evict_eligible=1024,
                                                             workers=1)),
            operations=("step", "forward"), timeout=600).result()
        assert trainer.info["workers"] == 4
        batches = [text_batch(_sequences(s, n=32)) for s in (0, 0, 0, 0)]
        losses = [trainer.step(b).result().loss for b in batches]
        assert losses[-1] < losses[0]
        # the client's declaration carries min_shard_bytes = 2 MiB: every tensor of this tiny model
        # is kept whole on each rank. A checkpoint of that job restores into a single worker.
        probe = text_batch(_sequences(9, n=8))
        before = trainer.forward(probe).result().loss
        trainer.save_checkpoint("from4").result()
        trainer.close()
        single = svc.create_training_client(
            Model("llama3-tiny", dtype="float32"), Optimizer(lr=3e-3, parameter_rounding="nearest"),
            batch=BatchConfig(tokens_per_step=512, microbatch_tokens=256),
            memory=Memory(device_gib=0.53, spill_gib=0.25), resources=Resources(gpus=1, backend="cpu"),
            preparation=Preparation(profiling=ProfilingOptions(enabled=False), calibrate=False,
                                    planning=PlanningOptions(minimum_object_bytes_evict_eligible=1024,
                                                             workers=1)),
            operations=("step", "forward"), checkpoint="from4", timeout=300).result()
        after = single.forward(probe).result().loss
        assert abs(after - before) < 1e-5 * max(1.0, abs(before))
        single.close()


def test_resumable_artifact_transfer_and_component_listing(service, tmp_path):
    import hashlib
    from shadowspill_b200.client.handles import upload_artifact
    src = tmp_path / "weights.bin"
    payload = np.random.default_rng(0).integers(0, 256, size=300_000, dtype=np.uint8).tobytes()
    src.write_bytes(payload)
    with ServiceClient(service.url, token="secret") as svc:
        ids = {c["id"] for c in svc.list_components("model").result()}
        assert {"llama3-8b@1", "shadowspill/regression@1"} <= ids
        assert all(c["kind"] == "objective" for c in svc.list_components("objective").result())
        # an upload that stopped after the first chunk resumes where the service stands
        _, begun = svc.transport.request("POST", "/v1/artifacts", {
            "name": "weights.bin", "size": len(payload), "sha256": hashlib.sha256(payload).hexdigest()})
        svc.transport.request("PUT", f"/v1/artifacts/{begun['artifact']}/chunks/0", payload[:65536])
        seen = []
        handle = upload_artifact(svc.transport, src, chunk_bytes=100_000,
                                 on_progress=lambda done, total: seen.append(done))
        assert handle.artifact == begun["artifact"] and seen[0] == 165_536 and seen[-1] == len(payload)
        # a download that already has a part file only fetches the rest
        dst = tmp_path / "copy.bin"
        (tmp_path / "copy.bin.part").write_bytes(payload[:120_000])
        got = []
        svc.download_artifact(handle, dst, chunk_bytes=64_000,
                              on_progress=lambda have, total: got.append(have)).result()
        assert dst.read_bytes() == payload and got[0] == 184_000
        # a corrupted part file is caught by the digest
        (tmp_path / "bad.bin.part").write_bytes(b"x" * 1000)
        with pytest.raises(IOError):
            svc.download_artifact(handle, tmp_path / "bad.bin").result()
        svc.delete_artifact(handle).result()
        from shadowspill_b200.client.transport import TransportError
        with pytest.raises(TransportError):
            svc.download_artifact(handle.artifact, tmp_path / "gone.bin").result()


def test_unsupported_optimizer_state_dtypes_are_refused(service):
    with ServiceClient(service.url, token="secret") as svc:
        with pytest.raises(Exception) as e:
            svc.describe_training(model=Model("llama3-tiny"), optimizer=Optimizer(opt_state_dtype="float32"),
                                  resources=Resources(backend="cpu")).result()
        assert "opt_state_dtype" in str(e.value)
        # fp32 master copies on a bf16 model are a supported request
        assert svc.describe_training(model=Model("llama3-tiny"), optimizer=Optimizer(master_dtype="float32"),
                                     resources=Resources(backend="cpu")).result()["workers"] == 1
        ok = svc.describe_training(model=Model("llama3-tiny", dtype="float32"),
                                   optimizer=Optimizer(master_dtype="float32", opt_state_dtype="float32"),
                                   resources=Resources(backend="cpu")).result()
        assert ok["workers"] == 1


def test_pretrained_weights_arrive_as_an_uploaded_artifact(service, tmp_path):
    """Hugging Face weights packed into a TAR, uploaded, and named by ``Weights.artifact``: the
    run starts from them (its first loss equals a local model's loss on the same weights)."""
    import tarfile
    import torch
    from shadowspill_b200.checkpoint import hf
    from shadowspill_b200.client.config import Weights
    from shadowspill_b200.client.packing import pack_batch
    from shadowspill_b200.data.synthetic import HostMicrobatch, to_device
    from shadowspill_b200.execution.resident import ResidentTrainer
    from shadowspill_b200.models.config import preset
    cfg = preset("llama3-tiny")
    local = ResidentTrainer(cfg, device="cpu", dtype=torch.float32, seed=77)
    hf.save_hf(cfg, local.state_dict(), tmp_path / "weights")
    with tarfile.open(tmp_path / "weights.tar", "w") as tar:
        tar.add(tmp_path / "weights", arcname="weights")
    batch = text_batch(_sequences(4))
    mbs = pack_batch(batch, microbatch_tokens=256, microbatches=2, slots=16)
    want = local.evaluate([to_device(HostMicrobatch(m.tokens, m.targets, m.weights, m.positions, m.cu_seqlens,
                                                    m.max_seqlen), "cpu") for m in mbs])
    with ServiceClient(service.url, token="secret") as svc:
        handle = svc.upload_artifact(tmp_path / "weights.tar").result()
        trainer = svc.create_training_client(
            Model("llama3-tiny", dtype="float32", weights=Weights.artifact(handle.artifact)),
            Optimizer(lr=1e-3, parameter_rounding="nearest"),
            batch=BatchConfig(tokens_per_step=512, microbatch_tokens=256),
            memory=Memory(device_gib=0.53, spill_gib=0.25), resources=Resources(gpus=1, backend="cpu"),
            preparation=Preparation(profiling=ProfilingOptions(enabled=False), calibrate=False,
                                    planning=PlanningOptions(minimum_object_bytes_evict_eligible=1024,
                                                             workers=1)),
            operations=("step", "forward"), timeout=300).result()
        got = trainer.forward(batch).result().loss
        trainer.close()
    assert abs(got - want) < 1e-5 * max(1.0, abs(want))


def test_other_optimizer_components_through_the_service(service):
    with ServiceClient(service.url, token="secret") as svc:
        assert {"adamw@1", "sgd@1", "lion@1"} <= {c["id"] for c in svc.list_components("optimizer").result()}
        trainer = svc.create_training_client(
            Model("llama3-tiny", dtype="float32"),
            Optimizer(id="lion@1", lr=3e-4, beta1=0.9, beta2=0.99, parameter_rounding="nearest"),
            batch=BatchConfig(tokens_per_step=512, microbatch_tokens=256),
            memory=Memory(device_gib=0.53, spill_gib=0.25), resources=Resources(gpus=1, backend="cpu"),
            preparation=Preparation(profiling=ProfilingOptions(enabled=False), calibrate=False,
                                    planning=PlanningOptions(minimum_object_bytes_evict_eligible=1024,
                                                             workers=1)),
            timeout=300).result()
        losses = [trainer.step(text_batch(_sequences(0))).result().loss for _ in range(5)]
        assert losses[-1] < losses[0]
        trainer.close()
        with pytest.raises(Exception) as e:
            svc.describe_training(model=Model("llama3-tiny"), optimizer=Optimizer(id="adagrad@1"),
                                  resources=Resources(backend="cpu")).result()
        assert "adagrad@1" in str(e.value)


def test_node_daemon_routes(service):
    """join -> heartbeat -> queued command delivered on poll until its receipt -> leave."""
    from shadowspill_b200.client.transport import HTTPTransport, TransportError
    t = HTTPTransport(service.url, token=service.node_token)
    inc = t.request("POST", "/v1/nodes/join", {"node_id": "node-x", "info": {"gpus": 8}})[1]["incarnation"]
    assert t.request("POST", "/v1/nodes/heartbeat", {"node_id": "node-x", "incarnation": inc})[1]["ok"]
    cid = service.membership.enqueue("node-x", {"kind": "drain"})
    got = t.request("POST", "/v1/nodes/poll", {"node_id": "node-x", "incarnation": inc})[1]["commands"]
    assert [c["id"] for c in got] == [cid] and got[0]["kind"] == "drain"
    assert t.request("POST", "/v1/nodes/receipt", {"node_id": "node-x", "incarnation": inc, "command": cid,
                                                   "outcome": {"state": "done"}})[1]["ok"]
    assert t.request("POST", "/v1/nodes/poll", {"node_id": "node-x", "incarnation": inc})[1]["commands"] == []
    with pytest.raises(TransportError) as e:          # a stale incarnation is fenced
        t.request("POST", "/v1/nodes/poll", {"node_id": "node-x", "incarnation": "0" * 32})
    assert e.value.status == 410
    with ServiceClient(service.url, token="secret") as svc:
        assert "node-x" in svc.list_hardware().result()["members"]
    assert t.request("POST", "/v1/nodes/leave", {"node_id": "node-x", "incarnation": inc})[1]["ok"]


def test_checkpoint_and_artifact_names_stay_inside_the_service_root(tmp_path):
    """Client-supplied names become single path components: separators, ``..`` and absolute
    paths are refused for checkpoints, sessions and artifacts, and a restore looks only inside
    its own session's directory."""
    from shadowspill_b200.server.service import Server, safe_name
    srv = Server(tmp_path / "root")
    good = srv.checkpoint_directory("sess-1", "after_5.v2")
    assert good == (tmp_path / "root" / "checkpoints" / "sess-1" / "after_5.v2").resolve()
    for bad in ("../../x", "..", ".", "/etc/passwd", "a/b", "", "x y", "a\\b", None):
        with pytest.raises(ValueError):
            srv.checkpoint_directory("sess-1", bad)
        with pytest.raises(ValueError):
            srv.checkpoint_directory(bad, "ok")
        with pytest.raises(ValueError):
            safe_name(bad, "artifact")
    other = tmp_path / "root" / "checkpoints" / "other" / "ck"
    other.mkdir(parents=True)
    with pytest.raises(FileNotFoundError):
        srv.resolve_checkpoint("sess-1", "ck")          # another session's checkpoint
    assert srv.resolve_checkpoint("other", "ck") == str(other.resolve())
    with pytest.raises(ValueError):
        srv.unpack_artifact("../checkpoints")


def test_reference_control_protocol_envelopes(tmp_path):
    """A request that asks for the reference client's control media type gets that protocol's
    envelope: ``service.info`` and ``service.hardware`` records on the connection routes, a
    ``service.error`` record (never a bare JSON body) on failures and on untranslated routes."""
    import json
    import urllib.error
    import urllib.request
    from shadowspill_b200.server.reference_protocol import CONTROL_MEDIA_TYPE
    token = "t" * 40
    with Server(tmp_path / "root", token=token) as srv:
        def ask(path, tok=token, method="GET", body=None):
            req = urllib.request.Request(srv.url + path, method=method, data=body,
                                         headers={"Accept": CONTROL_MEDIA_TYPE, "Authorization": f"Bearer {tok}",
                                                  "Content-Type": CONTROL_MEDIA_TYPE})
            try:
                with urllib.request.urlopen(req) as r:
                    return r.status, r.headers["Content-Type"], json.loads(r.read())
            except urllib.error.HTTPError as e:
                return e.code, e.headers["Content-Type"], json.loads(e.read())
        status, ctype, env = ask("/v1/info")
        assert status == 200 and ctype == CONTROL_MEDIA_TYPE
        assert set(env) == {"version", "kind", "value"} and env["version"] == 1 and env["kind"] == "service.info"
        assert set(env["value"]) == {"server_incarnation", "owner_id"}
        status, ctype, env = ask("/v1/hardware")
        assert status == 200 and env["kind"] == "service.hardware"
        node = env["value"]["nodes"][0]
        assert node["host_available_bytes"] <= node["host_capacity_bytes"] and node["cpu_count"] >= 1
        assert [d["index"] for d in node["devices"]] == list(range(len(node["devices"])))
        status, ctype, env = ask("/v1/info", tok="w" * 40)
        assert status == 401 and ctype == CONTROL_MEDIA_TYPE
        assert env["kind"] == "service.error" and env["value"]["code"] == "unauthenticated"
        status, ctype, env = ask("/v1/training/describe", method="POST", body=b"{}")
        assert status >= 400 and ctype == CONTROL_MEDIA_TYPE and env["kind"] == "service.error"
        status, ctype, env = ask("/v1/components")
        assert status == 501 and env["value"]["code"] == "unsupported" and "/v1/components" in env["value"]["message"]


def test_the_unmodified_reference_client_connects(tmp_path):
    """The reference's own client package (an unmodified copy, when one is present beside the
    baseline) opens a connection to this server, authenticates, reads the service identity and
    lists hardware; a training request is answered with a service error it can decode."""
    import sys
    from pathlib import Path
    ref = Path(__file__).resolve().parents[1] / "baseline" / "_ref"
    if not (ref / "shadowspill_client" / "__init__.py").exists():
        pytest.skip("no copy of the reference client in this checkout")
    sys.path.insert(0, str(ref))
    try:
        import shadowspill_client as rc
        from shadowspill_client.protocol.hardware import HardwareInventory
        token = "k" * 48
        with Server(tmp_path / "root", token=token) as srv:
            client = rc.ServiceClient(srv.url, token=token, timeout=30)
            try:
                assert client.info.owner_id == "local" and client.info.server_incarnation
                inventory = client.list_hardware().result(timeout=30)
                assert isinstance(inventory, HardwareInventory) and len(inventory.nodes) == 1
                with pytest.raises(Exception) as e:
                    client._request("GET", "/v1/components", HardwareInventory)
                assert "unsupported" in str(e.value) or getattr(e.value, "status", 0) == 501
            finally:
                client.close()
    finally:
        sys.path.remove(str(ref))
        for name in [m for m in sys.modules if m == "shadowspill_client" or m.startswith("shadowspill_client.")]:
            del sys.modules[name]


def test_axis_chunks_and_the_graph_frontend_through_the_service(service):
    """``text_chunks@1`` with ``rows`` selects the graph frontend and cuts the layer graphs into row
    chunks; the run trains, and its loss equals the unchunked stage-class run on the same data."""
    from shadowspill_b200.client import BuildOptions

    def run(preparation):
        with ServiceClient(service.url, token="secret") as svc:
            tr = svc.create_training_client(
                Model("llama3-tiny", dtype="float32"), Optimizer(lr=3e-3, parameter_rounding="nearest"),
                batch=BatchConfig(tokens_per_step=512, microbatch_tokens=256),
                memory=Memory(device_gib=0.53, spill_gib=0.25), resources=Resources(gpus=1, backend="cpu"),
                preparation=preparation, timeout=300).result()
            try:
                return [tr.step(text_batch(_sequences(s))).result().loss for s in range(2)]
            finally:
                tr.close()
    common = dict(profiling=ProfilingOptions(enabled=False), calibrate=False,
                  planning=PlanningOptions(minimum_object_bytes_evict_eligible=1024, workers=1))
    whole = run(Preparation(**common))
    cut = run(Preparation(policies=({"id": "shadowspill/text_chunks@1", "config": {"rows": 96}},), **common))
    graph = run(Preparation(build=BuildOptions(frontend="graph"), **common))
    for a, b, c in zip(whole, cut, graph):
        assert abs(a - b) < 1e-4 * max(1.0, abs(a)) and abs(a - c) < 1e-4 * max(1.0, abs(a)), (whole, cut, graph)


def test_a_restarted_service_replays_its_journals(tmp_path):
    """A run that was live when the service process stopped comes back as a read-only record:
    state ``interrupted``, its completed updates, loss history and checkpoint names from the
    journal; requests to it are refused, and a new run resumes from its checkpoint."""
    root = tmp_path / "root"
    common = dict(batch=BatchConfig(tokens_per_step=512, microbatch_tokens=256),
                  memory=Memory(device_gib=0.53, spill_gib=0.25), resources=Resources(gpus=1, backend="cpu"),
                  preparation=Preparation(profiling=ProfilingOptions(enabled=False), calibrate=False,
                                          planning=PlanningOptions(minimum_object_bytes_evict_eligible=1024,
                                                                   workers=1)), timeout=300)
    with Server(root, token="secret") as first:
        with ServiceClient(first.url, token="secret") as svc:
            tr = svc.create_training_client(Model("llama3-tiny", dtype="float32"),
                                            Optimizer(lr=3e-3, parameter_rounding="nearest"), **common).result()
            losses = [tr.step(text_batch(_sequences(s))).result().loss for s in range(2)]
            tr.save_checkpoint("after_two").result()
            session, run = svc.session, tr.run
            # the service goes away with the run still open (no close request)
    with Server(root, token="secret") as second:
        old = second.get_run(session, run)
        info = old.info()
        assert info["state"] == "interrupted" and info["recovered"] and "after_two" in info["error"]
        assert info["boundary"]["completed_updates"] == 2
        assert [round(m["loss"], 5) for m in old.metrics] == [round(x, 5) for x in losses]
        assert list(old.checkpoints) == ["after_two"]
        assert any(r["kind"] == "run_closed" and r["data"]["reason"] == "service restart"
                   for r in second.journal.records())
        import json
        import urllib.error
        import urllib.request
        req = urllib.request.Request(f"{second.url}/v1/runs/{session}/{run}/requests", method="POST",
                                     data=json.dumps({"request_id": "x", "operation": "step"}).encode(),
                                     headers={"Authorization": "Bearer secret", "Content-Type": "application/json"})
        with pytest.raises(urllib.error.HTTPError) as e:
            urllib.request.urlopen(req)
        assert e.value.code == 409 and "interrupted" in e.value.read().decode()
        with ServiceClient(second.url, token="secret") as svc:
            svc.session = session                        # the checkpoint belongs to that session
            again = svc.create_training_client(Model("llama3-tiny", dtype="float32"),
                                               Optimizer(lr=3e-3, parameter_rounding="nearest"),
                                               checkpoint="after_two", **common).result()
            nxt = again.step(text_batch(_sequences(2))).result()
            assert nxt.completed_updates == 3
            again.close()
    with Server(root, token="secret") as third:
        assert third.get_run(session, run).info()["state"] == "interrupted"      # stable across restarts


def test_a_run_prepared_in_separate_processes(service):
    """``Preparation(separate_processes=True)``: the service runs the four preparation phases as
    fresh processes, the worker opens their bundle, and training proceeds as usual."""
    with ServiceClient(service.url, token="secret") as svc:
        tr = svc.create_training_client(
            Model("llama3-tiny", dtype="float32"), Optimizer(lr=3e-3, parameter_rounding="nearest"),
            batch=BatchConfig(tokens_per_step=512, microbatch_tokens=256),
            memory=Memory(device_gib=0.53, spill_gib=0.25), resources=Resources(gpus=1, backend="cpu"),
            preparation=Preparation(profiling=ProfilingOptions(enabled=False), calibrate=False,
                                    separate_processes=True,
                                    planning=PlanningOptions(minimum_object_bytes_evict_eligible=1024, workers=1)),
            timeout=300).result()
        try:
            progress = " ".join(svc.get_progress(tr.run).result()["lines"])
            assert "separate processes" in progress and "prepared bundle" in progress
            losses = [tr.step(text_batch(_sequences(s))).result().loss for s in range(3)]
            assert losses[-1] < losses[0] + 0.05
        finally:
            tr.close()
    live = service.get_run(svc.session, tr.run)
    assert (live.dir / "preparation" / "job.json").exists()


def test_prepared_plans_are_exported_and_start_a_run_elsewhere(service, tmp_path):
    """``PlansHandle``: summary pages and a name for the plans of a prepared run; the bundle leaves
    the service as a file, comes back as an artifact (as it would on another service), and a new
    run that names it skips build, profile and plan."""
    common = dict(batch=BatchConfig(tokens_per_step=512, microbatch_tokens=256),
                  memory=Memory(device_gib=0.53, spill_gib=0.25), resources=Resources(gpus=1, backend="cpu"),
                  preparation=Preparation(profiling=ProfilingOptions(enabled=False), calibrate=False,
                                          planning=PlanningOptions(minimum_object_bytes_evict_eligible=1024,
                                                                   workers=1)))
    model, opt = Model("llama3-tiny", dtype="float32"), Optimizer(lr=3e-3, parameter_rounding="nearest")
    with ServiceClient(service.url, token="secret") as svc:
        prepared = svc.prepare_training(model=model, optimizer=opt, **common).result()
        plans = svc.plans_of(prepared["run"])
        page = plans.summary().result()
        assert page["plans"][0]["operation"] == "step" and page["plans"][0]["duration_seconds"] > 0
        assert plans.save(name="baseline").result()["plans"] == {"baseline": "step"}
        found = plans.named("baseline").result()
        assert found["operation"] == "step" and found["plan"]["duration_seconds"] == page["plans"][0]["duration_seconds"]
        with pytest.raises(TransportError):
            plans.named("never-saved").result()
        with pytest.raises(ValueError):
            plans.save(name="a/b")
        bundle = plans.export(tmp_path / "plans.tar").result()
        assert bundle.stat().st_size > 1000
    with ServiceClient(service.url, token="secret") as other:          # another session: nothing shared but the file
        imported = other.import_plans(bundle).result()
        assert imported.run is None and imported.create_arguments() == {"plans_artifact": imported.artifact.artifact}
        with pytest.raises(ValueError):
            imported.summary()
        screen = io.StringIO()
        tr = other.create_training_client(model, opt, plans=imported, timeout=300, progress=screen, **common).result()
        shown = screen.getvalue()
        assert "- Preparing" in shown and "- Ready" in shown and "taken from artifact" in shown
        try:
            fut = tr.step(text_batch(_sequences(1)))
            assert fut.operation == "step" and len(fut.request_id) == 32
            assert fut.accepted().result(60)["request_id"] == fut.request_id
            assert fut.result(60).request_id == fut.request_id
            again = tr.lookup_request(fut.request_id)               # after a lost reply: ask, do not resubmit
            assert again.loss == fut.result().loss and again.completed_updates == fut.result().completed_updates
            with pytest.raises(TransportError):
                tr.lookup_request("0" * 32)
            progress = " ".join(other.get_progress(tr.run).result()["lines"])
            assert "taken from artifact" in progress and "build, profile and plan skipped" in progress
            assert tr.step(text_batch(_sequences(0))).result().loss > 0
        finally:
            tr.close()


def test_an_extension_package_adds_components(tmp_path):
    """A service started with an extension package lists its components under the package's name,
    trains the model it defines, and resolves its policy preset; ids that exist are not replaced,
    and a broken package stops the start with its name."""
    import sys
    from pathlib import Path
    from shadowspill_b200.client import Policy
    from shadowspill_b200.training.extensions import ExtensionError
    sys.path.insert(0, str(Path(__file__).resolve().parents[1]))
    name = "examples.extensions.custom_training"
    with Server(tmp_path / "svc", token="secret", extensions=[name]) as srv:
        assert srv.extensions[name] == ["model:acme/llama3-wide@1", "policy:acme/short_rows@1"]
        with ServiceClient(srv.url, token="secret") as svc:
            listed = {c["id"]: c for c in svc.list_components().result()}
            assert listed["acme/llama3-wide@1"]["source"]["distribution"] == name
            assert listed["llama3-tiny@1"]["source"]["distribution"] == "shadowspill_b200"
            tr = svc.create_training_client(
                Model("acme/llama3-wide@1", dtype="float32"), Optimizer(lr=3e-3, parameter_rounding="nearest"),
                batch=BatchConfig(tokens_per_step=512, microbatch_tokens=256),
                memory=Memory(device_gib=0.53, spill_gib=0.25), resources=Resources(gpus=1, backend="cpu"),
                preparation=Preparation(profiling=ProfilingOptions(enabled=False), calibrate=False,
                                        policies=(Policy("acme/short_rows@1", {"rows": 64}),),
                                        planning=PlanningOptions(minimum_object_bytes_evict_eligible=1024, workers=1)),
                timeout=300).result()
            try:
                assert tr.info["provenance"]["model"] == "catalog acme/llama3-wide@1"
                assert tr.info["provenance"]["policy acme/short_rows@1"] == "preset of shadowspill/text_chunks@1"
                live = srv.get_run(svc.session, tr.run)
                from shadowspill_b200.models.config import preset
                assert live.resolved.cfg.d_ff == 2 * preset("llama3-tiny").d_ff
                assert live.resolved.setups[0]["axis_chunk_rows"] == 64 and live.resolved.setups[0]["frontend"] == "graph"
                assert tr.step(text_batch(_sequences(0))).result().loss > 0
            finally:
                tr.close()
    with pytest.raises(ExtensionError, match="cannot be imported"):
        Server(tmp_path / "bad", token="secret", extensions=["no_such_extension_module"])
    with pytest.raises(ExtensionError, match="already registered"):
        Server(tmp_path / "twice", token="secret", extensions=[name, name])


def test_norm_observations_reach_the_client_and_the_metric_journal(service):
    """``Execution(observe_norms=True)``: every update's result and journal record carry the norms."""
    from shadowspill_b200.client import Execution
    with ServiceClient(service.url, token="secret") as svc:
        tr = svc.create_training_client(
            Model("llama3-tiny", dtype="float32"), Optimizer(lr=3e-3, parameter_rounding="nearest"),
            batch=BatchConfig(tokens_per_step=512, microbatch_tokens=256),
            memory=Memory(device_gib=0.53, spill_gib=0.25), resources=Resources(gpus=1, backend="cpu"),
            execution=Execution(observe_norms=True),
            preparation=Preparation(profiling=ProfilingOptions(enabled=False), calibrate=False,
                                    planning=PlanningOptions(minimum_object_bytes_evict_eligible=1024, workers=1)),
            timeout=300).result()
        try:
            res = tr.step(text_batch(_sequences(0))).result()
            assert res.metrics["grad_norm"] > 0 and res.metrics["param_norm"] > 1
            xs, ys = tr.metrics.series("grad_norm")
            assert ys == [res.metrics["grad_norm"]]
        finally:
            tr.close()


def test_the_latent_attention_family_trains_through_the_service(service):
    """``glm53-tiny`` by its catalog name: the builder takes the graph frontend for it whatever the
    build option says, layers that share picks become one stage, and steps, accumulation, a forward
    and a checkpoint go through the public API."""
    with ServiceClient(service.url, token="secret") as svc:
        preview = svc.describe_training(model=Model("glm53-tiny", dtype="float32"),
                                        batch=BatchConfig(tokens_per_step=512, microbatch_tokens=256),
                                        memory=Memory(device_gib=0.6, spill_gib=0.25),
                                        resources=Resources(gpus=1, backend="cpu")).result()
        assert preview["parameters"] > 1_000_000
        tr = svc.create_training_client(
            Model("glm53-tiny", dtype="float32"), Optimizer(lr=3e-3, parameter_rounding="nearest"),
            batch=BatchConfig(tokens_per_step=512, microbatch_tokens=256),
            memory=Memory(device_gib=0.6, spill_gib=0.25), resources=Resources(gpus=1, backend="cpu"),
            preparation=Preparation(profiling=ProfilingOptions(enabled=False), calibrate=False,
                                    planning=PlanningOptions(minimum_object_bytes_evict_eligible=1024, workers=1)),
            operations=("step", "forward", "forward_backward", "optim_step"), timeout=300).result()
        try:
            seqs = lambda s: [np.asarray(x) % 128 for x in _sequences(s)]
            losses = [tr.step(text_batch(seqs(s % 2))).result().loss for s in range(4)]
            assert losses[2] < losses[0] and losses[3] < losses[1]
            tr.forward_backward(text_batch(seqs(2))).result()
            assert tr.optim_step().result().completed_updates == 5
            scored = tr.forward(text_batch(seqs(0))).result()
            assert 0 < scored.loss < losses[0] and len(scored.outputs["per_datum"]) == len(seqs(0))
            assert tr.save_checkpoint("glm").result().outputs["checkpoint"] == "glm"
        finally:
            tr.close()


def test_a_service_is_reached_through_an_owned_ssh_forward(service, monkeypatch):
    """``ServiceClient(ssh=SSH(...))`` starts the forward in its own process group, talks to the
    service over it and ends it on close; an ssh that exits says why. (A stand-in plays OpenSSH.)"""
    import urllib.parse
    from pathlib import Path
    from shadowspill_b200.client import SSH, SSHTunnel
    monkeypatch.setenv("SHADOWSPILL_SSH", str(Path(__file__).with_name("_fake_ssh.py")))
    port = urllib.parse.urlparse(service.url).port
    with ServiceClient(token="secret", ssh=SSH("training-host", port)) as svc:
        assert svc.tunnel.url != service.url and svc.info
        assert isinstance(svc.list_hardware().result(), dict)
        proc = svc.tunnel.proc
        assert proc.poll() is None
    assert proc.poll() is not None and svc.tunnel.closed            # the forward ended with the client
    with pytest.raises(ConnectionError, match="No route to host"):
        SSHTunnel(SSH("unreachable", port), timeout=10).open()
    with pytest.raises(ValueError):
        ServiceClient(service.url, token="secret", ssh=SSH("training-host", port))
    with pytest.raises(ValueError):
        SSH("-oProxyCommand=evil", port)
    cmd = SSH("box", 8123, jump_host="bastion", ssh_port=2222, config_file="/tmp/cfg").command(4000)
    assert cmd[-2:] == ["--", "box"] and "-J" in cmd and "127.0.0.1:4000:127.0.0.1:8123" in cmd and "-F" in cmd


def test_microbatch_groups_through_the_service(service):
    """Two sharded ranks, four microbatches per rank in two sweeps (``BuildOptions(walks=("breadth/2",))``):
    the run comes up with that walk and trains."""
    from shadowspill_b200.client import BuildOptions, data_parallel
    with ServiceClient(service.url, token="secret") as svc:
        tr = svc.create_training_client(
            Model("llama3-tiny", dtype="float32"), Optimizer(lr=3e-3, parameter_rounding="nearest"),
            batch=BatchConfig(tokens_per_step=1024, microbatch_tokens=256),
            memory=Memory(device_gib=0.53, spill_gib=0.25), resources=Resources(gpus=2, backend="cpu"),
            parallelism=data_parallel(2, min_shard_bytes=0),
            preparation=Preparation(build=BuildOptions(walks=("breadth/2",)),
                                    profiling=ProfilingOptions(enabled=False), calibrate=False,
                                    planning=PlanningOptions(minimum_object_bytes_evict_eligible=1024, workers=1)),
            operations=("step", "forward"), timeout=600).result()
        try:
            assert tr.info["workers"] == 2 and "groups2" in tr.info["plan_summary"]["ordering"]
            losses = [tr.step(text_batch(_sequences(0, n=48))).result().loss for _ in range(4)]
            assert losses[-1] < losses[0]
        finally:
            tr.close()


def test_the_read_only_command_line(service, capsys, tmp_path):
    """``python -m shadowspill_b200.client``: info, components, a run's record, its log and its metric
    journal (printed or exported), all without touching the run."""
    import json
    from shadowspill_b200.client.__main__ import main
    common = ["--url", service.url, "--token", "secret"]
    assert main(common + ["info"]) == 0 and json.loads(capsys.readouterr().out)
    assert main(common + ["components", "--kind", "optimizer"]) == 0
    listed = capsys.readouterr().out
    assert "adamw@1" in listed and "shadowspill_b200" in listed and "cross_entropy" not in listed
    with ServiceClient(service.url, token="secret") as svc:
        tr = svc.create_training_client(
            Model("llama3-tiny", dtype="float32"), Optimizer(lr=3e-3, parameter_rounding="nearest"),
            batch=BatchConfig(tokens_per_step=512, microbatch_tokens=256),
            memory=Memory(device_gib=0.53, spill_gib=0.25), resources=Resources(gpus=1, backend="cpu"),
            preparation=Preparation(profiling=ProfilingOptions(enabled=False), calibrate=False,
                                    planning=PlanningOptions(minimum_object_bytes_evict_eligible=1024, workers=1)),
            timeout=300).result()
        try:
            tr.step(text_batch(_sequences(0))).result()
            where = [svc.session, tr.run]
            assert main(common + ["run"] + where) == 0
            assert json.loads(capsys.readouterr().out)["state"] == "ready"
            assert main(common + ["progress"] + where) == 0 and "ready" in capsys.readouterr().out
            assert main(common + ["metrics"] + where) == 0
            rows = [json.loads(ln) for ln in capsys.readouterr().out.splitlines() if ln.strip()]
            assert rows and rows[0]["operation"] == "step" and rows[0]["loss"] > 0
            target = tmp_path / "m.jsonl"
            assert main(common + ["metrics"] + where + ["--jsonl", str(target)]) == 0
            assert len(target.read_text().splitlines()) == len(rows)
        finally:
            tr.close()
