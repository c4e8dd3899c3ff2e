"""Checkpoint archive format, round trip and resume equivalence (CPU, mock backend)."""
import json
import sys
import tarfile

import pytest
import torch

sys.path.insert(0, __file__.rsplit("/", 1)[0])
from test_executor_cpu import _batches, _setup  # noqa: E402

from shadowspill_b200.checkpoint import (CheckpointError, export_weights, load_checkpoint,
                                         read_manifest, save_checkpoint)
from shadowspill_b200.execution.executor import Executor, Hyperparameters
from shadowspill_b200.native import Blake3


def test_blake3_known_vectors():
    assert Blake3(b"").hexdigest() == \
        "af1349b9f5f9a1a6a0404dea36dcc9499bcb25c9adc112b7cc9a93cae41f3262"
    assert Blake3(bytes([0])).hexdigest() == \
        "2d3adedff11b61f14c886e35afa036736dcd87a74d27b5c1510225d0f592e213"
    data = bytes(i % 251 for i in range(70000))
    h = Blake3()
    for i in range(0, len(data), 1000):
        h.update(data[i:i + 1000])
    assert h.hexdigest() == Blake3(data).hexdigest()
    try:
        import blake3
    except ImportError:
        return
    for n in (1023, 1024, 1025, 4097, 70000):
        assert blake3.blake3(data[:n]).hexdigest() == Blake3(data[:n]).hexdigest()


def test_archive_layout_and_resume(tmp_path):
    cfg, plan, desc = _setup()
    hyper = Hyperparameters(lr=3e-3)
    a = Executor(plan, desc, device="cpu", seed=5, hyper=hyper)
    a.initialize()
    for s in range(2):
        a.run(_batches(cfg, s))
    path = save_checkpoint(a, tmp_path / "ckpt", metadata={"note": "after two updates"})
    # ---- the TAR layout
    with tarfile.open(path, "r:") as tar:
        names = tar.getnames()
    assert names[-2:] == ["manifest.json", "manifest.blake3"]
    assert names[0] == "tensors/0" and all(n.startswith("tensors/") for n in names[:-2])
    m = read_manifest(path)
    assert m["format"] == "shadowspill.checkpoint" and m["version"] == 1
    assert m["metadata"]["completed_updates"] == 2 and m["weights"] == "master"
    e = m["tensors"][0]
    # the reference's entry schema: str(torch.dtype), no region keys for a whole storage
    assert set(e) == {"name", "shape", "dtype", "stride", "storage_offset", "storage_elements",
                      "member", "bytes", "blake3"}
    assert e["dtype"] == "torch.float32" and m["additional_programs"] == {}
    assert "logical_ranks" not in m
    streams = m["metadata"]["random_streams"]
    assert {s["identity"]["component_path"][2] for s in streams} == {"python", "numpy", "torch"}
    assert path.stat().st_size % 512 == 0
    # ---- resume: a fresh executor continues exactly where the first one goes next
    b = Executor(plan, desc, device="cpu", seed=99, hyper=hyper)
    b.initialize()
    meta = load_checkpoint(b, tmp_path / "ckpt")
    assert meta["note"] == "after two updates" and b.completed_updates == 2
    la, lb = a.run(_batches(cfg, 2)).loss, b.run(_batches(cfg, 2)).loss
    assert la == lb
    sa, sb = a.state_dict(), b.state_dict()
    assert all(torch.equal(sa[k], sb[k]) for k in sa)
    w = export_weights(tmp_path / "ckpt")
    assert set(w) == {k for k in sa if not k.startswith("exp_avg")}
    a.close(); b.close()


def test_corruption_is_detected(tmp_path):
    cfg, plan, desc = _setup()
    ex = Executor(plan, desc, device="cpu", seed=1)
    ex.initialize()
    path = save_checkpoint(ex, tmp_path / "c")
    raw = bytearray(path.read_bytes())
    raw[512 + 100] ^= 0xFF                      # inside the first tensor member
    path.write_bytes(bytes(raw))
    with pytest.raises(CheckpointError):
        load_checkpoint(ex, tmp_path / "c")
    ex.close()


def test_hugging_face_names_round_trip(tmp_path):
    import torch
    from shadowspill_b200.checkpoint import hf
    from shadowspill_b200.execution.resident import ResidentTrainer
    from shadowspill_b200.models.config import preset
    for name in ("llama3-tiny", "qwen3-tiny", "olmoe-tiny", "qwen3moe-tiny", "qwen35-tiny",
                 "qwen35moe-tiny"):
        cfg = preset(name)
        assert hf.supported(cfg)
        tr = ResidentTrainer(cfg, device="cpu", dtype=torch.float32, seed=1)
        state = tr.state_dict()
        named = hf.to_hf(cfg, state)
        pre = "model.language_model." if name.startswith("qwen35") else "model."
        attn = next(i for i in range(cfg.n_layers) if cfg.layer_kind(i) == "attention")
        q = named[f"{pre}layers.{attn}.self_attn.q_proj.weight"]
        gated = 2 if cfg.gated_attention else 1
        assert q.shape == (gated * cfg.n_heads * cfg.head_dim, cfg.d_model)
        if cfg.gated_attention:
            # per-head interleave: rows [q_0, gate_0, q_1, ...]; ours keeps all q, then all gates
            ours = state[f"layer{attn}.wq"]
            dh = cfg.head_dim
            assert torch.equal(q[:dh], ours[:dh])
            assert torch.equal(q[dh:2 * dh], ours[cfg.n_heads * dh:cfg.n_heads * dh + dh])
            assert torch.equal(q[2 * dh:3 * dh], ours[dh:2 * dh])
        if cfg.full_attention_interval:
            la = f"{pre}layers.0.linear_attn."
            kw, vw = cfg.dn_qk_heads * cfg.dn_head_dim, cfg.dn_v_heads * cfg.dn_head_dim
            assert named[la + "in_proj_qkv.weight"].shape == (2 * kw + vw, cfg.d_model)
            assert named[la + "in_proj_z.weight"].shape == (vw, cfg.d_model)
            assert named[la + "in_proj_a.weight"].shape == (cfg.dn_v_heads, cfg.d_model)
            assert named[la + "conv1d.weight"].shape == (2 * kw + vw, 1, cfg.dn_conv_width)
        if cfg.family == "qwen35moe":
            assert named[f"{pre}layers.1.mlp.experts.gate_up_proj"].shape == \
                (cfg.n_experts, 2 * cfg.d_expert, cfg.d_model)
            if cfg.d_shared_expert:
                assert named[f"{pre}layers.1.mlp.shared_expert_gate.weight"].shape == (1, cfg.d_model)
        elif cfg.is_moe:
            assert f"{pre}layers.1.mlp.experts.{cfg.n_experts - 1}.down_proj.weight" in named
        else:
            assert named[f"{pre}layers.1.mlp.up_proj.weight"].shape == (cfg.d_ff, cfg.d_model)
        assert ("lm_head.weight" in named) == (not cfg.tied_embeddings)
        hf.save_hf(cfg, state, tmp_path / name)
        back = hf.load_hf(cfg, tmp_path / name)
        assert set(back) == set(state)
        for k, v in state.items():
            assert torch.equal(back[k], v), k
    # the vision tower and the extra prediction head of a full checkpoint are skipped;
    # anything else without a destination is an error
    cfg = preset("qwen35-tiny")
    state = ResidentTrainer(cfg, device="cpu", dtype=torch.float32, seed=1).state_dict()
    named = hf.to_hf(cfg, state)
    named["model.visual.patch_embed.weight"] = torch.zeros(2)
    named["mtp.fc.weight"] = torch.zeros(2)
    assert set(hf.from_hf(cfg, named)) == set(state)
    named["model.language_model.unknown"] = torch.zeros(2)
    import pytest
    with pytest.raises(ValueError):
        hf.from_hf(cfg, named)


def test_expert_banks_are_recorded_in_global_coordinates():
    """Under expert parallelism every rank holds its own rows of each bank; the checkpoint entries
    of all ranks must tile the whole bank so that a run with another rank count can load it."""
    import math
    import types
    import torch
    from shadowspill_b200.checkpoint.save import state_entries
    from shadowspill_b200.models.config import preset
    from shadowspill_b200.models.decoder import build_stages
    cfg = preset("olmoe-tiny")
    per_rank = []
    for rank in range(2):
        stages = build_stages(cfg, expert_parallel=(2, rank))
        obj = {f"{st.name}.{k}": 1 for st in stages for k in ("weights", "exp_avg", "exp_avg_sq")}
        fake = types.SimpleNamespace(world=2, rank=rank, stages=stages, _obj=obj,
                                     desc=types.SimpleNamespace(dtype=torch.float32))
        per_rank.append({e["name"]: e for e in state_entries(fake)})
    name = "layer0.w13"
    a, b = per_rank[0][name], per_rank[1][name]
    assert a["shape"] == b["shape"] == [cfg.n_experts, 2 * cfg.d_expert, cfg.d_model]
    total = math.prod(a["shape"])
    assert a["storage_elements"] == total
    from shadowspill_b200.checkpoint.save import entry_region
    assert entry_region(a) == (0, total // 2) and entry_region(b) == (total // 2, total // 2)
    assert (b["region_offset"], b["region_elements"]) == (total // 2, total // 2)
    # dense tensors of the same stage are still cut into flat shards
    d0, d1 = (entry_region(per_rank[r]["layer0.wq"]) for r in range(2))
    assert d0[0] == 0 and d1[0] == d0[1]
    assert d0[1] + d1[1] == per_rank[0]["layer0.wq"]["storage_elements"]


def test_master_copies_travel_with_the_checkpoint(tmp_path):
    """A bf16 run with fp32 master copies resumes bit for bit: the masters are state."""
    from shadowspill_b200.communication.info import CommunicationInfo
    from shadowspill_b200.frontend.capture import BatchGeometry, StepDataOrdering, build_step
    from shadowspill_b200.models.config import preset
    from shadowspill_b200.planning.plan import MemoryBudgets, SearchOptions, plan_program
    cfg = preset("llama3-tiny")
    geo = BatchGeometry(microbatch_tokens=256, n_microbatches=2, slots=16, mean_seqlen=64)

    def make():
        prog, desc = build_step(cfg, geo, StepDataOrdering(), dtype=torch.bfloat16, master_weights=True)
        plan = plan_program(prog, MemoryBudgets(32 << 20, 64 << 20, headroom_bytes=0), CommunicationInfo(),
                            SearchOptions(minimum_object_bytes_evict_eligible=1024, workers=1))
        return Executor(plan, desc, device="cpu", seed=5, hyper=Hyperparameters(lr=1e-4),
                        stochastic_rounding=False)
    a = make()
    a.initialize()
    for s in range(3):
        a.run(_batches(cfg, s))
    save_checkpoint(a, tmp_path / "ck")
    names = {e["name"] for e in read_manifest(tmp_path / "ck" / "rank0.tar")["tensors"]}
    # the masters are saved, the bf16 copies are derived from them on load
    assert "master.layer0.wqkv" in names and "exp_avg.layer0.wqkv" in names
    assert "layer0.wqkv" not in names
    assert "layer0.wqkv" in read_manifest(tmp_path / "ck" / "rank0.tar")["derived_tensors"]
    want = [a.run(_batches(cfg, s)).loss for s in (3, 4)]
    state = a.state_dict()
    a.close()
    b = make()
    b.initialize(seed=99)
    load_checkpoint(b, tmp_path / "ck")
    assert [b.run(_batches(cfg, s)).loss for s in (3, 4)] == want
    for k, v in b.state_dict().items():
        assert torch.equal(v, state[k]), k
    b.close()
    assert not any(k.startswith("master.") for k in export_weights(tmp_path / "ck"))


def test_reference_geometry_entries_load(tmp_path):
    """An archive whose entries carry exactly the reference's geometry keys (``torch.``-prefixed
    dtype, optional region_offset / region_elements, no ``region``, no ``logical_ranks``) loads."""
    from shadowspill_b200.checkpoint.archive import FORMAT, VERSION, ArchiveWriter
    from shadowspill_b200.checkpoint.save import state_entries, state_identity
    cfg, plan, desc = _setup()
    a = Executor(plan, desc, device="cpu", seed=5)
    a.initialize()
    a.run(_batches(cfg, 0))
    want = a.state_dict()
    views = dict(a.named_tensors(writable=False))
    w = ArchiveWriter(tmp_path / "ref" / "rank0.tar")
    entries = []
    for e in state_entries(a):
        flat = views[e["name"]].reshape(-1)
        entry = {"name": e["name"], "shape": e["shape"], "dtype": str(flat.dtype),
                 "stride": e["stride"], "storage_offset": 0, "storage_elements": flat.numel()}
        entries.append(entry)
        w.add_tensor(entry, flat.view(torch.uint8).numpy())
    w.finish({"format": FORMAT, "version": VERSION, "byteorder": sys.byteorder,
              "state": state_identity(entries, 1), "program": "0" * 64, "logical_rank": 0,
              "additional_programs": {"forward": "1" * 64}, "metadata": {"completed_updates": 1},
              "frozen_state_id": None, "omitted_parameters": [], "weights": "master",
              "derived_tensors": [], "gathered_tensors": [], "retained_weight_copies": []})
    b = Executor(plan, desc, device="cpu", seed=77)
    b.initialize()
    load_checkpoint(b, tmp_path / "ref")
    assert b.completed_updates == 1
    for k, v in b.state_dict().items():
        assert torch.equal(v, want[k]), k
    a.close(); b.close()


def test_frozen_base_is_omitted_and_generators_resume(tmp_path):
    """With a ``frozen_state_id`` a LoRA checkpoint holds only the adapters and their moments; it
    loads only under the same id, and the default generators continue where they were saved."""
    import random

    import numpy as np
    from shadowspill_b200.communication.info import CommunicationInfo
    from shadowspill_b200.frontend.capture import BatchGeometry, StepDataOrdering, build_step
    from shadowspill_b200.models.config import preset
    from shadowspill_b200.models.lora import LoRAConfig
    from shadowspill_b200.planning.plan import MemoryBudgets, SearchOptions, plan_program
    cfg = preset("llama3-tiny")
    geo = BatchGeometry(microbatch_tokens=256, n_microbatches=2, slots=16, mean_seqlen=64)

    def make(seed):
        prog, desc = build_step(cfg, geo, StepDataOrdering(), dtype=torch.float32, lora=LoRAConfig(rank=8))
        plan = plan_program(prog, MemoryBudgets(64 << 20, 128 << 20, headroom_bytes=0), CommunicationInfo(),
                            SearchOptions(minimum_object_bytes_evict_eligible=1024, workers=1))
        ex = Executor(plan, desc, device="cpu", seed=seed, hyper=Hyperparameters(lr=1e-3))
        ex.initialize()
        return ex
    a = make(5)
    a.run(_batches(cfg, 0))
    full = save_checkpoint(a, tmp_path / "full")
    slim = save_checkpoint(a, tmp_path / "slim", frozen_state_id="base-v1")
    m = read_manifest(slim)
    names = {e["name"] for e in m["tensors"]}
    assert m["frozen_state_id"] == "base-v1" and "embed.embed" in m["omitted_parameters"]
    assert not names & set(m["omitted_parameters"]) and any("lora" in n for n in names)
    assert slim.stat().st_size < full.stat().st_size / 4
    draws = (random.random(), float(np.random.rand()), float(torch.rand(1)))
    b = make(5)                      # same seed = same frozen base
    with pytest.raises(CheckpointError):
        load_checkpoint(b, tmp_path / "slim")
    with pytest.raises(CheckpointError):
        load_checkpoint(b, tmp_path / "slim", frozen_state_id="another")
    load_checkpoint(b, tmp_path / "slim", frozen_state_id="base-v1")
    assert (random.random(), float(np.random.rand()), float(torch.rand(1))) == draws
    sa, sb = a.state_dict(), b.state_dict()
    assert all(torch.equal(sa[k], sb[k]) for k in sa)
    a.close(); b.close()


def test_latent_attention_family_round_trips_through_hugging_face_names(tmp_path):
    """GLM 5.3 is exported in stages of several layers: each stage parameter finds its layer's
    checkpoint name through the module path the export recorded, and the round trip is exact."""
    import torch
    from shadowspill_b200.checkpoint import hf
    from shadowspill_b200.frontend.graph_stage import build_graph_stages
    from shadowspill_b200.models.config import preset
    cfg = preset("glm53-tiny")
    assert hf.supported(cfg) and hf.hf_config(cfg)["model_type"] == "glm_moe_dsa"
    stages = build_graph_stages(cfg, 256, 16, torch.float32)
    gen = torch.Generator().manual_seed(0)
    state = {f"{st.name}.{p.name}": torch.randn(p.shape, generator=gen) for st in stages for p in st.params}
    named = hf.to_hf(cfg, state, stages)
    c = cfg
    assert named["model.layers.1.self_attn.kv_b_proj.weight"].shape == \
        (c.n_heads * (c.qk_nope_head_dim + c.v_head_dim), c.kv_lora_rank)
    assert "model.layers.0.self_attn.indexer.wq_b.weight" in named          # layer 0 owns an indexer
    assert "model.layers.1.self_attn.indexer.wq_b.weight" not in named      # layer 1 shares its picks
    assert named["model.layers.2.self_attn.indexer.k_norm.bias"].shape == (c.index_head_dim,)
    assert named["model.layers.0.mlp.up_proj.weight"].shape == (c.d_ff, c.d_model)             # dense first layer
    assert named["model.layers.3.mlp.gate.e_score_correction_bias"].shape == (c.n_experts,)
    assert named[f"model.layers.1.mlp.experts.{c.n_experts - 1}.down_proj.weight"].shape == (c.d_model, c.d_expert)
    assert named["model.layers.2.mlp.shared_experts.gate_proj.weight"].shape == (c.d_shared_expert, c.d_model)
    # the second layer of the first group is stored under that layer's own number
    assert torch.equal(named["model.layers.1.self_attn.o_proj.weight"], state[f"{stages[1].name}.members_1_wo"])
    hf.save_hf(cfg, state, tmp_path / "glm", stages)
    back = hf.load_hf(cfg, tmp_path / "glm")
    assert set(back) == set(state)
    assert all(torch.equal(back[k], v) for k, v in state.items())


def test_hugging_face_checkpoints_load_one_stage_at_a_time(tmp_path):
    """``stream_hf`` reads a sharded checkpoint stage by stage and gives what ``load_hf`` gives;
    a tensor without a destination is still an error, found once everything else was read."""
    import json
    import pytest
    import torch
    from safetensors.torch import save_file
    from shadowspill_b200.checkpoint import hf
    from shadowspill_b200.execution.resident import ResidentTrainer
    from shadowspill_b200.models.config import preset
    cfg = preset("qwen35moe-tiny")
    state = ResidentTrainer(cfg, device="cpu", dtype=torch.float32, seed=3).state_dict()
    state = {k: v for k, v in state.items() if not k.startswith("exp_avg")}
    named = hf.to_hf(cfg, state)
    keys = sorted(named)
    d = tmp_path / "sharded"
    d.mkdir()
    for i in range(3):                                        # three shards, interleaved names
        save_file({k: named[k].contiguous() for k in keys[i::3]}, str(d / f"model-{i:05d}-of-00003.safetensors"))
    (d / "config.json").write_text(json.dumps(hf.hf_config(cfg)))
    whole = hf.load_hf(cfg, d)
    seen = {}
    order = []
    for stage, part in hf.stream_hf(cfg, d):
        order.append(stage)
        assert all(k.startswith(stage + ".") for k in part)
        seen.update(part)
    assert order[0] == "embed" and order[-1] == "head" and len(order) == cfg.n_layers + 2
    assert set(seen) == set(whole) == set(state)
    assert all(torch.equal(seen[k], whole[k]) and torch.equal(seen[k], state[k]) for k in state)
    save_file({"model.language_model.stray": torch.zeros(2)}, str(d / "model-extra.safetensors"))
    with pytest.raises(ValueError, match="no destination"):
        list(hf.stream_hf(cfg, d))
