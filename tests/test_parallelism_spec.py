"""Ownership declarations: validation, selector precedence, per-rank resolution."""
import pytest

from shadowspill_b200.client import parallelism as client_par
from shadowspill_b200.parallelism.spec import (Parallelism, ParameterStorage, Replicated, Sharded,
                                               data_parallel, expert_parallel, from_client_record)


def test_data_parallel_shards_all_state_and_keeps_small_tensors_whole():
    p = data_parallel(4)
    big = p.resolve("layer3.wqkv", rank=2, nbytes=64 << 20)
    assert big.storage_group == (0, 1, 2, 3) and big.storage_index == 2
    assert big.needs_gather() and big.gradient_reduction() == "reduce_scatter"
    assert big.compute_shards == 1
    small = p.resolve("layer3.attn_norm", rank=2, nbytes=8192)
    assert not small.needs_gather() and small.gradient_reduction() == "all_reduce"


def test_replicas_repeat_the_layout_at_rank_offsets():
    p = data_parallel(2, replicas=3)
    assert p.world_size == 6
    r = p.resolve("w", rank=5, nbytes=1 << 30)
    assert r.storage_group == (4, 5) and r.storage_index == 1
    with pytest.raises(ValueError):
        p.resolve("w", rank=6)


def test_expert_parallel_shards_banks_locally_and_replicates_dense_parts():
    p = expert_parallel(4, n_experts=64, top_k=8)
    bank = p.resolve("layer0.experts.w13", rank=3, nbytes=1 << 30)
    assert isinstance(bank.placement, Sharded) and bank.compute_shards == 4 and bank.compute_index == 3
    assert bank.storage_group == (3,) and bank.gradient_reduction() == "none"
    dense = p.resolve("layer0.wqkv", rank=3, nbytes=1 << 30)
    assert isinstance(dense.placement, Replicated)
    assert dense.storage.weights == "replicated" and dense.storage.optimizer == "sharded"
    assert dense.gradient_reduction() == "all_reduce" and dense.storage_shards("optimizer") == 4
    with pytest.raises(ValueError):
        expert_parallel(3, n_experts=64, top_k=8)
    with pytest.raises(ValueError):
        expert_parallel(4, n_experts=64, top_k=33)


def test_exact_selector_beats_pattern_and_longer_pattern_beats_shorter():
    p = Parallelism(2, parameter_storage={
        "layer*": ParameterStorage(weights="replicated"),
        "layer1.*": ParameterStorage(gradients="replicated"),
        "layer1.w2": ParameterStorage(optimizer="sharded", weights="sharded")})
    assert p.resolve("layer0.w2", 0, 1 << 30).storage.weights == "replicated"
    r = p.resolve("layer1.w13", 0, 1 << 30).storage
    assert (r.weights, r.gradients) == ("sharded", "replicated")      # inherits the default weights
    assert p.resolve("layer1.w2", 0, 1 << 30).storage.weights == "sharded"


def test_validation_and_round_trip():
    with pytest.raises(ValueError):
        Parallelism(4, groups={"halves": ((0, 1), (2,))})              # rank 3 uncovered
    with pytest.raises(ValueError):
        Parallelism(2, parameter_placements={"x": Sharded("nope")})
    with pytest.raises(TypeError):
        Parallelism(2, parameter_storage={"x": "sharded"})
    with pytest.raises(ValueError):
        Parallelism(2, default_parameter_storage=ParameterStorage("all_ranks", "sharded"))
    p = Parallelism(4, 2, groups={"all_ranks": ((0, 1, 2, 3),), "pairs": ((0, 1), (2, 3))},
                    parameter_placements={"*.experts.*": Sharded("pairs", 0, "flat")},
                    parameter_storage={"embed.*": ParameterStorage(group="pairs")})
    q = Parallelism.from_json(p.to_json())
    assert q.to_json() == p.to_json()
    r = q.resolve("l.experts.w", rank=6, nbytes=1 << 30)
    assert r.compute_group == (6, 7) and r.compute_index == 0 and r.storage_group == (4, 5, 6, 7)
    assert q.resolve("embed.embed", rank=1, nbytes=1 << 30).storage_group == (0, 1)


def test_client_records_convert():
    p = from_client_record(client_par.data_parallel(8, weights="replicated", gradients="replicated"))
    assert p.world_size == 8 and p.default_parameter_storage.optimizer == "sharded"
    e = from_client_record(client_par.expert_parallel(4, n_experts=32, top_k=4))
    assert e.resolve("layer0.experts.w2", 1, 1 << 30).compute_shards == 4


def test_collective_sequence_digest_is_rank_invariant_and_order_sensitive():
    import torch
    from dataclasses import replace
    from shadowspill_b200.frontend.capture import BatchGeometry, StepDataOrdering, build_step
    from shadowspill_b200.models.config import preset
    from shadowspill_b200.parallel.collectives import collective_sequence_digest
    cfg = preset("llama3-tiny")
    geo = BatchGeometry(microbatch_tokens=256, n_microbatches=2, slots=16, mean_seqlen=64)
    build = lambda c, rank, order=StepDataOrdering(): build_step(c, geo, order, dtype=torch.float32,
                                                                  world_size=2, rank=rank)[0]
    a, b = collective_sequence_digest(build(cfg, 0)), collective_sequence_digest(build(cfg, 1))
    assert a == b                                             # every rank of one job agrees
    deeper = replace(cfg, n_layers=3)
    assert collective_sequence_digest(build(deeper, 0)) != a  # another model: another sequence
    depth = StepDataOrdering(walk="depth", optimizer="tail")
    assert collective_sequence_digest(build(cfg, 0, depth)) != a
