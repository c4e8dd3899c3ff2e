"""Sharded data-parallel execution against the resident single-process trainer."""
import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

WORKER = Path(__file__).with_name("_dp_worker.py")


def _launch(world, device, arm, port, **extra_env):
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", NCCL_NVLS_ENABLE="0", **extra_env)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(port), str(WORKER), device, arm]
    out = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stdout[-3000:] + out.stderr[-3000:]
    assert out.stdout.count(" OK ") == world, out.stdout[-2000:]


def test_two_ranks_gloo_match_resident():
    _launch(2, "cpu", "dist", 29611)


def test_small_tensors_stay_whole_under_sharded_storage():
    """``min_shard_bytes``: small tensors are replicated and updated identically by every rank
    from the summed gradient; the job still matches the single-process model."""
    _launch(2, "cpu", "small-dist", 29641)


def test_lion_update_under_sharded_storage():
    """An update rule other than AdamW: gradients are summed with the library all-reduce and the
    rule is applied to the owned slices (small tensors whole); matches the single-process model."""
    _launch(2, "cpu", "lion-small-dist", 29651)


def test_master_copies_under_sharded_storage():
    """fp32 master shards: the update runs on them (unfused, after a library all-reduce) and is
    rounded into the weight shards; small tensors whole. Matches the single-process model."""
    _launch(2, "cpu", "master-small-dist", 29661)


ARMS_WITH_GROUPS = ["groups-dist", "groups-lion-small-dist", "groups-master-small-dist", "graph-groups-dist",
                    "tied-groups-dist", "tied-graph-groups-small-dist"]


@pytest.mark.parametrize("arm", ARMS_WITH_GROUPS)
def test_microbatch_groups_accumulate_in_shard_space(arm):
    """Four microbatches as two forward + backward sweeps: the first sweep's gradients are
    reduce-scattered into fp32 shard sums, the update after the second sweep starts from them.
    Matches the single-process model on the same eight microbatches."""
    _launch(2, "cpu", arm, 29671 + 2 * ARMS_WITH_GROUPS.index(arm))


def test_whole_parameter_weights_load_into_sharded_ranks():
    """Weights of another seed given as whole tensors: every rank keeps its slice, and the
    sharded job then trains exactly like a single-process model started from those weights."""
    _launch(2, "cpu", "pretrained-dist", 29631)


def test_two_replicas_of_two_shards_gloo_match_resident():
    """Hierarchical data parallelism: state sharded inside groups of two ranks, two such groups;
    gradients are summed over all four ranks, weights are gathered inside a group."""
    _launch(4, "cpu", "replicas-dist", 29621)


@pytest.mark.gpu
@pytest.mark.multigpu
@pytest.mark.parametrize("arm", ["peer", "dist", "small-peer", "lion-peer", "groups-peer", "groups-small-peer"])
def test_two_gpus_match_resident(arm):
    _launch(2, "cuda", arm, 29613 if arm == "peer" else 29615)


@pytest.mark.gpu
@pytest.mark.multigpu
def test_two_gpus_weight_gather_fused_into_the_gemm():
    """Sharded storage with the forward all-gather of every layer matrix done by the GEMM that
    first consumes it (peer loads inside the tcgen05 kernel); matches the resident model."""
    _launch(2, "cuda", "fused-peer", 29673)


@pytest.mark.gpu
@pytest.mark.multigpu
@pytest.mark.parametrize("nvls", ["0", "1"])
def test_fused_reduce_scatter_adamw_elementwise(nvls):
    """The fused kernel on its own: p, m and v of the owned slice against AdamW on the fp32-summed
    gradient, to one bf16 unit in the last place; ragged tails, fp32 gradients, and the in-switch
    sum when the fabric offers it."""
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", NCCL_NVLS_ENABLE="0", SS_NVLS=nvls)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
           "--master-addr", "127.0.0.1", "--master-port", "29671", str(WORKER.with_name("_rs_worker.py"))]
    out = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stdout[-3000:] + out.stderr[-3000:]
    assert out.stdout.count(" OK ") == 2, out.stdout[-2000:]


@pytest.mark.gpu
@pytest.mark.multigpu
def test_two_gpus_expert_parallel_planned_execution():
    """A routed model trains through the planned executor with its experts split over two
    GPUs (peer-memory dispatch/combine inside the layer tasks) and matches the resident
    single-process model that holds every expert."""
    _launch(2, "cuda", "ep", 29617)


@pytest.mark.gpu
@pytest.mark.multigpu
def test_two_gpus_in_switch_gradient_sum():
    """The sharded optimizer update with its gradient sum taken by multimem.ld_reduce inside the
    NVSwitch (SS_NVLS=1; falls back to peer loads where the fabric has no multicast)."""
    _launch(2, "cuda", "peer", 29619, SS_NVLS="1")


@pytest.mark.gpu
@pytest.mark.multigpu
def test_four_gpus_two_replicas_peer_kernels():
    import torch
    if torch.cuda.device_count() < 4:
        pytest.skip("needs four GPUs")
    _launch(4, "cuda", "replicas-peer", 29623)
