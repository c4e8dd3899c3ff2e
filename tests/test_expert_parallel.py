"""Expert-parallel routed experts (peer-memory dispatch, scatter-epilogue combine)
against the all-local routed-expert op."""
import os
import subprocess
import sys
from pathlib import Path

import pytest

WORKER = Path(__file__).with_name("_ep_worker.py")


@pytest.mark.gpu
@pytest.mark.multigpu
def test_two_gpus_match_local_experts():
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
           "--master-addr", "127.0.0.1", "--master-port", "29631", str(WORKER)]
    out = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stdout[-3000:] + out.stderr[-3000:]
    assert out.stdout.count(" OK ") == 2, out.stdout[-2000:]
