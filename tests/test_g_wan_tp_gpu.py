"""GPU test of the tensor-parallel video-DiT step on 2 GPUs of one node (skipped with fewer): heads and FFN columns
sharded, residual stream sequence-parallel (all-gather / reduce-scatter per piece) and, for comparison, replicated
with an NCCL all-reduce after the row-parallel projections; result against the fp32 restatement."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_wan_step_tensor_parallel_2_gpus():
    here = os.path.dirname(os.path.abspath(__file__))
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                        "--master-addr", "127.0.0.1", "--master-port", "29533", os.path.join(here, "wan_tp_worker.py")],
                       capture_output=True, text=True, timeout=400, env=env)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert "TP=2" in r.stdout
