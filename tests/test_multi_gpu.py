"""A scan-sharded run equals the single-GPU run: two ranks (one per GPU, NCCL) each run their scans and gather the
logits; rank 0 recomputes every scan alone and compares bit for bit.  Skipped on a box with one GPU; the
host-side sharding logic is covered on CPU (gloo) by tests/test_sharding.py."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_sharded_run_equals_single_gpu_run():
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29541", os.path.join(ROOT, "tests", "_sharded_worker.py")]
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    assert r.returncode == 0 and "SHARDED_OK" in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]
