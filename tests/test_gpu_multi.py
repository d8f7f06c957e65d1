"""Token-sharded decode on two real GPUs: child processes (one rank per GPU) exchange their partial
triples with the fused peer-memory kernel and must reproduce single-GPU attention over the whole
sequence. Skipped when fewer than two GPUs are visible. NVLS is switched off for the NCCL
cross-check; the exchange kernel itself uses plain peer stores."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_rank_sharded_decode():
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
           "127.0.0.1", "--master-port", "29533", os.path.join(HERE, "sharded_worker.py")]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=300)
    sys.stdout.write(r.stdout[-2000:])
    sys.stderr.write(r.stderr[-3000:])
    assert r.returncode == 0
