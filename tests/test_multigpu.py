"""Multi-process checks that need at least two GPUs on the box (skipped otherwise): the sequence-sharded
decode through the NCCL all-gather and through the peer-memory exchange, against the unsharded call."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_seq_sharded_paths_on_two_gpus():
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                        "--master-addr", "127.0.0.1", "--master-port", "29577", os.path.join(HERE, "mp_seq_sharded.py")],
                       capture_output=True, text=True, timeout=240, env=env)
    assert r.returncode == 0 and "MP_SEQ_SHARDED_OK 2" in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]
