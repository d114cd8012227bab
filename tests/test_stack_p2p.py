"""Two-GPU test of the column-parallel decode stack whose all-gather is fused into the decode kernels (peer
stores over NVLink plus a rank hand-shake).  Runs only where two GPUs are visible; each rank is a child process."""
import os
import socket
import subprocess
import sys

import pytest
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.mark.gpu
def test_peer_store_gather_matches_nccl_gather_on_two_gpus():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
           "--master-port", str(port), os.path.join(HERE, "p2p_stack_worker.py")]
    p = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=240)
    assert p.returncode == 0 and "P2P_STACK_OK" in p.stdout, p.stdout[-2000:] + p.stderr[-4000:]
