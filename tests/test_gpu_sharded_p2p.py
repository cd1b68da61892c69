"""Column-sharded Linear across the GPUs of one box, results exchanged by stores into the peers'
buffers.  Needs at least two GPUs (skipped otherwise); each rank is a child process."""

import os
import socket
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_p2p_exchange_matches_unsharded_on_every_rank(lib_built):
    world = 2
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(_free_port()), os.path.join(HERE, "_sharded_p2p_worker.py")]
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=240, env=env)
    assert "SHARDED_P2P_OK" in out.stdout, out.stdout[-2000:] + out.stderr[-2000:]
