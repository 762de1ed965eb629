"""Multi-GPU paths that need more than one device; skipped on a single-GPU machine."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


def device_count() -> int:
    try:
        import torch
        return torch.cuda.device_count()
    except Exception:
        return 0


@pytest.mark.skipif(device_count() < 2, reason="needs two GPUs")
def test_all_gather_by_peer_copies(built):
    """Two ranks, one process per GPU: every rank's block must land in slot `rank` of every rank's
    receive buffer (buffers shared across the processes, copy engines, channel barrier)."""
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
           "127.0.0.1", "--master-port", "29533", os.path.join(HERE, "peer_gather_worker.py")]
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=300, env=env)
    assert out.returncode == 0 and "PEER_GATHER_OK" in out.stdout, out.stdout[-2000:] + out.stderr[-2000:]


@pytest.mark.skipif(device_count() < 2, reason="needs two GPUs")
def test_sharded_dispatch_pushes_its_block_to_every_rank(built):
    """Two ranks, one process per GPU: each computes its column block of a W4A16 product and its
    kernel's epilogue stores the block into both ranks' full-width results (plain stores into peer
    memory, arrival words, bounded wait); every rank must then hold the complete, exact result,
    over several rounds that reuse two result buffers without any host-side barrier between them."""
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
           "127.0.0.1", "--master-port", "29534", os.path.join(HERE, "push_worker.py")]
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=300, env=env)
    assert out.returncode == 0 and "PUSH_OK" in out.stdout, out.stdout[-2000:] + out.stderr[-2000:]
