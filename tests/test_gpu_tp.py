"""Tensor-parallel parity on two and four GPUs (skipped where the box has fewer): see tp_worker.py."""
import os
import socket
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu


def _gpu_count() -> int:
    try:
        out = subprocess.run(["nvidia-smi", "-L"], capture_output=True, text=True, timeout=30).stdout
    except (OSError, subprocess.TimeoutExpired):
        return 0
    return sum(1 for line in out.splitlines() if line.startswith("GPU "))


@pytest.mark.parametrize("world", [2, 4])
def test_tensor_parallel_decode_matches_the_oracle(world):
    if _gpu_count() < world:
        pytest.skip("needs %d GPUs" % world)
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    here = os.path.dirname(os.path.abspath(__file__))
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(world), "--master-addr", "127.0.0.1",
           "--master-port", str(port), os.path.join(here, "tp_worker.py")]
    p = subprocess.run(cmd, capture_output=True, text=True, timeout=400, env=env)
    assert p.returncode == 0 and "TP_WORKER_OK" in p.stdout, p.stdout[-3000:] + p.stderr[-3000:]
