"""Multi-GPU parity on a box with at least two GPUs: one process per GPU under torchrun
(tests/multi_gpu_worker.py).  Skipped on a single GPU."""
import os
import socket
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_column_and_expert_parallel_match_one_gpu():
    env = dict(os.environ)
    env["NCCL_NVLS_ENABLE"] = "0"
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
           "127.0.0.1", "--master-port", str(_free_port()), os.path.join(ROOT, "tests", "multi_gpu_worker.py")]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    sys.stdout.write(res.stdout[-3000:])
    assert res.returncode == 0, res.stderr[-3000:]
    assert "MULTI_GPU_PARITY PASS" in res.stdout
