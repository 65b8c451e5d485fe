"""Multi-GPU tests: the sharded paths on real NCCL ranks, one process per GPU, against the single-GPU
result and the oracle.  They need at least two GPUs and are skipped on a one-GPU box; the host logic of
the same paths runs on CPU under gloo (test_sharding_gloo.py), and the two-launch kernel path on one GPU
with emulated ranks (test_gpu_two_phase.py)."""
import os
import socket
import subprocess
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.parametrize("mode", ["rows", "heads", "training"])
def test_sharded_paths_on_two_gpus(mode):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
           "127.0.0.1", "--master-port", str(_free_port()), str(ROOT / "tests" / "multi_gpu_workers.py"), mode]
    res = subprocess.run(cmd, cwd=ROOT, capture_output=True, text=True, timeout=600, env=dict(os.environ))
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-4000:]
    assert " ok on 2 GPUs" in res.stdout
