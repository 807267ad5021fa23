"""Multi-GPU checks that need real peers: launched as child processes, one rank per GPU,
when the machine has at least two GPUs (skipped otherwise)."""

import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("world", [2, 4])
def test_peer_gather_matches_library_gather_and_single_gpu(world):
    if not torch.cuda.is_available() or torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", NCCL_DEBUG_FILE="/dev/stderr")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(29600 + world),
           os.path.join(ROOT, "tests", "multi_gpu_gather_check.py")]
    r = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and f"MULTI_GPU_GATHER_OK {world}" in r.stdout, r.stdout[-2000:] + r.stderr[-4000:]
