"""GPU suite (needs two GPUs, skipped otherwise): the peer-memory gradient exchange between
two processes, one per GPU, against a single-GPU run of the same steps."""
import os
import subprocess
import sys

import pytest
import torch

from conftest import ROOT

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("mode", [0, 3])
def test_two_gpu_peer_exchange_matches_single_gpu(gemm_lib, mode):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
           "--master-addr", "127.0.0.1", "--master-port", str(29611 + mode),
           os.path.join(ROOT, "tests", "peer_worker.py"), str(mode)]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "PEER_OK" in r.stdout
