"""The decoder under tensor parallelism on two GPUs (skipped where there is one): see tests/serve_tp_ranks.py."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu


def test_tensor_parallel_decoder_two_ranks():
    import torch

    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    here = os.path.dirname(os.path.abspath(__file__))
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    proc = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
                           "127.0.0.1", "--master-port", "29534", os.path.join(here, "serve_tp_ranks.py")],
                          capture_output=True, text=True, timeout=600, env=env)
    assert proc.returncode == 0, proc.stdout[-2000:] + proc.stderr[-2000:]
    assert "failures 0, status 0" in proc.stdout
