"""Batched prompt pass on a tensor-parallel decoder (needs two GPUs; skipped on a single-GPU box)."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_tensor_parallel_prefill_matches_single_gpu():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    here = os.path.dirname(os.path.abspath(__file__))
    env = dict(os.environ, NCCL_DEBUG="WARN")
    out = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
                          "--master-port", "29571", os.path.join(here, "tp_prefill_check.py")], capture_output=True, text=True, timeout=600, env=env)
    assert "TP_PREFILL_OK" in out.stdout, out.stdout[-2000:] + out.stderr[-2000:]
