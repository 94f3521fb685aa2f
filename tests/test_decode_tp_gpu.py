"""Tensor-parallel decode over two GPUs of one box: the plan's exchanges (stores into the peer's activation memory and
a flag barrier between the GPUs) must give the single-GPU plan's tokens and logits bit for bit. Needs two GPUs; on a
one-GPU box there is nothing to run and the test is skipped (the host-side logic is covered on CPU in
test_decode_tp_cpu.py)."""
import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="tensor-parallel decode needs two GPUs")
def test_two_ranks_match_single_gpu_bitwise():
    env = {k: v for k, v in os.environ.items() if not k.startswith("B2_")}   # no switches left over from other tests
    env["NCCL_NVLS_ENABLE"] = "0"
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1", "--master-port", "29641",
           str(ROOT / "tests" / "tp_decode_worker.py")]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env, cwd=str(ROOT))
    assert r.returncode == 0 and "TP_OK" in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]
