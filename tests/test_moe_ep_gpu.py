"""Expert-parallel MoE over two GPUs: NCCL all-to-all dispatch / combine around the local grouped-expert kernels must
give the single-GPU layer's output bit for bit. Needs two GPUs (skipped on a one-GPU box; the dispatch / combine logic
runs on gloo ranks in test_dist_cpu.py)."""
import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="expert parallelism needs two GPUs")
def test_two_ranks_match_single_gpu_bitwise():
    env = {k: v for k, v in os.environ.items() if not k.startswith("B2_")}   # no switches left over from other tests
    env["NCCL_NVLS_ENABLE"] = "0"
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1", "--master-port", "29643",
           str(ROOT / "tests" / "ep_moe_worker.py")]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env, cwd=str(ROOT))
    assert r.returncode == 0 and "EP_OK" in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]
