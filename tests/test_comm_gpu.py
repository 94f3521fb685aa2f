"""The C ABI's own multi-GPU entry points (b2_comm_init, b2_matmul_sharded, b2_moe_ep: NCCL opened by the library itself)
on two GPUs: tensor-parallel dense matmul and expert-parallel routed experts, each bit-identical to the single-GPU call.
Needs two GPUs (skipped on a one-GPU box); the symbols' presence and the decline without a communicator are checked on
one."""
import os
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

import oxinfer_b200 as ob
from oxinfer_b200 import synth

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def test_sharded_calls_need_a_communicator(backend):
    ref = synth.q4_k(256, 256, 1)
    dev = backend.upload(ref, 256, 256)
    x = torch.zeros((4, 256), device="cuda")
    y = torch.zeros((4, 256), device="cuda")
    with pytest.raises(ob.BackendError, match="no communicator"):
        backend.matmul_sharded(dev, x, y)


def test_one_rank_communicator_is_the_single_gpu_call(backend):
    """world = 1: the same entry points with a one-rank NCCL communicator give the plain calls' bits."""
    assert backend.comm_init(1, 0, ob.Backend.comm_unique_id())
    try:
        n_out, n_in, t = 512, 512, 40
        ref = synth.q4_k(n_out, n_in, 2)
        dev = backend.upload(ref, n_out, n_in)
        x = torch.from_numpy(synth.activations(t, n_in, 3)).cuda()
        y, want = torch.zeros((t, n_out), device="cuda"), torch.zeros((t, n_out), device="cuda")
        assert backend.matmul_sharded(dev, x, y) and backend.matmul_dev(dev, x, want)
        torch.cuda.synchronize()
        assert torch.equal(y, want)
    finally:
        backend.comm_free()


@pytest.mark.parametrize("ranks", [2, 4])
def test_ranks_through_the_c_abi_match_single_gpu_bitwise(ranks):
    if torch.cuda.device_count() < ranks:
        pytest.skip(f"needs {ranks} GPUs")
    env = {k: v for k, v in os.environ.items() if not k.startswith("B2_")}
    env["NCCL_NVLS_ENABLE"] = "0"
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={ranks}", "--master-addr", "127.0.0.1", "--master-port",
           str(29651 + ranks), str(ROOT / "tests" / "comm_worker.py")]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env, cwd=str(ROOT))
    assert r.returncode == 0 and "COMM_OK" in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]
