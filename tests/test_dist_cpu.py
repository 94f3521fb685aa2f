"""Host logic of the two sharded paths on CPU ranks (gloo, world size 2): row-sharded dense layers with
an all-gather of y, and expert-parallel MoE with all-to-all dispatch / combine. The local compute is
the pinned oracle; the sharded results must equal the single-process result bit for bit."""
import os
import socket
import sys
from pathlib import Path

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))

from oxinfer_b200.dist import ExpertParallel, expert_shard, gather_columns, row_shard  # noqa: E402


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _tp_worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from oracle import oracle as O
    from oxinfer_b200 import synth
    from util import oracle_matrix

    n_out, n_in, t = 96, 512, 9
    ref = synth.q4_k(n_out, n_in, 800)
    x = synth.activations(t, n_in, 801)
    r0, r1 = row_shard(n_out, world, rank)
    rb = n_in // 256 * 144
    shard = ref.data.reshape(n_out, rb)[r0:r1].reshape(-1).copy()
    m = O.Matrix.gguf(O.Q4_K, shard, r1 - r0, n_in)
    y_local = torch.from_numpy(m.matmul_prefill(x, threads=1))
    y = gather_columns(y_local, n_out)
    full = oracle_matrix(ref, n_out, n_in).matmul_prefill(x, threads=1)
    out[rank] = bool(np.array_equal(y.numpy(), full))
    dist.destroy_process_group()


def _ep_worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from oracle import oracle as O
    from oxinfer_b200 import synth
    from util import oracle_matrix

    n_experts, k, h, inter, t_total = 8, 3, 256, 256, 22
    gu = [oracle_matrix(synth.mlx4(2 * inter, h, 810 + 2 * e), 2 * inter, h) for e in range(n_experts)]
    dn = [oracle_matrix(synth.mlx4(h, inter, 811 + 2 * e), h, inter) for e in range(n_experts)]
    rng = np.random.default_rng(812)
    logits = (rng.standard_normal((t_total, n_experts)) + rng.standard_normal(n_experts)).astype(np.float32)
    ids, w = np.zeros((t_total, k), np.int32), np.zeros((t_total, k), np.float32)
    for i in range(t_total):
        ids[i], w[i] = O.route_top_k(logits[i], k)
    x = synth.activations(t_total, h, 813)
    want = O.moe_forward(gu, dn, h, inter, x, ids, w, exact=True, threads=1)

    e0, e1 = expert_shard(n_experts, world, rank)
    t0, t1 = (0, 13) if rank == 0 else (13, t_total)  # ragged token shards

    def local_experts(rows, eids):
        one = np.ones((rows.shape[0], 1), np.float32)
        o = O.moe_forward(gu[e0:e1], dn[e0:e1], h, inter, rows.numpy(), eids.numpy().reshape(-1, 1), one, exact=True, threads=1)
        return torch.from_numpy(o)

    ep = ExpertParallel(n_experts)
    y = torch.zeros((t1 - t0, h))
    ep.forward(torch.from_numpy(x[t0:t1]), torch.from_numpy(ids[t0:t1]), torch.from_numpy(w[t0:t1]), y, local_experts)
    out[rank] = bool(np.array_equal(y.numpy(), want[t0:t1]))
    dist.destroy_process_group()


def _run(worker):
    world, port = 2, _free_port()
    with mp.Manager() as mgr:
        out = mgr.dict()
        mp.spawn(worker, args=(world, port, out), nprocs=world, join=True)
        assert dict(out) == {0: True, 1: True}


def test_row_shard_covers_rows_once():
    for n_out, world, mult in [(14336, 8, 1), (28672, 8, 128), (1000, 4, 1), (300, 8, 128), (7, 8, 1)]:
        spans = [row_shard(n_out, world, r, mult) for r in range(world)]
        assert spans[0][0] == 0 and spans[-1][1] == n_out
        for (a0, a1), (b0, b1) in zip(spans, spans[1:]):
            assert a1 == b0 and a0 <= a1
        assert all(s[0] % mult == 0 for s in spans if s[1] > s[0])
    assert [expert_shard(128, 8, r) for r in (0, 7)] == [(0, 16), (112, 128)]


def test_tensor_parallel_gather_matches_single_process():
    _run(_tp_worker)


def test_expert_parallel_dispatch_combine_matches_single_process():
    _run(_ep_worker)
