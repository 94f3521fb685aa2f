"""Host-side logic of tensor-parallel decode plans, on CPU: the per-rank graphs (shares, offsets, where the exchanges
sit) and the handle exchange between two gloo ranks."""
import os
import sys
from dataclasses import dataclass
from pathlib import Path

import numpy as np
import torch.distributed as dist
import torch.multiprocessing as mp

from oxinfer_b200 import _lib
from oxinfer_b200 import decode as D

ROOT = Path(__file__).resolve().parent.parent


@dataclass
class FakeWeight:
    handle: int
    n_out: int
    n_in: int
    fmt: int = 12


def fake_model(cfg, world):
    """Row shards as shard_llama would return them (shapes only)."""
    h, hd = cfg.h, cfg.hd
    L = {"q": FakeWeight(1, cfg.nh * hd // world, h), "k": FakeWeight(2, cfg.nkv * hd // world, h), "v": FakeWeight(3, cfg.nkv * hd // world, h),
         "o": FakeWeight(4, h // world, cfg.nh * hd), "gate": FakeWeight(5, cfg.inter // world, h), "up": FakeWeight(6, cfg.inter // world, h),
         "down": FakeWeight(7, h // world, cfg.inter), "ln_pre": np.ones(h, np.float32), "ln_post": np.ones(h, np.float32)}
    return [dict(L) for _ in range(cfg.n_layers)], FakeWeight(8, cfg.vocab // world, h)


def test_rank_graphs_shares_and_exchanges():
    cfg = D.LlamaConfig(n_layers=3, h=4096, nh=32, nkv=8, hd=128, inter=14336, vocab=128256)
    single = D.llama_graph(cfg, *[fake_model(cfg, 1)[0]], np.ones(4096, np.float32), fake_model(cfg, 1)[1])
    assert sum(o.kind == _lib.OP_EXCHANGE for o in single.ops) == 0 and len(single.ops) == 3 * 10 + 2
    for world in (2, 4, 8):
        for rank in range(world):
            layers, head = fake_model(cfg, world)
            g = D.llama_graph(cfg, layers, np.ones(4096, np.float32), head, rank, world)
            ex = [o for o in g.ops if o.kind == _lib.OP_EXCHANGE]
            assert len(ex) == 3 * 4 + 1
            assert [o.n for o in ex[:4]] == [4096, 4096, 14336, 4096] and ex[-1].n == 128256
            assert all(o.n % (32 * world) == 0 for o in ex)
            assert g.kv == [(8 // world, 128)] * 3
            lin = [o for o in g.ops if o.kind == _lib.OP_LINEAR]
            o_proj, pair, down, head_op = lin[3], lin[4], lin[5], lin[-1]
            assert o_proj.y.off == rank * 4096 // world and o_proj.mode == _lib.MODE_ADD and o_proj.n_in == 4096
            assert pair.y.off == rank * 14336 // world and pair.mode == _lib.MODE_SILU_PAIR
            assert down.y.off == rank * 4096 // world and down.n_in == 14336
            assert head_op.y.off == rank * 128256 // world
            att = [o for o in g.ops if o.kind == _lib.OP_ATTEND][0]
            assert att.nh == 32 // world and att.nkv == 8 // world and att.y.off == rank * 4096 // world
            # every exchange directly follows the op that wrote this rank's part of the vector
            for i, o in enumerate(g.ops):
                if o.kind == _lib.OP_EXCHANGE:
                    prev = g.ops[i - 1]
                    assert prev.y.buf == o.x.buf and prev.kind in (_lib.OP_LINEAR, _lib.OP_ATTEND)


def _handle_worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    mine = bytes([rank]) * _lib.PLAN_HANDLE_BYTES      # what export_handle() would return
    handles = [None] * world
    dist.all_gather_object(handles, mine)
    blob = b"".join(handles)                           # what attach_peers() passes to the library
    ok = len(blob) == world * _lib.PLAN_HANDLE_BYTES and all(blob[p * _lib.PLAN_HANDLE_BYTES] == p for p in range(world))
    out[rank] = ok
    dist.destroy_process_group()


def test_handles_travel_in_rank_order_gloo_world2():
    with mp.Manager() as m:
        out = m.dict()
        mp.spawn(_handle_worker, args=(2, 29653, out), nprocs=2, join=True)
        assert out[0] and out[1]
