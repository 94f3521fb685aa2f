"""One rank of the C-ABI tensor- / expert-parallel test (launched by test_comm_gpu.py through torch.distributed.run, which here
only starts the processes and carries the NCCL id between them on the host: gloo). Everything on the GPUs goes through
b2_comm_init, b2_matmul_sharded, b2_matmul_sharded_peer and b2_moe_ep, i.e. the library's own NCCL use, as a non-Python host would drive it.

Checks, against the single-GPU calls on rank 0's device over the unsharded matrix / all experts and tokens:
  * the row-sharded dense matmul gives the full y on every rank, bit for bit, through the library collective and through the
    GEMM epilogue's own peer stores;
  * the expert-parallel layer gives every rank's token rows bit for bit (ragged token shards, an expert nobody routes to).
"""
import os
import sys
from pathlib import Path

import numpy as np
import torch
import torch.distributed as dist

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))

import oxinfer_b200 as ob  # noqa: E402
from oxinfer_b200 import synth  # noqa: E402


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("gloo")
    be = ob.Backend(local)
    be.set_stream(torch.cuda.current_stream().cuda_stream)
    box = [ob.Backend.comm_unique_id() if rank == 0 else None]
    dist.broadcast_object_list(box, src=0)
    assert be.comm_init(world, rank, box[0])
    ok = True

    # ---- tensor parallel: y = x W^T with W's rows sharded ----
    n_out, n_in, t = 256 * world * 3, 1024, 100
    full = synth.q4_k(n_out, n_in, 800)
    dfull = be.upload(full, n_out, n_in)
    per = n_out // world
    shard = be.shard_rows(dfull, rank * per, (rank + 1) * per)
    x = torch.from_numpy(synth.activations(t, n_in, 801)).cuda()
    y = torch.full((t, n_out), float("nan"), device="cuda")
    assert be.matmul_sharded(shard, x, y)
    want = torch.empty((t, n_out), device="cuda")
    assert be.matmul_dev(dfull, x, want)
    torch.cuda.synchronize()
    be.check_status()
    if not torch.equal(y.view(torch.int32), want.view(torch.int32)):
        print(f"rank {rank}: sharded matmul differs from the unsharded product", flush=True)
        ok = False

    # ---- the same with the gather done by the GEMM's epilogue (peer stores): several calls in a row (the two result areas
    # alternate), a larger product afterwards (the buffers are made again, collectively), ragged token counts ----
    for (tt, seed) in ((100, 801), (300, 802), (300, 803), (300, 804), (777, 805)):
        xx = torch.from_numpy(synth.activations(tt, n_in, seed)).cuda()
        ww = torch.empty((tt, n_out), device="cuda")
        assert be.matmul_dev(dfull, xx, ww)
        got = be.matmul_sharded_peer(shard, xx)
        assert got is not None, be.last_declined
        torch.cuda.synchronize()
        be.check_status()
        if got.shape != ww.shape or not torch.equal(got.view(torch.int32), ww.view(torch.int32)):
            print(f"rank {rank}: peer-store sharded matmul differs from the unsharded product at t = {tt}", flush=True)
            ok = False
    assert be.matmul_sharded_peer(shard, x[:4]) is None    # the matrix-vector routes do not store to peers: declined

    # ---- expert parallel ----
    E, K, H, I, T = 4 * world, 3, 512, 256, 157
    refs = [(synth.mlx4(2 * I, H, 810 + 2 * e), synth.mlx4(H, I, 811 + 2 * e)) for e in range(E)]
    rng = np.random.default_rng(82)
    logits = (rng.standard_normal((T, E)) + rng.standard_normal(E)).astype(np.float32)
    logits[:, 1] = -1e9                                   # an expert no token routes to
    ids = np.argsort(-logits, axis=1, kind="stable")[:, :K].astype(np.int32)
    top = np.take_along_axis(logits, ids, axis=1)
    w = np.exp(top - top[:, :1])
    w = (w / w.sum(axis=1, keepdims=True)).astype(np.float32)
    xs = synth.activations(T, H, 83)
    y0 = np.random.default_rng(84).standard_normal((T, H)).astype(np.float32)   # the layer adds into y
    pe = E // world
    gu = [be.upload(refs[e][0], 2 * I, H) for e in range(rank * pe, (rank + 1) * pe)]
    dn = [be.upload(refs[e][1], H, I) for e in range(rank * pe, (rank + 1) * pe)]
    local_moe = be.upload_moe(gu, dn, H, I)
    assert local_moe is not None, be.last_declined
    share = -(-T // world)
    t0, t1 = min(T, rank * share), min(T, (rank + 1) * share)
    xd = torch.from_numpy(xs[t0:t1]).cuda()
    yd = torch.from_numpy(y0[t0:t1]).cuda()
    for _ in range(2):                                    # twice: the second call adds again (scratch reuse, counts redone)
        assert be.moe_ep(xd, ids[t0:t1], w[t0:t1], local_moe, E, yd)
    torch.cuda.synchronize()
    be.check_status()
    agu = [be.upload(refs[e][0], 2 * I, H) for e in range(E)]
    adn = [be.upload(refs[e][1], H, I) for e in range(E)]
    fullm = be.upload_moe(agu, adn, H, I)
    wd = torch.from_numpy(y0[t0:t1]).cuda()
    for _ in range(2):
        assert be.moe_dev(torch.from_numpy(xs[t0:t1]).cuda(), ids[t0:t1], w[t0:t1], fullm, wd)
    torch.cuda.synchronize()
    if not torch.equal(yd.view(torch.int32), wd.view(torch.int32)):
        print(f"rank {rank}: expert-parallel layer differs, max {float((yd - wd).abs().max())}", flush=True)
        ok = False

    flags = [None] * world
    dist.all_gather_object(flags, ok)
    be.comm_free()
    if rank == 0 and all(flags):
        print(f"COMM_OK world={world}", flush=True)
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if all(flags) else 1)


if __name__ == "__main__":
    main()
