"""One rank of the expert-parallel MoE test on GPUs (launched by test_moe_ep_gpu.py through torch.distributed.run):
tokens sharded over the ranks, experts sharded over the ranks, dispatch and combine by NCCL all-to-all
(oxinfer_b200.dist.ExpertParallel), the local experts on this rank's GPU through b2_moe_dev. The result must equal the
single-GPU b2_moe over all tokens and experts bit for bit: every (token, route) pair runs the same kernels on the same
inputs and the combine keeps the route order."""
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
from oxinfer_b200.dist import ExpertParallel, expert_shard  # noqa: E402


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    be = ob.Backend(local)
    be.set_stream(torch.cuda.current_stream().cuda_stream)
    E, K, H, I, T = 16, 4, 512, 256, 203
    refs = [(synth.mlx4(2 * I, H, 600 + 2 * e), synth.mlx4(H, I, 601 + 2 * e)) for e in range(E)]
    rng = np.random.default_rng(77)
    logits = (rng.standard_normal((T, E)) + rng.standard_normal(E)).astype(np.float32)
    ids = np.argsort(-logits, axis=1, kind="stable")[:, :K].astype(np.int32)
    top = np.take_along_axis(logits, ids, axis=1)
    w = np.exp(top - top[:, :1])
    w = (w / w.sum(axis=1, keepdims=True)).astype(np.float32)
    x = synth.activations(T, H, 78)

    e0, e1 = expert_shard(E, world, rank)
    gu = [be.upload(refs[e][0], 2 * I, H) for e in range(e0, e1)]
    dn = [be.upload(refs[e][1], H, I) for e in range(e0, e1)]
    local_moe = be.upload_moe(gu, dn, H, I)
    assert local_moe is not None, be.last_declined
    per = -(-T // world)
    t0, t1 = min(T, rank * per), min(T, (rank + 1) * per)

    def local_experts(rows, eids):
        # every received row is one (token, route) pair of a local expert with weight 1
        o = torch.zeros_like(rows)
        torch.cuda.synchronize()
        ok = be.moe_dev(rows.contiguous(), eids.cpu().numpy().reshape(-1, 1), np.ones((rows.shape[0], 1), np.float32), local_moe, o)
        assert ok, be.last_declined
        torch.cuda.synchronize()
        be.check_status()
        return o

    ep = ExpertParallel(E)
    y = torch.zeros((t1 - t0, H), device="cuda")
    ep.forward(torch.from_numpy(x[t0:t1]).cuda(), torch.from_numpy(ids[t0:t1]).cuda(), torch.from_numpy(w[t0:t1]).cuda(), y, local_experts)
    torch.cuda.synchronize()
    ok = True
    if rank == 0:
        agu = [be.upload(refs[e][0], 2 * I, H) for e in range(E)]
        adn = [be.upload(refs[e][1], H, I) for e in range(E)]
        full = be.upload_moe(agu, adn, H, I)
        want = np.zeros((T, H), np.float32)
        assert be.moe(x, ids, w, full, want)
    ys = [torch.zeros((min(T, (r + 1) * per) - min(T, r * per), H), device="cuda") for r in range(world)]
    dist.all_gather(ys, y) if all(t.shape == ys[0].shape for t in ys) else None
    if rank == 0:
        if all(t.shape == ys[0].shape for t in ys):
            got = torch.cat(ys).cpu().numpy()
            ok = bool(np.array_equal(got, want))
        else:   # ragged shards: compare rank 0's rows only
            ok = bool(np.array_equal(y.cpu().numpy(), want[t0:t1]))
        if not ok:
            print("MISMATCH", float(np.max(np.abs(y.cpu().numpy() - want[t0:t1]))), flush=True)
    flag = [ok]
    dist.broadcast_object_list(flag, src=0)
    if rank == 0 and flag[0]:
        print(f"EP_OK world={world}", flush=True)
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if flag[0] else 1)


if __name__ == "__main__":
    main()
