"""One rank of the tensor-parallel decode test (launched by test_decode_tp_gpu.py through torch.distributed.run).

Every rank builds the same seeded model, keeps its row shards, and runs the collective plan; rank 0 also runs the
single-GPU plan and checks that tokens and logits are bit-identical (every output row is computed by the same kernel
over the same inputs, only on another GPU)."""
import os
import sys
from pathlib import Path

import numpy as np
import torch
import torch.distributed as dist

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))

import oxinfer_b200 as ob  # noqa: E402
from oxinfer_b200 import decode as D  # noqa: E402
from oxinfer_b200 import synth  # noqa: E402


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    dist.init_process_group("gloo")
    torch.cuda.set_device(local)
    be = ob.Backend(local)
    cfg = dict(n_layers=2, h=512, nh=8, nkv=4, hd=64, inter=1024, vocab=2048)
    layers, final_norm, head, embed, shapes = synth.llama_weights(seed=4242, **cfg)
    full = []
    for L in layers:
        d = {name: be.upload(L[name], *shapes[name]) for name in shapes}
        d["ln_pre"], d["ln_post"] = L["ln_pre"], L["ln_post"]
        full.append(d)
    dhead = be.upload(head, cfg["vocab"], cfg["h"])
    dembed = be.upload(embed, cfg["vocab"], cfg["h"])
    lc = D.LlamaConfig(eps=1e-5, **cfg)
    max_len, n0, n = 256, 70, 12
    sh_layers, sh_head = D.shard_llama(be, full, dhead, lc, rank, world)
    plan = D.decode_plan(be, D.llama_graph(lc, sh_layers, final_norm, sh_head, rank, world), max_len)
    assert plan is not None, be.last_declined
    handles = [None] * world
    dist.all_gather_object(handles, plan.export_handle())
    plan.attach_peers(rank, world, handles)

    rng = np.random.default_rng(11)
    row = cfg["nkv"] * cfg["hd"]
    kv = [(rng.standard_normal((n0, row)).astype(np.float32), rng.standard_normal((n0, row)).astype(np.float32)) for _ in range(cfg["n_layers"])]
    per = row // world   # this rank's KV heads are a contiguous run of every row
    for li, (k, v) in enumerate(kv):
        plan.kv_write(li, 0, np.ascontiguousarray(k[:, rank * per:(rank + 1) * per]), np.ascontiguousarray(v[:, rank * per:(rank + 1) * per]))
    inv_freq = D.rope_inv_freq(cfg["hd"], lc.rope_theta)
    table = np.stack([D.rope_table(n0 + i, inv_freq) for i in range(n)])
    dist.barrier()
    toks, ms = plan.generate(dembed, 3, n0, n, table)
    # one host-driven step too (collective): logits of the position after the generated ones
    x = np.random.default_rng(5).standard_normal(cfg["h"]).astype(np.float32)
    hid, logits = plan.step(n0 + n, x, D.rope_table(n0 + n, inv_freq))
    ok = True
    if rank == 0:
        single = D.decode_plan(be, D.llama_graph(lc, full, final_norm, dhead), max_len)
        for li, (k, v) in enumerate(kv):
            single.kv_write(li, 0, k, v)
        ref_toks, _ = single.generate(dembed, 3, n0, n, table)
        ref_hid, ref_logits = single.step(n0 + n, x, D.rope_table(n0 + n, inv_freq))
        ok = toks.tolist() == ref_toks.tolist() and np.array_equal(logits, ref_logits) and np.array_equal(hid, ref_hid)
        if not ok:
            print("MISMATCH", toks.tolist(), ref_toks.tolist(), float(np.max(np.abs(logits - ref_logits))), flush=True)
        single.close()
    flag = [ok]
    dist.broadcast_object_list(flag, src=0)
    dist.barrier()
    plan.close()
    be.close()
    if rank == 0 and flag[0]:
        print(f"TP_OK world={world} tokens={toks.tolist()} ms={ms:.3f}", flush=True)
    dist.destroy_process_group()
    sys.exit(0 if flag[0] else 1)


if __name__ == "__main__":
    main()
