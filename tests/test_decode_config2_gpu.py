"""One decoder layer and the output head at the benchmark's true shape against the CPU oracle's decoder step:
hidden 4096, 32 query heads and 8 KV heads of 128, SwiGLU FFN 14336, vocabulary 128256; Q4_K projections, Q6_K head,
interleaved RoPE with theta 500000 (the Llama branch of src/qwen.rs:1177-1528).

The other decode tests use a small model, which leaves the launch shapes of the real one untested: K = 14336 planes
(more than 48 KB of shared memory), the fused q/k/v launch at 6144 rows, four query heads per KV head at 128 dims, the
128256-row head. The positions cover an empty cache, the last key before and the first key after the 2048-token
context of the benchmark, and its last decoded token. The oracle runs exact products (f64 sums over the bit-exact
dequantized weights); bound 1e-4 of the vector's largest magnitude, as for the small model.
"""
import numpy as np
import pytest

from oracle import oracle as O
from oxinfer_b200 import decode as D
from oxinfer_b200 import synth

from util import oracle_matrix, row_err

pytestmark = pytest.mark.gpu

CFG = dict(n_layers=1, h=4096, nh=32, nkv=8, hd=128, inter=14336, vocab=128256)
MAX_LEN = 2304


def test_one_layer_and_head_at_the_benchmark_shape(backend):
    layers, final_norm, head, _, shapes = synth.llama_weights(seed=0xB2000020, **CFG)
    L = layers[0]
    dev = {name: backend.upload(L[name], *shapes[name]) for name in shapes}
    cpu_l = {name: oracle_matrix(L[name], *shapes[name]) for name in shapes}
    for name in ("ln_pre", "ln_post"):
        dev[name] = cpu_l[name] = L[name]
    dhead = backend.upload(head, CFG["vocab"], CFG["h"])
    lc = D.LlamaConfig(eps=1e-5, rope_theta=500000.0, rope_interleaved=True, **CFG)
    plan = D.decode_plan(backend, D.llama_graph(lc, [dev], final_norm, dhead), MAX_LEN)
    assert plan is not None, backend.last_declined
    ocfg = O.LlamaCfg(1, CFG["h"], CFG["nh"], CFG["nkv"], CFG["hd"], CFG["inter"], CFG["vocab"], 1, 1e-5, lc.scale)
    cpu = O.Llama(ocfg, [cpu_l], final_norm, oracle_matrix(head, CFG["vocab"], CFG["h"]), MAX_LEN)
    inv_freq = O.rope_inv_freq(CFG["hd"], lc.rope_theta)
    rng = np.random.default_rng(41)
    row = CFG["nkv"] * CFG["hd"]
    k = rng.standard_normal((MAX_LEN, row)).astype(np.float32)
    v = rng.standard_normal((MAX_LEN, row)).astype(np.float32)
    cpu.kc[0], cpu.vc[0] = k, v
    plan.kv_write(0, 0, k, v)
    for pos in (0, 2047, 2048, 2303):
        x = rng.standard_normal(CFG["h"]).astype(np.float32)
        cs = O.rope_table(pos, inv_freq)
        hid, logits = plan.step(pos, x, cs)
        rh, rl = cpu.step(pos, x, cs, exact=True)
        eh, el = row_err(hid[None], rh[None]), row_err(logits[None], rl[None])
        print(f"config-2 shape, position {pos}: hidden row error {eh:.2e}, logits row error {el:.2e}")
        assert eh < 1e-4, (pos, eh)
        assert el < 1e-4, (pos, el)
        assert int(np.argmax(logits)) == int(np.argmax(rl))
        kk, vv = plan.kv_read(0, pos, 1)
        assert row_err(kk.reshape(1, -1), cpu.kc[0, pos][None]) < 1e-4
        assert row_err(vv.reshape(1, -1), cpu.vc[0, pos][None]) < 1e-4
        # the step overwrote row `pos` on both sides; put the random row back so that later positions see the same cache
        cpu.kc[0, pos], cpu.vc[0, pos] = k[pos], v[pos]
        plan.kv_write(0, pos, k[pos : pos + 1], v[pos : pos + 1])
    plan.close()
