"""Steps of several tokens (`Backend::decode_plan_multi`, src/gpu.rs:273-276; `Step::t`, src/gpu_decode.rs:538-570).

The contract is the reference's for its multi-token kernels (src/cuda_decode.cu:176-179): a step of t tokens gives every
token the hidden state, logits and cache rows that t one-token steps give, bit for bit. The one-token plan is held to the
CPU oracle elsewhere; here the two plans run over the same uploaded weights and the same cache contents and their
outputs are compared with `array_equal`.
"""
import numpy as np
import pytest

import oxinfer_b200 as ob
from oracle import oracle as O
from oxinfer_b200 import decode as D
from oxinfer_b200 import synth

from util import oracle_matrix, row_err

pytestmark = pytest.mark.gpu

SMALL = dict(n_layers=2, h=256, nh=4, nkv=2, hd=64, inter=512, vocab=1024)
# products that write the next product's planes in their epilogue, grouped heads of 128
WIDE = dict(n_layers=3, h=512, nh=4, nkv=2, hd=128, inter=1024, vocab=512)


def two_plans(backend, cfg, seed, tokens=4, max_len=512, kv_f16=False, interleaved=True, with_cpu=False):
    layers, final_norm, head, embed, shapes = synth.llama_weights(seed=seed, **cfg)
    dev_layers, cpu_layers = [], []
    for L in layers:
        d = {name: backend.upload(L[name], n_out, n_in) for name, (n_out, n_in) in shapes.items()}
        d["ln_pre"], d["ln_post"] = L["ln_pre"], L["ln_post"]
        dev_layers.append(d)
        if with_cpu:
            c = {name: oracle_matrix(L[name], n_out, n_in) for name, (n_out, n_in) in shapes.items()}
            c["ln_pre"], c["ln_post"] = L["ln_pre"], L["ln_post"]
            cpu_layers.append(c)
    dhead = backend.upload(head, cfg["vocab"], cfg["h"])
    lc = D.LlamaConfig(eps=1e-5, rope_interleaved=interleaved, **cfg)
    g = D.llama_graph(lc, dev_layers, final_norm, dhead)
    one = D.decode_plan(backend, g, max_len, kv_f16=kv_f16)
    many = D.decode_plan_multi(backend, g, max_len, tokens, kv_f16=kv_f16)
    assert one is not None and many is not None, backend.last_declined
    inv_freq = O.rope_inv_freq(cfg["hd"], lc.rope_theta)
    cpu = None
    if with_cpu:
        ocfg = O.LlamaCfg(cfg["n_layers"], cfg["h"], cfg["nh"], cfg["nkv"], cfg["hd"], cfg["inter"], cfg["vocab"], int(interleaved), 1e-5, lc.scale)
        cpu = O.Llama(ocfg, cpu_layers, final_norm, oracle_matrix(head, cfg["vocab"], cfg["h"]), max_len)
    return one, many, inv_freq, cpu, (dev_layers, dhead, g)


def fill(plans, cfg, n, seed, cpu=None):
    """The same random keys and values in positions 0 .. n-1 of every cache of every plan."""
    rng = np.random.default_rng(seed)
    row = cfg["nkv"] * cfg["hd"]
    for li in range(cfg["n_layers"]):
        k = rng.standard_normal((n, row)).astype(np.float32)
        v = rng.standard_normal((n, row)).astype(np.float32)
        for p in plans:
            p.kv_write(li, 0, k, v)
        if cpu is not None:
            cpu.kc[li, :n], cpu.vc[li, :n] = k, v


def one_by_one(plan, pos, xs, inv_freq):
    out = [plan.step(pos + i, xs[i], O.rope_table(pos + i, inv_freq)) for i in range(len(xs))]
    return np.stack([o[0] for o in out]), np.stack([o[1] for o in out])


def rope_rows(pos, t, inv_freq):
    return np.stack([O.rope_table(pos + i, inv_freq) for i in range(t)])


def same_caches(a, b, cfg, pos0, n):
    for li in range(cfg["n_layers"]):
        ka, va = a.kv_read(li, pos0, n)
        kb, vb = b.kv_read(li, pos0, n)
        assert np.array_equal(ka, kb) and np.array_equal(va, vb), li


@pytest.mark.parametrize("cfg", [SMALL, WIDE], ids=["small", "wide"])
@pytest.mark.parametrize("kv_f16", [False, True], ids=["f32cache", "f16cache"])
def test_a_step_of_t_tokens_equals_t_steps_bit_for_bit(backend, cfg, kv_f16):
    one, many, inv_freq, _, keep = two_plans(backend, cfg, seed=1201, kv_f16=kv_f16)
    assert many.tokens() == 4 and one.tokens() == 1
    rng = np.random.default_rng(77)
    # contexts whose new keys land before, on and behind the edges of the attention kernel's 64-key tiles
    for pos in (0, 1, 61, 62, 63, 64, 126, 200):
        for t in (2, 3, 4):
            if pos:
                fill((one, many), cfg, pos, 500 + pos)
            xs = rng.standard_normal((t, cfg["h"])).astype(np.float32)
            h1, l1 = one_by_one(one, pos, xs, inv_freq)
            hm, lm = many.step_multi(pos, xs, rope_rows(pos, t, inv_freq))
            assert np.array_equal(hm, h1), (pos, t)
            assert np.array_equal(lm, l1), (pos, t)
            same_caches(one, many, cfg, pos, t)
    one.close()
    many.close()


def test_non_interleaved_rope_and_one_token_steps_of_the_same_plan(backend):
    one, many, inv_freq, cpu, keep = two_plans(backend, SMALL, seed=1202, interleaved=False, with_cpu=True)
    rng = np.random.default_rng(78)
    pos = 90
    fill((one, many), SMALL, pos, 41, cpu)
    xs = rng.standard_normal((3, SMALL["h"])).astype(np.float32)
    h1, l1 = one_by_one(one, pos, xs, inv_freq)
    hm, lm = many.step_multi(pos, xs, rope_rows(pos, 3, inv_freq))
    assert np.array_equal(hm, h1) and np.array_equal(lm, l1)
    # the oracle's decoder over the same three tokens
    for i in range(3):
        rh, rl = cpu.step(pos + i, xs[i], O.rope_table(pos + i, inv_freq), exact=True)
        assert row_err(hm[i][None], rh[None]) < 1e-4 and row_err(lm[i][None], rl[None]) < 1e-4
    # t = 1 through both entry points of the several-token plan
    x = rng.standard_normal((1, SMALL["h"])).astype(np.float32)
    ha, la = many.step_multi(pos + 3, x, rope_rows(pos + 3, 1, inv_freq))
    hb, lb = many.step(pos + 3, x[0], O.rope_table(pos + 3, inv_freq))
    hc, lc = one.step(pos + 3, x[0], O.rope_table(pos + 3, inv_freq))
    assert np.array_equal(ha[0], hb) and np.array_equal(hb, hc) and np.array_equal(la[0], lb) and np.array_equal(lb, lc)
    one.close()
    many.close()


def test_rejected_tokens_are_overwritten_by_the_next_step(backend):
    """Speculative verification: of four drafted tokens two are accepted; the next step starts behind them, and nothing of
    the two rejected tokens may remain (their cache rows are written again)."""
    one, many, inv_freq, _, keep = two_plans(backend, SMALL, seed=1203)
    rng = np.random.default_rng(79)
    pos = 130
    fill((one, many), SMALL, pos, 43)
    drafted = rng.standard_normal((4, SMALL["h"])).astype(np.float32)
    many.step_multi(pos, drafted, rope_rows(pos, 4, inv_freq))
    one_by_one(one, pos, drafted[:2], inv_freq)
    follow = rng.standard_normal((3, SMALL["h"])).astype(np.float32)
    hm, lm = many.step_multi(pos + 2, follow, rope_rows(pos + 2, 3, inv_freq))
    h1, l1 = one_by_one(one, pos + 2, follow, inv_freq)
    assert np.array_equal(hm, h1) and np.array_equal(lm, l1)
    same_caches(one, many, SMALL, 0, pos + 5)
    one.close()
    many.close()


def test_two_rope_tables_arrive_table_by_table(backend):
    """A graph with two RoPE tables of different widths: the step's rope_cs holds table 0's rows for all tokens, then
    table 1's (Step::rope_cs); the one-token step takes one row of each side by side."""
    nh, nkv, hd = 4, 2, 64
    nq = nh * hd

    def graph():
        g = D.Graph()
        q0, q1 = g.buf(nq + 2 * nkv * hd), g.buf(nq + 2 * nkv * hd)
        o0, o1, a0, out = g.buf(nq), g.buf(nq), g.buf(nq), g.buf(2 * nq)
        g.qk_rope(q0, o0, 0, nh, nkv, hd, hd // 2, nq, nq + nkv * hd, True, 1e-6, rope=0)
        g.attend(o0, out, 0, nh, nkv, hd, hd ** -0.5)
        g.norm(q0, q1, None, nq + 2 * nkv * hd, 1e-6)            # the second layer's input: something derived from the first's
        g.qk_rope(q1, o1, 1, nh, nkv, hd, hd // 4, nq, nq + nkv * hd, False, 1e-6, rope=1)
        g.attend(o1, out.at(nq), 1, nh, nkv, hd, hd ** -0.5)
        g.input, g.n_input, g.hidden, g.n_hidden = q0, nq + 2 * nkv * hd, out, 2 * nq
        g.kv, g.rope_halves = [(nkv, hd), (nkv, hd)], [hd // 2, hd // 4]
        return g

    g = graph()
    one = D.decode_plan(backend, g, 256)
    many = D.decode_plan_multi(backend, g, 256, 4)
    assert one is not None and many is not None, backend.last_declined
    rng = np.random.default_rng(80)
    inv0 = O.rope_inv_freq(hd, 1e6)
    inv1 = O.rope_inv_freq(hd // 2, 1e4)
    pos, t = 63, 4
    row = nkv * hd
    for li in range(2):
        k = rng.standard_normal((pos, row)).astype(np.float32)
        v = rng.standard_normal((pos, row)).astype(np.float32)
        one.kv_write(li, 0, k, v)
        many.kv_write(li, 0, k, v)
    xs = rng.standard_normal((t, nq + 2 * row)).astype(np.float32)
    t0 = np.stack([O.rope_table(pos + i, inv0) for i in range(t)])
    t1 = np.stack([O.rope_table(pos + i, inv1) for i in range(t)])
    h1 = np.stack([one.step(pos + i, xs[i], np.concatenate([t0[i], t1[i]]), want_logits=False)[0] for i in range(t)])
    hm, _ = many.step_multi(pos, xs, np.concatenate([t0.reshape(-1), t1.reshape(-1)]), want_logits=False)
    assert np.array_equal(hm, h1)
    for li in range(2):
        ka, va = one.kv_read(li, pos, t)
        kb, vb = many.kv_read(li, pos, t)
        assert np.array_equal(ka, kb) and np.array_equal(va, vb)
    one.close()
    many.close()


def test_argument_errors_and_declined_requests(backend):
    one, many, inv_freq, _, keep = two_plans(backend, SMALL, seed=1204, tokens=2, max_len=64)
    g = keep[2]
    assert many.tokens() == 2
    x = np.zeros((3, SMALL["h"]), dtype=np.float32)
    with pytest.raises(ob.BackendError, match="3 tokens in a step of a plan made for 2"):
        many.step_multi(0, x, rope_rows(0, 3, inv_freq))
    with pytest.raises(ob.BackendError, match="past the 64"):
        many.step_multi(63, x[:2], rope_rows(63, 2, inv_freq))
    with pytest.raises(ob.BackendError, match="made for 1"):
        one.step_multi(0, x[:2], rope_rows(0, 2, inv_freq))
    # the context is still good, and steps of more than four tokens are declined (the caller verifies through matmul)
    h, _ = many.step_multi(10, x[:2], rope_rows(10, 2, inv_freq))
    assert np.isfinite(h).all()
    assert D.decode_plan_multi(backend, g, 64, 5) is None and "four" in backend.last_declined
    one.close()
    many.close()
