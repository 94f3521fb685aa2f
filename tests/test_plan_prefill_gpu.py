"""Prefill plans (`Backend::decode_plan_prefill`, src/gpu.rs:283-289): steps of many tokens on batched kernels.

The reference says of such a plan that "its results differ from one-token steps in rounding". Here the products are the
tensor-core GEMMs (activations rounded to f16 per row, weights to f16: held to 1e-3 per product against the oracle
elsewhere) and attention rounds q, k, v and the probabilities to f16, so the bound on a whole step is the
reduced-precision one of this suite, 2e-3 of the row's largest magnitude per layer of depth (`row_err`,
src/cuda.rs:1582-1592), against the one-token plan (itself within 1e-4 of the CPU oracle) and against the oracle directly.
"""
import os

import numpy as np
import pytest

import oxinfer_b200 as ob
from oracle import oracle as O
from oxinfer_b200 import decode as D
from oxinfer_b200 import synth

from util import oracle_matrix, row_err

pytestmark = pytest.mark.gpu

SMALL = dict(n_layers=2, h=256, nh=4, nkv=2, hd=64, inter=512, vocab=1024)
WIDE = dict(n_layers=3, h=512, nh=8, nkv=2, hd=128, inter=1024, vocab=512)


def plans(backend, cfg, seed, tokens, max_len=512, kv_f16=False, interleaved=True, with_cpu=False, mixed=False):
    layers, final_norm, head, embed, shapes = synth.llama_weights(seed=seed, mixed=mixed, **cfg)
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
    one = D.decode_plan(backend, D.llama_graph(lc, dev_layers, final_norm, dhead), max_len, kv_f16=kv_f16)
    gp = D.llama_graph(lc, dev_layers, final_norm, dhead, prefill=True)
    pre = D.decode_plan_prefill(backend, gp, max_len, tokens, kv_f16=kv_f16)
    assert one is not None and pre is not None, backend.last_declined
    inv_freq = O.rope_inv_freq(cfg["hd"], lc.rope_theta)
    cpu = None
    if with_cpu:
        ocfg = O.LlamaCfg(cfg["n_layers"], cfg["h"], cfg["nh"], cfg["nkv"], cfg["hd"], cfg["inter"], cfg["vocab"], int(interleaved), 1e-5, lc.scale)
        cpu = O.Llama(ocfg, cpu_layers, final_norm, oracle_matrix(head, cfg["vocab"], cfg["h"]), max_len)
    return one, pre, inv_freq, cpu, (dev_layers, dhead, gp, lc, final_norm)


def fill(ps, cfg, n, seed, cpu=None):
    rng = np.random.default_rng(seed)
    row = cfg["nkv"] * cfg["hd"]
    for li in range(cfg["n_layers"]):
        k = rng.standard_normal((n, row)).astype(np.float32)
        v = rng.standard_normal((n, row)).astype(np.float32)
        for p in ps:
            p.kv_write(li, 0, k, v)
        if cpu is not None:
            cpu.kc[li, :n], cpu.vc[li, :n] = k, v


def rope_rows(pos, t, inv_freq):
    return np.stack([O.rope_table(pos + i, inv_freq) for i in range(t)])


def one_by_one(plan, pos, xs, inv_freq):
    return np.stack([plan.step(pos + i, xs[i], O.rope_table(pos + i, inv_freq), want_logits=False)[0] for i in range(len(xs))])


def cache_err(a, b, cfg, pos0, n):
    worst = 0.0
    for li in range(cfg["n_layers"]):
        ka, va = a.kv_read(li, pos0, n)
        kb, vb = b.kv_read(li, pos0, n)
        worst = max(worst, row_err(ka.reshape(n, -1), kb.reshape(n, -1).astype(np.float64)), row_err(va.reshape(n, -1), vb.reshape(n, -1).astype(np.float64)))
    return worst


@pytest.mark.parametrize("cfg", [SMALL, WIDE], ids=["small", "wide"])
@pytest.mark.parametrize("kv_f16", [False, True], ids=["f32cache", "f16cache"])
def test_prefill_steps_match_one_token_steps(backend, cfg, kv_f16):
    one, pre, inv_freq, _, keep = plans(backend, cfg, seed=1301, tokens=200, kv_f16=kv_f16)
    assert pre.tokens() == 200
    bound = 2e-3 * cfg["n_layers"]
    rng = np.random.default_rng(91)
    # token counts around the 64-token query tiles and the 128 / 256-token GEMM tiles; contexts around the 64-key tiles
    for pos, t in ((0, 1), (0, 5), (0, 64), (0, 65), (0, 200), (37, 130), (100, 63), (129, 200), (250, 129)):
        if pos:
            fill((one, pre), cfg, pos, 700 + pos)
        xs = rng.standard_normal((t, cfg["h"])).astype(np.float32)
        h1 = one_by_one(one, pos, xs, inv_freq)
        hp, none = pre.step_multi(pos, xs, rope_rows(pos, t, inv_freq))
        assert none is None
        assert row_err(hp, h1.astype(np.float64)) < bound, (pos, t, row_err(hp, h1.astype(np.float64)))
        assert cache_err(pre, one, cfg, pos, t) < bound, (pos, t)
    one.close()
    pre.close()


def test_prefill_with_q6k_and_q8_0_products(backend):
    """A body in the formats of a Q4_K_M checkpoint's heavier layers: v and down in Q6_K, o in Q8_0 (all three on the
    tensor-core GEMM in the prefill plan, on the exact matrix-vector kernels in the one-token plan)."""
    cfg = WIDE
    one, pre, inv_freq, _, keep = plans(backend, cfg, seed=1305, tokens=160, mixed=True)
    rng = np.random.default_rng(95)
    pos, t = 45, 160
    fill((one, pre), cfg, pos, 66)
    xs = rng.standard_normal((t, cfg["h"])).astype(np.float32)
    h1 = one_by_one(one, pos, xs, inv_freq)
    hp, _ = pre.step_multi(pos, xs, rope_rows(pos, t, inv_freq))
    assert row_err(hp, h1.astype(np.float64)) < 2e-3 * cfg["n_layers"]
    assert cache_err(pre, one, cfg, pos, t) < 2e-3 * cfg["n_layers"]
    one.close()
    pre.close()


def test_prefill_against_the_oracle_and_chunking(backend):
    cfg = SMALL
    one, pre, inv_freq, cpu, keep = plans(backend, cfg, seed=1302, tokens=128, interleaved=False, with_cpu=True)
    rng = np.random.default_rng(92)
    n = 96
    xs = rng.standard_normal((n, cfg["h"])).astype(np.float32)
    ref = np.stack([cpu.step(i, xs[i], O.rope_table(i, inv_freq), exact=True)[0] for i in range(n)])
    whole, _ = pre.step_multi(0, xs, rope_rows(0, n, inv_freq))
    assert row_err(whole, ref) < 4e-3
    # the same tokens in chunks of 40 (a later chunk attends to the rows the earlier ones left in the plan's caches)
    parts = []
    for c in range(0, n, 40):
        m = min(40, n - c)
        parts.append(pre.step_multi(c, xs[c:c + m], rope_rows(c, m, inv_freq))[0])
    chunks = np.concatenate(parts)
    assert row_err(chunks, ref) < 4e-3 and row_err(chunks, whole.astype(np.float64)) < 4e-3
    # prefill, hand the caches to the one-token plan (as a session does through the host caches), decode a token
    for li in range(cfg["n_layers"]):
        k, v = pre.kv_read(li, 0, n)
        one.kv_write(li, 0, k, v)
    x = rng.standard_normal(cfg["h"]).astype(np.float32)
    hid, logits = one.step(n, x, O.rope_table(n, inv_freq))
    rh, rl = cpu.step(n, x, O.rope_table(n, inv_freq), exact=True)
    assert row_err(hid[None], rh[None]) < 4e-3 and row_err(logits[None], rl[None]) < 4e-3
    one.close()
    pre.close()


def test_batched_attention_against_the_one_token_kernel(backend):
    """The same prefill plan with its attention done token by token by the decode kernel (f32 arithmetic): what the
    tensor-core attention's f16 roundings cost, separated from the products'."""
    cfg = WIDE
    out = {}
    rng = np.random.default_rng(93)
    xs = rng.standard_normal((150, cfg["h"])).astype(np.float32)
    for mode in ("rows", "loop"):
        try:
            if mode == "loop":
                os.environ["B2_PREFILL_ATTEND"] = "loop"
            one, pre, inv_freq, _, keep = plans(backend, cfg, seed=1303, tokens=150)
        finally:
            os.environ.pop("B2_PREFILL_ATTEND", None)
        fill((pre,), cfg, 70, 55)
        out[mode] = pre.step_multi(70, xs, rope_rows(70, 150, inv_freq))[0]
        one.close()
        pre.close()
    assert row_err(out["rows"], out["loop"].astype(np.float64)) < 2e-3


def test_sliding_window_and_head_norms(backend):
    """A hand-made graph: per-head q / k norms in the RoPE op and a sliding window of 48 keys in the attention."""
    nh, nkv, hd = 4, 2, 64
    nq, row = nh * hd, nkv * hd
    rng = np.random.default_rng(94)
    qn = (1 + 0.1 * rng.standard_normal(hd)).astype(np.float32)
    kn = (1 + 0.1 * rng.standard_normal(hd)).astype(np.float32)

    def graph():
        g = D.Graph()
        bq, bo, ba = g.buf(nq + 2 * row), g.buf(nq), g.buf(nq)
        g.qk_rope(bq, bo, 0, nh, nkv, hd, hd // 2, nq, nq + row, True, 1e-6, q_norm=qn, k_norm=kn)
        g.attend(bo, ba, 0, nh, nkv, hd, hd ** -0.5, window=48)
        g.input, g.n_input, g.hidden, g.n_hidden = bq, nq + 2 * row, ba, nq
        g.kv, g.rope_halves = [(nkv, hd)], [hd // 2]
        return g

    g = graph()
    one = D.decode_plan(backend, g, 512)
    pre = D.decode_plan_prefill(backend, g, 512, 256)
    assert one is not None and pre is not None, backend.last_declined
    inv = O.rope_inv_freq(hd, 1e6)
    pos, t = 30, 170
    k = rng.standard_normal((pos, row)).astype(np.float32)
    v = rng.standard_normal((pos, row)).astype(np.float32)
    one.kv_write(0, 0, k, v)
    pre.kv_write(0, 0, k, v)
    xs = rng.standard_normal((t, nq + 2 * row)).astype(np.float32)
    h1 = one_by_one(one, pos, xs, inv)
    hp, _ = pre.step_multi(pos, xs, rope_rows(pos, t, inv))
    assert row_err(hp, h1.astype(np.float64)) < 2e-3
    ka, va = one.kv_read(0, pos, t)
    kb, vb = pre.kv_read(0, pos, t)
    assert np.array_equal(ka, kb) and np.array_equal(va, vb)   # the RoPE kernel's arithmetic is the one-token one
    one.close()
    pre.close()


def test_declined_graphs_and_argument_errors(backend):
    one, pre, inv_freq, _, keep = plans(backend, SMALL, seed=1304, tokens=32, max_len=64)
    dev_layers, dhead, gp, lc, final_norm = keep
    x = np.zeros((33, SMALL["h"]), dtype=np.float32)
    with pytest.raises(ob.BackendError, match="33 tokens"):
        pre.step_multi(0, x, rope_rows(0, 33, inv_freq))
    with pytest.raises(ob.BackendError, match="64 positions"):
        pre.step_multi(40, x[:30], rope_rows(40, 30, inv_freq))
    h, _ = pre.step_multi(3, x[:30], rope_rows(3, 30, inv_freq))
    assert np.isfinite(h).all()
    # a graph with the head is the decode graph, not a prefill graph
    with_head = D.llama_graph(lc, dev_layers, final_norm, dhead)
    assert D.decode_plan_prefill(backend, with_head, 64, 32) is None and "without logits" in backend.last_declined
    assert D.decode_plan_prefill(backend, gp, 16384, 8193) is None and "8192" in backend.last_declined
    # a product in a format without a tensor-core kernel (Q5_K runs on the generic matrix-vector kernel only)
    g2 = D.llama_graph(lc, dev_layers, final_norm, dhead, prefill=True)
    q5 = backend.upload(synth.other_blocks(13, SMALL["h"], SMALL["h"], 9), SMALL["h"], SMALL["h"])
    g2.linear(q5, g2.hidden, g2.input)
    assert D.decode_plan_prefill(backend, g2, 64, 32) is None and "tensor-core" in backend.last_declined
    one.close()
    pre.close()


@pytest.mark.parametrize("hd", [64, 128])
@pytest.mark.parametrize("kv_f16", [False, True], ids=["f32cache", "f16cache"])
def test_one_query_head_per_kv_head(backend, hd, kv_f16):
    """No grouping (as many KV heads as query heads, three of them): the attention kernel's one-head-per-CTA form."""
    nh = nkv = 3
    nq = nh * hd
    g = D.Graph()
    bq, bo, ba = g.buf(3 * nq), g.buf(nq), g.buf(nq)
    g.qk_rope(bq, bo, 0, nh, nkv, hd, hd // 2, nq, 2 * nq, False, 1e-6)
    g.attend(bo, ba, 0, nh, nkv, hd, hd ** -0.5)
    g.input, g.n_input, g.hidden, g.n_hidden = bq, 3 * nq, ba, nq
    g.kv, g.rope_halves = [(nkv, hd)], [hd // 2]
    one = D.decode_plan(backend, g, 400, kv_f16=kv_f16)
    pre = D.decode_plan_prefill(backend, g, 400, 200, kv_f16=kv_f16)
    assert one is not None and pre is not None, backend.last_declined
    rng = np.random.default_rng(96 + hd)
    inv = O.rope_inv_freq(hd, 1e4)
    pos, t = 101, 133
    k = rng.standard_normal((pos, nq)).astype(np.float32)
    v = rng.standard_normal((pos, nq)).astype(np.float32)
    one.kv_write(0, 0, k, v)
    pre.kv_write(0, 0, k, v)
    xs = rng.standard_normal((t, 3 * nq)).astype(np.float32)
    h1 = one_by_one(one, pos, xs, inv)
    hp, _ = pre.step_multi(pos, xs, rope_rows(pos, t, inv))
    assert row_err(hp, h1.astype(np.float64)) < 2e-3
    one.close()
    pre.close()


def test_prefill_over_fp8_weights(backend):
    """One layer with every product in FP8 e4m3 with 128 x 128 block scales (config 4's format): the prefill plan multiplies
    them on the tensor-core GEMM (e4m3 expanded to f16), the one-token plan on its FP8 matrix-vector kernel; both within the
    FP8 bound of each other."""
    cfg = dict(n_layers=1, h=256, nh=4, nkv=2, hd=64, inter=512, vocab=512)
    shapes = {"q": (256, 256), "k": (128, 256), "v": (128, 256), "o": (256, 256), "gate": (512, 256), "up": (512, 256), "down": (256, 512)}
    rng = np.random.default_rng(97)
    L = {name: backend.upload(synth.f8_e4m3(n_out, n_in, 1400 + i), n_out, n_in) for i, (name, (n_out, n_in)) in enumerate(shapes.items())}
    L["ln_pre"] = (1.0 + 0.1 * rng.standard_normal(cfg["h"])).astype(np.float32)
    L["ln_post"] = (1.0 + 0.1 * rng.standard_normal(cfg["h"])).astype(np.float32)
    final_norm = (1.0 + 0.1 * rng.standard_normal(cfg["h"])).astype(np.float32)
    head = backend.upload(synth.f8_e4m3(cfg["vocab"], cfg["h"], 1410), cfg["vocab"], cfg["h"])
    lc = D.LlamaConfig(eps=1e-5, **cfg)
    one = D.decode_plan(backend, D.llama_graph(lc, [L], final_norm, head), 256)
    pre = D.decode_plan_prefill(backend, D.llama_graph(lc, [L], final_norm, head, prefill=True), 256, 140)
    assert one is not None and pre is not None, backend.last_declined
    inv_freq = O.rope_inv_freq(cfg["hd"], lc.rope_theta)
    pos, t = 20, 140
    fill((one, pre), cfg, pos, 71)
    xs = rng.standard_normal((t, cfg["h"])).astype(np.float32)
    h1 = one_by_one(one, pos, xs, inv_freq)
    hp, _ = pre.step_multi(pos, xs, rope_rows(pos, t, inv_freq))
    assert row_err(hp, h1.astype(np.float64)) < 4e-3   # two FP8 paths against each other: twice the 2e-3 of an FP8 row
    one.close()
    pre.close()
