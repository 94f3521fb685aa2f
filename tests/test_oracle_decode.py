"""The oracle's decode-step pieces against independent numpy / float64 restatements (CPU only).

The reference pins these functions by their own unit tests on closed forms (rotation preserves the pair norm, a
softmax sums to one, fast_exp within 1e-6 of exp: src/kernels.rs tests); there are no golden vectors for them, so the
checks here are the same closed forms plus a float64 attention."""
import numpy as np

from oracle import oracle as O


def test_fast_exp_and_softmax():
    xs = np.linspace(-80, 80, 4001).astype(np.float32)
    got = np.array([O.lib().orc_fast_exp(float(v)) for v in xs], dtype=np.float64)
    assert np.max(np.abs(got / np.exp(xs.astype(np.float64)) - 1)) < 1e-6   # "relative error ~1e-7", src/kernels.rs:2224
    s = O.softmax(np.array([0.5, -1.0, 3.0, 3.0], np.float32))
    assert abs(s.sum() - 1) < 1e-6 and s[2] == s[3] and s[1] < s[0] < s[2]


def test_rmsnorm_matches_float64():
    rng = np.random.default_rng(1)
    x = rng.standard_normal(4096).astype(np.float32)
    w = (1 + 0.1 * rng.standard_normal(4096)).astype(np.float32)
    ref = x.astype(np.float64) / np.sqrt(np.mean(x.astype(np.float64) ** 2) + 1e-5) * w
    assert np.max(np.abs(O.rmsnorm_f32w(x, w, 1e-5) - ref)) < 2e-6 * np.max(np.abs(ref))


def test_rope_tables_and_rotation():
    f = O.rope_inv_freq(128, 500000.0)
    assert f[0] == 1.0 and abs(f[1] - 500000.0 ** (-2 / 128)) < 1e-7 and f.size == 64
    half = O.rope_inv_freq(128, 10000.0, 0.5)
    assert np.all(half[32:] == 0) and np.all(half[:32] > 0)     # "proportional" RoPE: zeros past the rotated part
    cs = O.rope_table(1234, f)
    a = np.float32(1234) * f
    assert np.max(np.abs(cs[:64] - np.cos(a.astype(np.float64)))) < 1e-6
    rng = np.random.default_rng(2)
    v = rng.standard_normal(128).astype(np.float32)
    for inter in (True, False):
        r = O.apply_rope(v, cs, inter)
        pairs = (lambda z: z.reshape(64, 2)) if inter else (lambda z: np.stack([z[:64], z[64:]], 1))
        assert np.allclose(np.linalg.norm(pairs(r), axis=1), np.linalg.norm(pairs(v), axis=1), rtol=1e-5)
        # position 0 is the identity
        assert np.array_equal(O.apply_rope(v, O.rope_table(0, f), inter), v)


def test_attention_matches_float64():
    rng = np.random.default_rng(3)
    nh, nkv, hd, n = 8, 2, 64, 300
    q = rng.standard_normal((nh, hd)).astype(np.float32) * 0.3
    kc = rng.standard_normal((n, nkv, hd)).astype(np.float32)
    vc = rng.standard_normal((n, nkv, hd)).astype(np.float32)
    for lo in (0, 100):
        got = O.attention(q, kc, vc, n, nh, nkv, hd, lo=lo).reshape(nh, hd)
        for h in range(nh):
            k = kc[lo:, h // (nh // nkv)].astype(np.float64)
            s = k @ q[h].astype(np.float64)
            p = np.exp(s - s.max())
            ref = (p / p.sum()) @ vc[lo:, h // (nh // nkv)].astype(np.float64)
            assert np.max(np.abs(got[h] - ref)) < 1e-5
