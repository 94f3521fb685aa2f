"""Pins the CPU oracle to the reference's own known answers and invariants (no GPU needed).

Sources of truth, all from the reference tree:
  - REF_HASHES (src/ggml.rs:1547-1577) over fixture(kind) = random_blocks(kind, 1024 / block, 1000 + id)
    (src/ggml.rs:1437-1496, 1535-1541): the dequantized values of Q4_K, Q6_K, Q8_0, F16, BF16, F32 and of
    Q4_0, Q4_1, Q5_0, Q5_1, Q2_K, Q3_K, Q5_K, IQ4_NL, IQ4_XS, MXFP4.
  - e4m3: the closed form of src/ggml.rs:258-271 for all 256 bytes (test e4m3_scaled_matches_the_table).
  - f16 / bf16 conversions: IEEE round-to-nearest-even (crate half 2.7.1), checked against numpy for
    every f16 value (the reference's f16c_matches_software_conversion, src/kernels_x86.rs:592-606).
  - MLX repack error < 2e-4 of the row's range (mlx_affine_q4_matches_reference, src/kernels.rs:2458-2502).
  - multi-token == one-token results (src/ggml.rs:1829-1848), decode vs exact within 1e-2 / 3e-2.
"""
import math

import numpy as np
import pytest

from oracle import oracle as O
from oxinfer_b200 import synth

from util import FORMATS, make_pair, row_err


@pytest.mark.parametrize("kind", [O.Q4_K, O.Q6_K, O.Q8_0, O.F16, O.BF16, O.F32, *O.OTHER_KINDS])
def test_dequantization_matches_reference_hashes(kind):
    d = O.dequantize_row(kind, O.fixture(kind), O.FIXTURE_ELEMS)
    assert O.fnv_f32(d) == O.REF_HASHES[kind]


def test_lcg_matches_its_definition():
    import ctypes as C

    s = C.c_uint64(12345)
    v = O.lib().orc_lcg(C.byref(s))
    exp = (12345 * 6364136223846793005 + 1442695040888963407) % 2**64
    assert s.value == exp and v == exp >> 33


def test_e4m3_every_byte():
    tab = O.e4m3_table()
    for b in range(256):
        e, m = (b >> 3) & 0xF, b & 7
        if e == 0xF and m == 7:
            assert math.isnan(tab[b])
            continue
        v = m / 8.0 * 2.0**-6 if e == 0 else (1 + m / 8.0) * 2.0 ** (e - 7)
        v = -v if b & 0x80 else v
        assert tab[b] == np.float32(v), hex(b)
    assert tab[0x7E] == 448.0 and tab[0x01] == 2.0**-9


def test_e4m3_encoder_round_trips_and_rounds_to_nearest_even():
    tab = O.e4m3_table()
    L = O.lib()
    for b in range(256):
        if (b & 0x7F) == 0x7F:
            continue
        back = L.orc_f32_to_e4m3(float(tab[b]))
        assert tab[back] == tab[b], hex(b)
    # ties go to the even mantissa; saturation at 448
    assert tab[L.orc_f32_to_e4m3(1.0625)] == 1.0       # halfway 1.0 / 1.125 -> even (1.0)
    assert tab[L.orc_f32_to_e4m3(1.1875)] == 1.25      # halfway 1.125 / 1.25 -> even (1.25)
    assert tab[L.orc_f32_to_e4m3(1000.0)] == 448.0 and tab[L.orc_f32_to_e4m3(-1000.0)] == -448.0
    # against torch's converter on random in-range values
    import torch

    x = np.random.default_rng(0).uniform(-440, 440, 4096).astype(np.float32)
    mine = np.array([L.orc_f32_to_e4m3(float(v)) for v in x], dtype=np.uint8)
    ref = torch.from_numpy(x).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    assert np.array_equal(tab[mine], tab[ref])


def test_f16_conversion_every_value():
    L = O.lib()
    allh = np.arange(65536, dtype=np.uint16)
    ref = allh.view(np.float16).astype(np.float32)
    for h in range(65536):
        v = L.orc_f16_to_f32(h)
        if np.isnan(ref[h]):
            assert math.isnan(v)
        else:
            assert v == ref[h]
            assert L.orc_f32_to_f16(float(ref[h])) == h or ref[h] == 0
    x = np.random.default_rng(1).standard_normal(20000).astype(np.float32) * np.float32(10.0) ** np.random.default_rng(2).integers(-8, 5, 20000)
    mine = np.array([L.orc_f32_to_f16(float(v)) for v in x], dtype=np.uint16)
    assert np.array_equal(mine, x.astype(np.float16).view(np.uint16))


def test_bf16_round_to_nearest_even():
    L = O.lib()
    x = np.random.default_rng(3).standard_normal(5000).astype(np.float32)
    mine = np.array([L.orc_f32_to_bf16(float(v)) for v in x], dtype=np.uint16)
    assert np.array_equal(mine, synth.f32_to_bf16_bits(x))
    assert L.orc_f32_to_bf16(float(np.float32(1.0) + np.float32(2.0**-8))) == 0x3F80  # tie -> even


def test_quantize_act_properties():
    x = np.random.default_rng(4).standard_normal((3, 256)).astype(np.float32)
    x[1, 32:64] = 0.0
    q, scales, sums, fsums, hsums = O.quantize_act(x)
    xb = x.reshape(3, 8, 32)
    amax = np.abs(xb).max(axis=2)
    assert np.array_equal(scales, (amax / np.float32(127.0)).astype(np.float32))
    assert np.abs(q).max() <= 127 and (q[1, 32:64] == 0).all()
    assert np.array_equal(sums, q.reshape(3, 8, 32).sum(axis=2))
    deq = q.reshape(3, 8, 32) * scales[..., None]
    assert np.abs(deq - xb).max() <= (scales.max() / 2) * 1.0001
    assert np.allclose(fsums, xb.sum(axis=2), atol=1e-5) and np.allclose(hsums.reshape(3, 8, 2), xb.reshape(3, 8, 2, 16).sum(axis=3), atol=1e-5)
    # round half away from zero
    x2 = np.zeros((1, 32), np.float32)
    x2[0, 0], x2[0, 1], x2[0, 2] = 127.0, 0.5, -0.5
    q2 = O.quantize_act(x2)[0]
    assert q2[0, 0] == 127 and q2[0, 1] == 1 and q2[0, 2] == -1


def test_route_top_k_order_ties_and_weights():
    logits = np.array([0.5, 2.0, 2.0, -1.0, 0.5, 3.0], dtype=np.float32)
    ids, w = O.route_top_k(logits, 4)
    assert list(ids) == [5, 1, 2, 0]  # ties to the lower index
    e = np.exp(logits[ids] - logits[ids[0]])
    assert np.allclose(w, e / e.sum(), rtol=1e-6) and abs(w.sum() - 1) < 1e-6


def test_mlx_repack_error_and_layout():
    n_out, n_in = 16, 512
    ref, m = make_pair("mlx4", n_out, n_in, 7)
    deq = m.dequantize_rows()
    for r in range(n_out):
        exact = O.mlx_dequant_row(ref.w[r], ref.scales[r], ref.biases[r], 64, n_in)
        rng = exact.max() - exact.min()
        assert np.abs(deq[r] - exact).max() < 2e-4 * rng  # src/kernels.rs:2484-2491
    # nibble e of a row is (w[e/8] >> 4 (e%8)) & 15 and the value is (nib - 8) d + offset
    s = synth.bf16_bits_to_f32(ref.scales[0, 0:1])[0]
    b = synth.bf16_bits_to_f32(ref.biases[0, 0:1])[0]
    off = synth.bf16_round(np.array([np.float32(b) + np.float32(8.0) * np.float32(s)], np.float32))[0]
    nib = (int(ref.w[0, 0]) >> 4) & 15
    assert deq[0, 1] == np.float32(np.float32(nib - 8) * np.float32(s)) + off


@pytest.mark.parametrize("fmt", FORMATS)
def test_prefill_path_matches_f64_product(fmt):
    """The f32 GEMM arithmetic (sequential FMA) stays within 1e-4 of the f64 definition (src/cuda.rs:1684)."""
    n_out, n_in, t = 48, 512, 9
    _, m = make_pair(fmt, n_out, n_in, 11)
    x = synth.activations(t, n_in, 12)
    exact = m.matmul_f64(x)
    assert row_err(m.matmul_cpu(x), exact) < 1e-4
    assert np.array_equal(m.matmul_cpu(x), m.matmul_prefill(x))  # t > 7: the CPU path IS the prefill GEMM


@pytest.mark.parametrize("fmt", ["mlx4", "q4_k", "q6_k", "q8_0"])
def test_decode_path_is_int8_approximate_and_token_independent(fmt):
    n_out, n_in = 64, 1024
    _, m = make_pair(fmt, n_out, n_in, 13)
    x = synth.activations(4, n_in, 14)
    y = m.matmul_cpu(x)
    exact = m.matmul_f64(x)
    err = row_err(y, exact)
    assert 1e-6 < err < 3e-2, err  # approximate by design (src/cuda.rs:1686-1690, src/ggml.rs:1903)
    for i in range(4):  # multi-token == one-token, bit for bit (src/ggml.rs:1829-1848)
        assert np.array_equal(m.matmul_cpu(x[i : i + 1])[0], y[i])
    # thread count does not change a bit
    assert np.array_equal(m.matmul_cpu(x, threads=1), m.matmul_cpu(x, threads=4))


def test_fp8_is_dense_f32_path_at_one_token():
    """FP8 matrices take f32 activations at every t (src/ggml.rs:220-225, 433-443)."""
    _, m = make_pair("f8_e4m3", 256, 512, 15)
    x = synth.activations(1, 512, 16)
    assert row_err(m.matmul_cpu(x), m.matmul_f64(x)) < 1e-5


def test_encoders_produce_blocks_that_decode_close():
    rng = np.random.default_rng(17)
    w = (0.02 * rng.standard_normal(4096)).astype(np.float32)
    for kind, tol in [(O.Q8_0, 0.01), (O.Q4_K, 0.12), (O.Q6_K, 0.04)]:
        blk = O.encode(kind, w)
        d = O.dequantize_row(kind, blk, w.size)
        assert np.abs(d - w).max() < tol * np.abs(w).max(), kind


def test_golden_vectors():
    """Outputs of the pinned oracle on small seeded cases, committed as fixtures (tests/golden)."""
    from pathlib import Path

    g = np.load(Path(__file__).parent / "golden" / "oracle_small.npz")
    for fmt in FORMATS:
        n_out, n_in, t = int(g[f"{fmt}_shape"][0]), int(g[f"{fmt}_shape"][1]), int(g[f"{fmt}_shape"][2])
        _, m = make_pair(fmt, n_out, n_in, int(g[f"{fmt}_seed"]))
        x = synth.activations(t, n_in, int(g[f"{fmt}_seed"]) + 1)
        assert O.fnv_f32(m.dequantize_rows()) == int(g[f"{fmt}_deq_fnv"])
        assert np.array_equal(m.matmul_prefill(x), g[f"{fmt}_y_prefill"])
        assert np.array_equal(m.matmul_f64(x), g[f"{fmt}_y_f64"])


def test_avx2_decode_kernels_give_the_bits_of_the_scalar_restatements():
    """The reference's own invariant (src/kernels_ggml_x86.rs:576-624; src/kernels_x86.rs tests): its AVX2 decode kernels
    equal the portable ones bit for bit. The oracle's AVX2 kernels (the ones timed as the CPU baseline) are held to its
    scalar restatements the same way, for every format, one to seven rows, odd row counts and several thread counts."""
    from oxinfer_b200 import synth

    from util import oracle_matrix

    for fmt, n_out, n_in in [("mlx4", 77, 1024), ("q4_k", 50, 768), ("q6_k", 33, 512), ("q8_0", 41, 256)]:
        ref = synth.make(fmt, n_out, n_in, 60)
        m = oracle_matrix(ref, n_out, n_in)
        for t in (1, 2, 7):
            x = synth.activations(t, n_in, 61 + t) * np.float32(1.7)
            O.set_decode_scalar(True)
            try:
                want = m.matmul_cpu(x, 3)
            finally:
                O.set_decode_scalar(False)
            for threads in (1, 4):
                got = m.matmul_cpu(x, threads)
                assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), (fmt, t, threads)


def test_nvfp4_decode_matches_its_closed_form():
    """NVFP4 has no known-answer hash in the reference; the decode arm (src/ggml.rs:936-947, ue4m3_half :477-491) is a closed form:
    value = ue4m3(scale byte) / 2 * (doubled E2M1 value), checked here for all 256 scale bytes x 16 codes, with the layout
    of a block (four scale bytes, then eight bytes per 16 values: element j in the low nibble, j + 8 in the high one)."""
    kv = np.array([0, 1, 2, 3, 4, 6, 8, 12, 0, -1, -2, -3, -4, -6, -8, -12], np.float64)
    scale = np.zeros(256)
    for x in range(256):
        if x in (0, 0x7F):
            continue
        e, m = (x >> 3) & 0xF, x & 7
        scale[x] = (m * 2.0**-9 if e == 0 else (1 + m / 8) * 2.0 ** (e - 7)) * 0.5
    blocks = np.zeros((64, 36), np.uint8)       # block i: scale bytes 4 i .. 4 i + 3, codes cycling so every pair occurs
    for i in range(64):
        blocks[i, :4] = np.arange(4 * i, 4 * i + 4)
        blocks[i, 4:] = (np.arange(32) * 37 + 11 * i) % 256
    got = O.dequantize_row(O.NVFP4, blocks.reshape(-1), 64 * 64).reshape(64, 4, 16)
    for i in range(64):
        for s in range(4):
            q = blocks[i, 4 + 8 * s: 12 + 8 * s]
            want = np.concatenate([kv[q & 0xF], kv[q >> 4]]) * scale[4 * i + s]
            assert np.array_equal(got[i, s].astype(np.float64), want), (i, s)
    # a global scale on top (BlockScales over the whole matrix, src/ggml.rs:420-432)
    m = O.Matrix.gguf(O.NVFP4, blocks.reshape(-1), 4, 1024, np.array([[0.37]], np.float32), 4, 1024)
    assert np.array_equal(m.dequantize_rows(), (got.reshape(4, 1024) * np.float32(0.37)).astype(np.float32))
