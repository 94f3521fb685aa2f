"""Prefill dequant-GEMM (tcgen05) on the GPU against the pinned CPU oracle, through the C ABI.

Bound: max relative error per output row 1e-3 against the f64 product of the bit-exact dequantized
weights; the reference's CPU prefill path (f32 FMA GEMM, src/kernels.rs:1998-2038) is compared too.
"""
import numpy as np
import pytest
import torch

import oxinfer_b200 as ob
from oracle import oracle as O
from oxinfer_b200 import synth

from util import make_pair, row_err

pytestmark = pytest.mark.gpu
TOL = 1e-3


@pytest.mark.parametrize("shape", [(256, 256, 9), (512, 512, 64), (1000, 1024, 130), (208, 4096, 128), (2048, 2048, 300), (4096, 768, 512)])
def test_q4k_matmul_matches_oracle(backend, shape):
    n_out, n_in, t = shape
    ref, m = make_pair("q4_k", n_out, n_in, 400 + t)
    dev = backend.upload(ref, n_out, n_in)
    x = synth.activations(t, n_in, 401)
    y = np.full((t, n_out), np.nan, np.float32)
    assert backend.matmul(x, [ob.Job(dev, y)])
    assert np.isfinite(y).all()
    exact = m.matmul_f64(x)
    err = row_err(y, exact)
    assert err < TOL, err
    assert row_err(y, m.matmul_cpu(x)) < TOL  # the reference CPU path's own f32 result


@pytest.mark.parametrize("fmt", ["q4_k", "mlx4", "f8_e4m3"])
@pytest.mark.parametrize("t", [4, 12, 100, 300])
def test_matmul_rows_of_very_different_magnitude(backend, fmt, t):
    """Token rows scaled by 1e-3, 1, 300 and 2e5, the magnitudes of the reference's input() (src/cuda.rs:1579-1700): a row
    of 2e5 would overflow f16 and a row of 1e-3 would lose bits to its subnormals, so every row is multiplied by a power
    of two on its way to f16 and its results are scaled back in the epilogue. The reference holds its f32 kernels to
    1e-4 there; f16 operands give 1e-3 (2e-3 for FP8), the bound this engine states, at every magnitude alike."""
    n_out, n_in = 640, 1024
    ref, m = make_pair(fmt, n_out, n_in, 440 + t)
    dev = backend.upload(ref, n_out, n_in)
    x = synth.activations(t, n_in, 441) * np.array([1e-3, 1.0, 300.0, 2e5], np.float32)[np.arange(t) % 4, None]
    y = np.full((t, n_out), np.nan, np.float32)
    assert backend.matmul(x, [ob.Job(dev, y)])
    assert np.isfinite(y).all()
    exact = m.matmul_f64(x)
    errs = [row_err(y[i::4], exact[i::4]) for i in range(4)]
    print(f"{fmt} t={t}: row errors by magnitude 1e-3 / 1 / 300 / 2e5: " + " ".join(f"{e:.2e}" for e in errs))
    assert max(errs) < (2e-3 if fmt == "f8_e4m3" else TOL), errs


@pytest.mark.parametrize("fmt", ["q4_k", "mlx4"])
@pytest.mark.parametrize("shape", [(640, 1024, 100), (1000, 2048, 300), (333, 512, 9)])
def test_exact_switch_meets_the_reference_kernels_bound(backend, fmt, shape):
    """b2_set_exact (gpu::set_exact, src/gpu.rs:313-338): activations as two f16 terms and, for Q4_K, weights as two f16 terms.
    The reference holds its f32 CUDA kernels to row_err < 1e-4 against the f64 product on rows scaled by 1e-3, 1, 300 and 2e5
    (src/cuda.rs:1579-1700); with the switch on this engine's tensor-core GEMM meets the same bound on the same kind of rows."""
    n_out, n_in, t = shape
    ref, m = make_pair(fmt, n_out, n_in, 450 + t)
    dev = backend.upload(ref, n_out, n_in)
    x = synth.activations(t, n_in, 451) * np.array([1e-3, 1.0, 300.0, 2e5], np.float32)[np.arange(t) % 4, None]
    exact = m.matmul_f64(x)
    y = np.full((t, n_out), np.nan, np.float32)
    backend.set_exact(True)
    try:
        assert backend.matmul(x, [ob.Job(dev, y)])
    finally:
        backend.set_exact(False)
    err = row_err(y, exact)
    print(f"exact switch, {fmt} {shape}: row error {err:.2e}")
    assert err < 1e-4, err
    y1 = np.zeros_like(y)
    assert backend.matmul(x, [ob.Job(dev, y1)])      # and the default path afterwards is the default path again
    assert row_err(y1, exact) < TOL


def test_q4k_matmul_two_jobs_share_x_and_stats(backend):
    n_in, t = 1024, 96
    refs = [make_pair("q4_k", n, n_in, 410 + n) for n in (384, 640)]
    devs = [backend.upload(r, n, n_in) for (r, _), n in zip(refs, (384, 640))]
    x = synth.activations(t, n_in, 411)
    ys = [np.zeros((t, n), np.float32) for n in (384, 640)]
    before = backend.launch_count()
    assert backend.matmul(x, [ob.Job(d, y) for d, y in zip(devs, ys)])
    assert backend.launch_count() > before
    for (_, m), y in zip(refs, ys):
        assert row_err(y, m.matmul_f64(x)) < TOL
    assert "launches" in backend.stats()


def test_q4k_matmul_dev_bf16_in_bf16_out(backend):
    n_out, n_in, t = 1024, 2048, 256
    ref, m = make_pair("q4_k", n_out, n_in, 420)
    dev = backend.upload(ref, n_out, n_in)
    x = synth.activations(t, n_in, 421)
    xd = torch.from_numpy(x).cuda().to(torch.bfloat16)  # exact: the values are bf16-representable
    yd = torch.empty((t, n_out), device="cuda", dtype=torch.bfloat16)
    backend.set_stream(torch.cuda.current_stream().cuda_stream)
    assert backend.matmul_dev(dev, xd, yd)
    torch.cuda.synchronize()
    backend.check_status()
    backend.set_stream(0)
    exact = m.matmul_f64(x)
    assert row_err(yd.float().cpu().numpy(), exact) < 6e-3  # bf16 output rounding (2^-9) on top
    yf = torch.empty((t, n_out), device="cuda", dtype=torch.float32)
    assert backend.matmul_dev(dev, xd, yf)
    torch.cuda.synchronize()
    assert row_err(yf.cpu().numpy(), exact) < TOL


def test_q4k_matmul_full_size_config(backend):
    """M = 512, K = 4096, N = 14336: the benchmark's shape, checked on 16 of its token rows against
    the oracle and on all rows by linearity: matmul(a x1 + b x2) = a matmul(x1) + b matmul(x2)."""
    n_out, n_in, t = 14336, 4096, 512
    ref, m = make_pair("q4_k", n_out, n_in, 430)
    dev = backend.upload(ref, n_out, n_in)
    x = synth.activations(t, n_in, 431)
    x[np.abs(x) < 2.0**-10] = 0.0  # keep 2 x exact in f16 too (no f16 subnormals) for the doubling property below
    y = np.zeros((t, n_out), np.float32)
    assert backend.matmul(x, [ob.Job(dev, y)])
    rows = np.arange(0, t, 32)
    exact = m.matmul_f64(x[rows])
    assert row_err(y[rows], exact) < TOL
    # size-independent properties over all rows. (1) Reordering and doubling the tokens reorders and
    # doubles the outputs bit for bit (every output is its own k-ordered accumulation).
    perm = np.arange(t)[::-1].copy()
    x2 = (2.0 * x[perm]).astype(np.float32)
    y2 = np.zeros((t, n_out), np.float32)
    assert backend.matmul(x2, [ob.Job(dev, y2)])
    assert np.array_equal(y2, 2.0 * y[perm])
    # (2) Linearity: matmul(a x1 + b x2) = a matmul(x1) + b matmul(x2), up to the f16 rounding of the
    # combined activations (2^-12 per element).
    x3 = (0.5 * x[:256] + 0.25 * x[256:]).astype(np.float32)
    y3 = np.zeros((256, n_out), np.float32)
    assert backend.matmul(x3, [ob.Job(dev, y3)])
    assert row_err(y3, 0.5 * y[:256].astype(np.float64) + 0.25 * y[256:].astype(np.float64)) < 5e-4


@pytest.mark.parametrize("fmt", ["q6_k", "q8_0"])
@pytest.mark.parametrize("shape", [(256, 512, 64), (1000, 2048, 9), (4099, 4096, 131)])
def test_many_tokens_under_the_exact_switch_for_q6k_and_q8_0(backend, fmt, shape):
    """Q6_K and Q8_0 at t > 8 with the exact switch on: the tokens run four at a time through the multi-row matrix-vector
    kernel, so the bound is the matrix-vector one and every row equals its one-token result bit for bit (ragged token and row
    counts included)."""
    n_out, n_in, t = shape
    ref, m = make_pair(fmt, n_out, n_in, 440 + t)
    dev = backend.upload(ref, n_out, n_in)
    x = synth.activations(t, n_in, 441)
    y = np.full((t, n_out), np.nan, np.float32)
    backend.set_exact(True)
    try:
        assert backend.matmul(x, [ob.Job(dev, y)])
        assert np.isfinite(y).all()
        assert row_err(y, m.matmul_f64(x)) < 2e-5
        for i in (0, t // 2, t - 1):
            y1 = np.zeros((1, n_out), np.float32)
            assert backend.matmul(x[i:i + 1], [ob.Job(dev, y1)])
            assert np.array_equal(y1[0], y[i])
    finally:
        backend.set_exact(False)


@pytest.mark.parametrize("fmt", ["q6_k", "q8_0"])
@pytest.mark.parametrize("shape", [(256, 512, 64), (176, 256, 9), (1000, 2048, 130), (4099, 4096, 131), (4096, 768, 512), (32064, 4096, 300),
                                   (2048, 14336, 257)])
def test_q6k_and_q8_0_matmul_on_the_tensor_cores(backend, fmt, shape):
    """Q6_K and Q8_0 prefill products (t > 8) on the tcgen05 kernel: the row planes come in through the copy engine
    (128-byte rows of low nibbles / int8, Q6_K's 64-byte rows of high bit pairs through a second tensor map), are expanded to
    f16 (w = f16(d sc) (q - 32) resp. f16(d) q, the integer exact) and multiplied like the 4-bit formats. The bound is the
    prefill one: 1e-3 per row against the f64 product of the bit-exact weights; ragged row and token counts, rows that are not
    a multiple of 4 (direct stores), the vocabulary-sized head and a long K included."""
    n_out, n_in, t = shape
    ref, m = make_pair(fmt, n_out, n_in, 470 + t)
    dev = backend.upload(ref, n_out, n_in)
    x = synth.activations(t, n_in, 471)
    y = np.full((t, n_out), np.nan, np.float32)
    launches0 = backend.launch_count()
    assert backend.matmul(x, [ob.Job(dev, y)])
    assert backend.launch_count() - launches0 == 2          # the conversion to f16 and one GEMM, not t / 4 matrix-vector launches
    assert np.isfinite(y).all()
    err = row_err(y, m.matmul_f64(x))
    assert err < TOL, err
    # device-resident bf16 activations and bf16 results take the same kernel
    xd = torch.from_numpy(x).cuda().to(torch.bfloat16)
    yd = torch.zeros((t, n_out), device="cuda", dtype=torch.bfloat16)
    assert backend.matmul_dev(dev, xd, yd)
    torch.cuda.synchronize()
    exact = m.matmul_f64(xd.float().cpu().numpy())
    assert row_err(yd.float().cpu().numpy(), exact) < 6e-3   # bf16 results: 8 bits


def test_matmul_declines_what_it_cannot_take(backend):
    """A shape outside every kernel (n_in not a multiple of the block size is refused at upload; here: bf16 activations for a
    format that only has the f32 matrix-vector path) is declined with nothing written (src/gpu.rs:158-160)."""
    n_out, n_in, t = 256, 512, 64
    ref = synth.other_blocks(13, n_out, n_in, 440)   # Q5_K: the generic matrix-vector kernel only
    dev = backend.upload(ref, n_out, n_in)
    x = torch.from_numpy(synth.activations(t, n_in, 441)).cuda().to(torch.bfloat16)
    y = torch.full((t, n_out), 7.0, device="cuda", dtype=torch.float32)
    assert backend.matmul_dev(dev, x, y) is False
    torch.cuda.synchronize()
    assert bool((y == 7.0).all())


@pytest.mark.parametrize("shape", [(256, 256, 9), (4096, 4096, 64), (1536, 2048, 100), (2048, 768, 257), (1000, 1024, 512)])
def test_mlx4_matmul_matches_oracle(backend, shape):
    """MLX affine 4-bit through the same tensor-core kernel (config 0's format at prefill sizes and the
    MoE expert shapes): the oracle's weights are the reference's own repack, (nib - 8) f16(s) + bf16(b + 8 s)."""
    n_out, n_in, t = shape
    ref, m = make_pair("mlx4", n_out, n_in, 450 + t)
    dev = backend.upload(ref, n_out, n_in)
    x = synth.activations(t, n_in, 451)
    y = np.full((t, n_out), np.nan, np.float32)
    assert backend.matmul(x, [ob.Job(dev, y)])
    assert np.isfinite(y).all()
    err = row_err(y, m.matmul_f64(x))
    assert err < TOL, err
    assert row_err(y, m.matmul_cpu(x)) < TOL


@pytest.mark.parametrize("shape", [(256, 256, 9), (1000, 1024, 130), (3584, 1536, 128), (512, 12288, 64)])
def test_fp8_matmul_matches_oracle(backend, shape):
    """FP8 e4m3 weights with 128 x 128 f32 block scales: the reference's definition (e4m3 * s against f32
    activations, src/ggml.rs:433-443), bound 2e-3 per output row. The weights go through the tensor cores
    as f16 (exact e4m3 -> f16, one rounding for the scale); activations are NOT quantized to e4m3."""
    n_out, n_in, t = shape
    ref, m = make_pair("f8_e4m3", n_out, n_in, 460 + t)
    dev = backend.upload(ref, n_out, n_in)
    x = synth.activations(t, n_in, 461)
    y = np.full((t, n_out), np.nan, np.float32)
    assert backend.matmul(x, [ob.Job(dev, y)])
    assert np.isfinite(y).all()
    err = row_err(y, m.matmul_f64(x))
    assert err < 2e-3 and err < 1e-3, err
    # a row shard that starts inside the scale grid (multiple of 128 rows)
    sh = backend.shard_rows(dev, 128, n_out) if n_out > 256 else None
    if sh is not None:
        ys = np.zeros((t, n_out - 128), np.float32)
        assert backend.matmul(x, [ob.Job(sh, ys)])
        assert np.array_equal(ys, y[:, 128:])


def test_split_k_adds_two_shares(backend):
    """B2_GEMM_SPLIT_K=2: grids that fill half the SMs or less run K in two halves whose sums are added into a zeroed y
    (two shares only, so the result does not depend on which lands first). Same bound against the f64 definition, and
    within f32 reassociation of the unsplit result; a wide matrix (more CTAs than half the SMs) is not split and keeps its bits."""
    import os

    if os.environ.get("B2_GEMM_SPLIT_K"):
        pytest.skip("the split is switched on for the whole run: nothing to compare it with")
    for n_out, n_in, t, split_expected in ((1792, 4096, 512, True), (1000, 2048, 300, True), (14336, 1024, 64, False)):
        ref, m = make_pair("q4_k", n_out, n_in, 770 + n_out)
        dev = backend.upload(ref, n_out, n_in)
        x = synth.activations(t, n_in, 771)
        exact = m.matmul_f64(x)
        y1 = np.full((t, n_out), np.nan, np.float32)
        assert backend.matmul(x, [ob.Job(dev, y1)])
        os.environ["B2_GEMM_SPLIT_K"] = "2"
        try:
            y2 = np.full((t, n_out), np.nan, np.float32)
            assert backend.matmul(x, [ob.Job(dev, y2)])
            y3 = np.full((t, n_out), np.nan, np.float32)
            assert backend.matmul(x, [ob.Job(dev, y3)])
        finally:
            os.environ.pop("B2_GEMM_SPLIT_K", None)
        assert np.isfinite(y2).all() and np.array_equal(y2, y3)          # the same bits run after run
        assert row_err(y1, exact) < 1e-3 and row_err(y2, exact) < 1e-3
        assert row_err(y2, y1.astype(np.float64)) < 1e-5
        assert np.array_equal(y1, y2) == (not split_expected)


@pytest.mark.parametrize("fmt", ["q4_k", "mlx4"])
@pytest.mark.parametrize("shape", [(48, 256, 300), (1000, 512, 700), (3000, 1024, 1024), (14336, 4096, 512)])
def test_cta_pair_form_equals_the_single_cta_form(backend, fmt, shape):
    """B2_GEMM_PAIR=1: more than 256 tokens of a dense 4-bit product run as pairs of CTAs that share each weight tile (one
    M = 256 instruction over both CTAs' tokens, tcgen05 cta_group::2). Every output is the same k-ordered accumulation as in
    the single-CTA form: the results must be equal bit for bit, ragged token and row counts included, and within the bound
    of the f64 product on a sample of rows."""
    import os

    n_out, n_in, t = shape
    ref, m = make_pair(fmt, n_out, n_in, 470 + t)
    dev = backend.upload(ref, n_out, n_in)
    x = synth.activations(t, n_in, 471)
    y1 = np.full((t, n_out), np.nan, np.float32)
    assert backend.matmul(x, [ob.Job(dev, y1)])
    os.environ["B2_GEMM_PAIR"] = "1"
    try:
        y = np.full((t, n_out), np.nan, np.float32)
        assert backend.matmul(x, [ob.Job(dev, y)])
    finally:
        del os.environ["B2_GEMM_PAIR"]
    assert np.isfinite(y).all()
    rows = np.unique(np.concatenate([np.arange(0, t, 37), [t - 1, 255, 256]]))
    assert row_err(y[rows], m.matmul_f64(x[rows])) < TOL
    assert np.array_equal(y, y1)
