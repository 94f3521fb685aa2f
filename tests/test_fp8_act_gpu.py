"""FP8 weights x FP8 activations (b2_set_fp8_activations; tcgen05 kind::f8f6f4) against the CPU oracle, through the C ABI.

The reference multiplies FP8 weights by unquantized activations (src/ggml.rs:433-443) and has no f32 -> e4m3 encoder, so the
oracle for this mode applies the same activation quantizer on the CPU (orc_quantize_act_e4m3: per token and per 128 k,
scale = amax / 448, round to nearest even, saturate at 448), dequantizes, and takes the f64 product with the bit-exact
dequantized weights. Both operands are then exactly what the tensor cores multiply, so the bound is tight (1e-5 per output
row: f32 accumulation of 128-k partial sums) and a single activation quantized differently on the GPU would show. The
distance to the reference's own definition (unquantized activations) is e4m3's quantization noise; it is reported and
bounded loosely.
"""
import numpy as np
import pytest
import torch

import oxinfer_b200 as ob
from oracle import oracle as O
from oxinfer_b200 import synth

from util import make_pair, row_err

pytestmark = pytest.mark.gpu


def oracle_fp8_act(m, x):
    q, s = O.quantize_act_e4m3(x, 128)
    xq = (O.e4m3_table()[q].astype(np.float64).reshape(x.shape[0], -1, 128) * s.astype(np.float64)[:, :, None]).reshape(x.shape)
    return m.matmul_f64(xq.astype(np.float32)), xq


@pytest.fixture
def fp8_backend(backend):
    backend.set_fp8_activations(True)
    yield backend
    backend.set_fp8_activations(False)


@pytest.mark.parametrize("shape", [(512, 1024, 100), (1000, 2048, 300), (256, 128, 1), (2304, 4096, 9), (640, 12288, 130)])
def test_fp8_activation_matmul_matches_oracle_with_the_same_quantizer(fp8_backend, shape):
    n_out, n_in, t = shape
    ref, m = make_pair("f8_e4m3", n_out, n_in, 500 + t)
    dev = fp8_backend.upload(ref, n_out, n_in)
    x = synth.activations(t, n_in, 501) * np.array([1e-3, 1.0, 300.0, 2e5], np.float32)[np.arange(t) % 4, None]
    x[0, :128] = 0.0                      # an all-zero block: scale 1, all quants zero
    y = np.full((t, n_out), np.nan, np.float32)
    assert fp8_backend.matmul(x, [ob.Job(dev, y)])
    want, xq = oracle_fp8_act(m, x)
    err = row_err(y, want)
    far = row_err(y, m.matmul_f64(x))
    print(f"fp8 x fp8 {shape}: row error {err:.2e} against the oracle with the same quantizer, {far:.2e} against unquantized activations")
    assert err < 1e-5, err
    assert far < 1e-1


def test_fp8_activation_matmul_bf16_output_and_row_shards(fp8_backend):
    n_out, n_in, t = 1024, 2048, 260
    ref, m = make_pair("f8_e4m3", n_out, n_in, 510)
    dev = fp8_backend.upload(ref, n_out, n_in)
    x = synth.activations(t, n_in, 511)
    want, _ = oracle_fp8_act(m, x)
    xd = torch.from_numpy(x).cuda().to(torch.bfloat16)   # exact: the values are bf16-representable
    yd = torch.empty((t, n_out), device="cuda", dtype=torch.bfloat16)
    fp8_backend.set_stream(torch.cuda.current_stream().cuda_stream)
    try:
        assert fp8_backend.matmul_dev(dev, xd, yd)
        yf = torch.empty((t, n_out), device="cuda", dtype=torch.float32)
        assert fp8_backend.matmul_dev(dev, xd, yf)
        # a row shard that starts on a scale-block boundary: the same bits as the unsharded rows
        sh = fp8_backend.shard_rows(dev, 384, 896)
        ys = torch.empty((t, 512), device="cuda", dtype=torch.float32)
        assert fp8_backend.matmul_dev(sh, xd, ys)
        torch.cuda.synchronize()
        fp8_backend.check_status()
    finally:
        fp8_backend.set_stream(0)
    assert row_err(yf.cpu().numpy(), want) < 1e-5
    assert row_err(yd.float().cpu().numpy(), want) < 6e-3   # bf16 output rounding
    assert torch.equal(ys, yf[:, 384:896])


def test_default_keeps_the_reference_definition(backend):
    """Without the switch FP8 weights multiply unquantized activations (src/ggml.rs:433-443), within the FP8 bound 2e-3."""
    n_out, n_in, t = 512, 1024, 64
    ref, m = make_pair("f8_e4m3", n_out, n_in, 520)
    dev = backend.upload(ref, n_out, n_in)
    x = synth.activations(t, n_in, 521)
    y = np.zeros((t, n_out), np.float32)
    assert backend.matmul(x, [ob.Job(dev, y)])
    assert row_err(y, m.matmul_f64(x)) < 2e-3


@pytest.mark.parametrize("shape", [(1000, 2048, 700), (2304, 4096, 1024), (256, 256, 129)])
def test_fp8_cta_pair_form_equals_the_single_cta_form(fp8_backend, shape):
    """B2_F8_PAIR=1: more than 128 tokens run as pairs of CTAs that share each weight tile (M = 256 instructions, tcgen05
    cta_group::2). Each output is the same sequence of 128-k partial sums promoted in the same order: the results must be
    equal to the single-CTA form's bit for bit, ragged token and row counts included."""
    import os

    n_out, n_in, t = shape
    ref, m = make_pair("f8_e4m3", n_out, n_in, 520 + t)
    dev = fp8_backend.upload(ref, n_out, n_in)
    x = synth.activations(t, n_in, 521)
    y1 = np.full((t, n_out), np.nan, np.float32)
    assert fp8_backend.matmul(x, [ob.Job(dev, y1)])
    os.environ["B2_F8_PAIR"] = "1"
    try:
        y = np.full((t, n_out), np.nan, np.float32)
        assert fp8_backend.matmul(x, [ob.Job(dev, y)])
    finally:
        del os.environ["B2_F8_PAIR"]
    assert np.isfinite(y).all()
    assert np.array_equal(y, y1)
    rows = np.unique(np.concatenate([np.arange(0, t, 53), [t - 1, 127, 128]]))
    want, _ = oracle_fp8_act(m, x[rows])
    assert row_err(y[rows], want) < 1e-5
