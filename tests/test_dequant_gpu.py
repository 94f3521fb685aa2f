"""Bit-exact dequantization on the GPU: the CUDA kernels against the reference's known-answer hashes
and against the pinned CPU oracle, through the C ABI (b2_upload_* + b2_dequantize_rows)."""
import numpy as np
import pytest

import oxinfer_b200 as ob
from oracle import oracle as O
from oxinfer_b200 import synth

from util import FORMATS, KIND, make_pair

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name,kind,fmt", [("q4_k", O.Q4_K, ob.FMT_Q4_K), ("q6_k", O.Q6_K, ob.FMT_Q6_K), ("q8_0", O.Q8_0, ob.FMT_Q8_0)])
def test_gpu_dequant_reproduces_reference_hashes(backend, name, kind, fmt):
    """REF_HASHES of src/ggml.rs:1547-1577, computed by the CUDA kernels on the reference's fixtures."""
    fx = O.fixture(kind)
    dev = backend.upload(ob.Gguf(fmt, fx), 1, O.FIXTURE_ELEMS)
    assert dev is not None
    d = backend.dequantize_rows(dev)
    assert O.fnv_f32(d) == O.REF_HASHES[kind]
    # the same blocks as a 4 x 256 matrix (rows are runs of whole blocks)
    if kind != O.Q8_0:
        dev4 = backend.upload(ob.Gguf(fmt, fx), 4, 256)
        assert O.fnv_f32(backend.dequantize_rows(dev4)) == O.REF_HASHES[kind]


def test_gpu_e4m3_every_byte_times_scale(backend):
    """src/ggml.rs:1505-1523: e4m3 * s bit for bit for every byte, NaN bytes included."""
    data = np.tile(np.arange(256, dtype=np.uint8), 2)
    for s in [1.0, 0.003741, -2.5]:
        dev = backend.upload(ob.Gguf(ob.FMT_F8E4M3, data.copy(), np.full((1, 1), s, np.float32), 128, 512), 1, 512)
        got = backend.dequantize_rows(dev)[0]
        want = O.e4m3_table()[data] * np.float32(s)
        assert np.array_equal(got.view(np.uint32)[~np.isnan(want)], want.view(np.uint32)[~np.isnan(want)])
        assert np.isnan(got[np.isnan(want)]).all()


@pytest.mark.parametrize("fmt", FORMATS)
@pytest.mark.parametrize("shape", [(8, 256), (136, 768), (300, 2048)])
def test_gpu_dequant_bit_exact_with_oracle(backend, fmt, shape):
    n_out, n_in = shape
    ref, m = make_pair(fmt, n_out, n_in, 200 + n_out)
    dev = backend.upload(ref, n_out, n_in)
    assert dev is not None and dev.bytes() > 0
    want = m.dequantize_rows()
    got = backend.dequantize_rows(dev)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    # a row range in the middle, and an empty range
    r0, r1 = n_out // 3, n_out // 3 + 5
    assert np.array_equal(backend.dequantize_rows(dev, r0, r1), want[r0:r1])
    assert backend.dequantize_rows(dev, 3, 3).shape == (0, n_in)
    # row shards share the memory and give the same bits
    sh = backend.shard_rows(dev, r0, n_out)
    assert np.array_equal(backend.dequantize_rows(sh), want[r0:])


@pytest.mark.parametrize("shape", [(8, 256), (136, 768), (300, 2048)])
def test_q4matrix_upload_gives_the_same_device_values_as_the_mlx_triple(backend, shape):
    """b2_upload_q4 takes the layout a backend is actually handed, WeightRef::Q4(&Q4Matrix) (src/gpu.rs:15-21,
    src/quant.rs:427-440): what from_mlx_q4 made of the MLX triple. Both uploads must dequantize to the same bits (and to
    dequantize_rows_q4's), and multiply to the same bits."""
    import torch

    n_out, n_in = shape
    ref, m = make_pair("mlx4", n_out, n_in, 230 + n_out)
    q, sc, off, group = m.q4_parts()
    dev_a = backend.upload(ref, n_out, n_in)
    dev_b = backend.upload(ob.Q4Matrix(q, sc, off, group), n_out, n_in)
    assert dev_b is not None, backend.last_declined
    want = m.dequantize_rows()
    a, b = backend.dequantize_rows(dev_a), backend.dequantize_rows(dev_b)
    assert np.array_equal(a.view(np.uint32), want.view(np.uint32)) and np.array_equal(b.view(np.uint32), want.view(np.uint32))
    x = synth.activations(1, n_in, 231)
    ya, yb = np.zeros((1, n_out), np.float32), np.zeros((1, n_out), np.float32)
    assert backend.matvec_rows(x, [ob.RowsJob(dev_a, ya)]) and backend.matvec_rows(x, [ob.RowsJob(dev_b, yb)])
    assert np.array_equal(ya, yb)
    # plain Q4 (no offsets: a scale per 32 weights, w = (nibble - 8) * scale, src/quant.rs:586-606) is what Q4_0 blocks hold
    # and runs through the generic kernels: bit-exact values, products within the matrix-vector bound
    dev_p = backend.upload(ob.Q4Matrix(q, sc, None, group), n_out, n_in)
    assert dev_p is not None, backend.last_declined
    nib = np.stack([q.reshape(n_out, n_in // 32, 16) & 0xF, q.reshape(n_out, n_in // 32, 16) >> 4], axis=2).reshape(n_out, n_in // 32, 32)
    plain = ((nib.astype(np.float32) - 8.0) * sc.view(np.float16).astype(np.float32).reshape(n_out, n_in // 32, 1)).reshape(n_out, n_in)
    assert np.array_equal(backend.dequantize_rows(dev_p).view(np.uint32), plain.view(np.uint32))
    yp = np.zeros((1, n_out), np.float32)
    assert backend.matvec_rows(x, [ob.RowsJob(dev_p, yp)])
    from util import row_err
    assert row_err(yp, x.astype(np.float64) @ plain.astype(np.float64).T) < 2e-5
    # a matrix whose 64-groups do not share a scale is declined
    sc2 = sc.copy()
    sc2[1] ^= 1
    assert backend.upload(ob.Q4Matrix(q, sc2, off, group), n_out, n_in) is None and "differ in scale" in backend.last_declined


def test_gpu_dequant_golden(backend):
    from pathlib import Path

    g = np.load(Path(__file__).parent / "golden" / "oracle_small.npz")
    for fmt in FORMATS:
        n_out, n_in = int(g[f"{fmt}_shape"][0]), int(g[f"{fmt}_shape"][1])
        ref = synth.make(fmt, n_out, n_in, int(g[f"{fmt}_seed"]))
        dev = backend.upload(ref, n_out, n_in)
        assert O.fnv_f32(backend.dequantize_rows(dev)) == int(g[f"{fmt}_deq_fnv"])


def test_upload_rejects_bad_shapes(backend):
    assert backend.upload(ob.Gguf(ob.FMT_Q4_K, np.zeros(144, np.uint8)), 1, 128) is None  # n_in not a multiple of 256
    assert backend.upload(ob.Gguf(9, np.zeros(36, np.uint8)), 1, 32) is None              # Q8_1: no device kernels
    with pytest.raises(ob.BackendError):
        backend.dequantize_rows(ob.DeviceWeight(backend, 99999, 1, 256, ob.FMT_Q4_K))
