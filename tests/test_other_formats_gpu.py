"""The other GGUF block formats (Q4_0, Q4_1, Q5_0, Q5_1, Q2_K, Q3_K, Q5_K, IQ4_NL, IQ4_XS, MXFP4) on the GPU, through the C ABI:
the reference's known-answer hashes (src/ggml.rs:1547-1577) reproduced by the CUDA decoders, bit-exact rows against the pinned
oracle, and matrix-vector / several-token products against the f64 product of the decoded weights."""
import numpy as np
import pytest

import oxinfer_b200 as ob
from oracle import oracle as O
from oxinfer_b200 import synth

from util import row_err

pytestmark = pytest.mark.gpu

KINDS = list(O.OTHER_KINDS)
IDS = [O.KIND_NAMES[k] for k in KINDS]


def blocks(kind, n_out, n_in, seed):
    data, _ = O.random_blocks(kind, n_out * n_in // O.block_size(kind), seed)
    return ob.Gguf(kind, data), O.Matrix.gguf(kind, data, n_out, n_in, None, 0, 0)


@pytest.mark.parametrize("kind", KINDS, ids=IDS)
def test_gpu_decoders_reproduce_reference_hashes(backend, kind):
    fx = O.fixture(kind)
    dev = backend.upload(ob.Gguf(kind, fx), 1, O.FIXTURE_ELEMS)
    assert dev is not None
    assert O.fnv_f32(backend.dequantize_rows(dev)) == O.REF_HASHES[kind]
    dev4 = backend.upload(ob.Gguf(kind, fx), 4, 256)  # the same blocks as four rows
    assert O.fnv_f32(backend.dequantize_rows(dev4)) == O.REF_HASHES[kind]


@pytest.mark.parametrize("kind", KINDS, ids=IDS)
@pytest.mark.parametrize("shape", [(8, 256), (77, 768), (300, 2048)])
def test_rows_bit_exact_with_oracle_and_shards(backend, kind, shape):
    n_out, n_in = shape
    ref, m = blocks(kind, n_out, n_in, 31 * kind + n_out)
    dev = backend.upload(ref, n_out, n_in)
    want = m.dequantize_rows()
    got = backend.dequantize_rows(dev)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    r0 = n_out // 3
    assert np.array_equal(backend.dequantize_rows(dev, r0, r0 + 5), want[r0 : r0 + 5])
    assert backend.dequantize_rows(dev, 3, 3).shape == (0, n_in)
    sh = backend.shard_rows(dev, r0, n_out)
    assert np.array_equal(backend.dequantize_rows(sh), want[r0:])


@pytest.mark.parametrize("kind", KINDS, ids=IDS)
@pytest.mark.parametrize("shape", [(64, 256), (333, 1024), (1024, 4096)])
def test_matvec_and_several_tokens(backend, kind, shape):
    n_out, n_in = shape
    ref, m = blocks(kind, n_out, n_in, 7 * kind + n_in)
    dev = backend.upload(ref, n_out, n_in)
    w64 = m.dequantize_rows().astype(np.float64)
    x = synth.activations(11, n_in, 5 + kind)
    want = x.astype(np.float64) @ w64.T
    # one token through the device-pointer matrix-vector entry point (the decode path)
    y1 = np.zeros((1, n_out), np.float32)
    assert backend.matmul(x[:1], [ob.Job(dev, y1)])
    assert row_err(y1, want[:1]) < 2e-5
    # 11 tokens: four at a time, every row the one-token result bit for bit (src/ggml.rs:1829-1848)
    y = np.zeros((11, n_out), np.float32)
    assert backend.matmul(x, [ob.Job(dev, y)])
    assert row_err(y, want) < 2e-5
    assert np.array_equal(y[0].view(np.uint32), y1[0].view(np.uint32))
    for i in (3, 4, 10):
        yi = np.zeros((1, n_out), np.float32)
        assert backend.matmul(x[i : i + 1], [ob.Job(dev, yi)])
        assert np.array_equal(yi[0].view(np.uint32), y[i].view(np.uint32))
    # the speculative-decode form, and a row shard computing its slice of the full product
    yr = np.zeros((3, n_out), np.float32)
    assert backend.matvec_rows(x[:3], [ob.RowsJob(dev, yr)])
    assert np.array_equal(yr.view(np.uint32), y[:3].view(np.uint32))
    r0 = n_out // 4
    sh = backend.shard_rows(dev, r0, n_out)
    ys = np.zeros((1, n_out - r0), np.float32)
    assert backend.matmul(x[:1], [ob.Job(sh, ys)])
    assert np.array_equal(ys[0].view(np.uint32), y1[0, r0:].view(np.uint32))


@pytest.mark.parametrize("kind", [O.Q4_0, O.Q5_K, O.MXFP4], ids=["q4_0", "q5_k", "mxfp4"])
def test_gate_up_pair(backend, kind):
    n_out, n_in = 512, 1024
    g_ref, g_m = blocks(kind, n_out, n_in, 11)
    u_ref, u_m = blocks(kind, n_out, n_in, 12)
    g, u = backend.upload(g_ref, n_out, n_in), backend.upload(u_ref, n_out, n_in)
    x = synth.activations(2, n_in, 3) * 0.01
    y = np.zeros((2, n_out), np.float32)
    assert backend.matvec_rows(x, [ob.RowsJob(g, y, u)])
    a = x.astype(np.float64) @ g_m.dequantize_rows().astype(np.float64).T
    b = x.astype(np.float64) @ u_m.dequantize_rows().astype(np.float64).T
    with np.errstate(over="ignore"):
        want = a / (1.0 + np.exp(-a)) * b
    assert row_err(y, want) < 1e-4


def test_formats_without_a_device_path_are_declined(backend):
    # Q8_1 (id 9) has no device kernels; plans and expert stacks decline the generic formats.
    assert backend.upload(ob.Gguf(9, np.zeros(36 * 8, np.uint8)), 1, 256) is None
    ref, _ = blocks(O.Q4_0, 256, 256, 1)
    dev = backend.upload(ref, 256, 256)
    assert backend.upload_moe([dev], [dev], 256, 256) is None


@pytest.mark.parametrize("gscale", [None, 0.0371])
def test_nvfp4_rows_and_products(backend, gscale):
    """NVFP4 (blocks of 64, an unsigned E4M3 scale per 16, optionally the tensor's global scale): rows bit-exact with the oracle
    (which is pinned to the closed form on the CPU; the reference holds no hash for this type), products within the bound."""
    n_out, n_in = 300, 2048
    data, _ = O.random_blocks(O.NVFP4, n_out * n_in // 64, 4040)
    bs = None if gscale is None else np.array([[gscale]], np.float32)
    ref = ob.Gguf(O.NVFP4, data, bs, n_out, n_in)
    m = O.Matrix.gguf(O.NVFP4, data, n_out, n_in, bs, n_out, n_in)
    dev = backend.upload(ref, n_out, n_in)
    assert dev is not None, backend.last_declined
    want = m.dequantize_rows()
    assert np.array_equal(backend.dequantize_rows(dev).view(np.uint32), want.view(np.uint32))
    sh = backend.shard_rows(dev, 101, n_out)
    assert np.array_equal(backend.dequantize_rows(sh), want[101:])
    x = synth.activations(5, n_in, 41)
    y = np.zeros((5, n_out), np.float32)
    assert backend.matmul(x, [ob.Job(dev, y)])
    assert row_err(y, x.astype(np.float64) @ want.astype(np.float64).T) < 2e-5
    y1 = np.zeros((1, n_out), np.float32)
    assert backend.matmul(x[4:5], [ob.Job(dev, y1)])
    assert np.array_equal(y1[0].view(np.uint32), y[4].view(np.uint32))
    # scale blocks that are not one value for the whole matrix are declined
    assert backend.upload(ob.Gguf(O.NVFP4, data, np.ones((3, 16), np.float32), 128, 128), n_out, n_in) is None
