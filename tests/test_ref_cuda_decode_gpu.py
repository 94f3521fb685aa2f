"""The decode ops around the products against the reference's OWN CUDA kernels (dnorm, dqk_rope, dattn_* + dattn_combine
and dglu of src/cuda_decode.cu, the prefill kernel gemm_q4a of src/cuda.rs; compiled into oracle/_ref by
oracle/build_ref.py where the reference's tree is present). Each op runs through a decode plan of one or two ops on the
same inputs as the reference kernel. Both sides compute in f32 with different summation orders, so the bound is 1e-5 of
the vector's largest magnitude (`row_err`); RoPE and the cache rows are elementwise and must agree to 1e-6."""
import numpy as np
import pytest
import torch

import oxinfer_b200 as ob
from oracle import oracle as O
from oxinfer_b200 import decode as D
from oxinfer_b200 import synth

from util import oracle_matrix, row_err

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ref():
    L = O.ref_cuda()
    if L is None:
        pytest.skip("oracle/_ref/libref_cuda.so was not built (the reference's tree is not on this machine)")
    return L


def cuda(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


@pytest.mark.parametrize("n", [256, 4096, 5120])
@pytest.mark.parametrize("weighted", [True, False])
def test_norm_matches_reference_dnorm(backend, ref, n, weighted):
    rng = np.random.default_rng(n)
    x = (rng.standard_normal(n) * 3).astype(np.float32)
    w = (1 + 0.1 * rng.standard_normal(n)).astype(np.float32) if weighted else None
    g = D.Graph()
    bx, bo = g.buf(n), g.buf(n)
    g.norm(bx, bo, w, n, 1e-5)
    g.input, g.n_input, g.hidden, g.n_hidden = bx, n, bo, n
    g.kv, g.rope_halves = [(1, 64)], [32]
    plan = D.decode_plan(backend, g, 64)
    assert plan is not None, backend.last_declined
    hid, _ = plan.step(0, x, np.zeros(64, np.float32))
    out = torch.zeros(1, n, device="cuda")
    O.ref_norm(ref, cuda(x[None]), out, cuda(w) if weighted else None, 1e-5)
    assert row_err(hid[None], out.cpu().numpy().astype(np.float64)) < 1e-5
    plan.close()


SHAPES = [(8, 2, 128), (4, 2, 64), (4, 4, 128), (8, 1, 64)]


def rope_plan(backend, nh, nkv, hd, interleaved, qn, kn, max_len, attend):
    """qkv -> QkRope (-> Attend): hidden is the attention output with `attend`, else the rotated queries."""
    g = D.Graph()
    nq = nh * hd
    bq, bo, ba = g.buf(nq + 2 * nkv * hd), g.buf(nq), g.buf(nq)
    g.qk_rope(bq, bo, 0, nh, nkv, hd, hd // 2, nq, nq + nkv * hd, interleaved, 1e-6, q_norm=qn, k_norm=kn)
    if attend:
        g.attend(bo, ba, 0, nh, nkv, hd, hd ** -0.5)
    g.input, g.n_input, g.hidden, g.n_hidden = bq, nq + 2 * nkv * hd, (ba if attend else bo), nq
    g.kv, g.rope_halves = [(nkv, hd)], [hd // 2]
    plan = D.decode_plan(backend, g, max_len)
    assert plan is not None, backend.last_declined
    return plan


@pytest.mark.parametrize("shape", SHAPES)
@pytest.mark.parametrize("interleaved", [True, False])
@pytest.mark.parametrize("head_norms", [False, True])
def test_qk_rope_matches_reference_dqk_rope(backend, ref, shape, interleaved, head_norms):
    nh, nkv, hd = shape
    max_len, pos = 128, 77
    rng = np.random.default_rng(nh * 1000 + hd)
    qkv = rng.standard_normal((nh + 2 * nkv) * hd).astype(np.float32)
    qn = (1 + 0.1 * rng.standard_normal(hd)).astype(np.float32) if head_norms else None
    kn = (1 + 0.1 * rng.standard_normal(hd)).astype(np.float32) if head_norms else None
    cs = O.rope_table(pos, O.rope_inv_freq(hd, 1e6))
    plan = rope_plan(backend, nh, nkv, hd, interleaved, qn, kn, max_len, attend=False)
    q, _ = plan.step(pos, qkv, cs)
    k, v = plan.kv_read(0, pos, 1)

    row = nkv * hd
    kc, vc = torch.zeros(max_len, row, device="cuda"), torch.zeros(max_len, row, device="cuda")
    q_ref, k_ref, v_ref = torch.zeros(nh * hd, device="cuda"), torch.zeros(row, device="cuda"), torch.zeros(row, device="cuda")
    sp = torch.tensor([pos, pos, 1, 0], dtype=torch.int32, device="cuda")
    O.ref_qk_rope(ref, cuda(qkv), q_ref, kc, vc, k_ref, v_ref, cuda(qn) if head_norms else None, cuda(kn) if head_norms else None, cuda(cs), sp,
                  nh, nkv, hd, hd // 2, interleaved, 1e-6)
    assert row_err(q[None], q_ref.cpu().numpy().astype(np.float64)[None]) < 1e-6
    assert row_err(k.reshape(1, -1), kc[pos].cpu().numpy().astype(np.float64)[None]) < 1e-6
    assert np.array_equal(v.reshape(-1), vc[pos].cpu().numpy())
    assert np.array_equal(kc[pos].cpu().numpy(), k_ref.cpu().numpy())
    plan.close()


@pytest.mark.parametrize("shape", SHAPES)
def test_attention_matches_reference_dattn(backend, ref, shape):
    """Contexts of one key, around the 64-key tiles of this kernel, and past 256 keys where the reference splits the keys
    over blocks and combines partials (and this kernel splits too)."""
    nh, nkv, hd = shape
    max_len = 6144
    plan = rope_plan(backend, nh, nkv, hd, True, None, None, max_len, attend=True)
    row = nkv * hd
    rng = np.random.default_rng(hd + nh)
    inv = O.rope_inv_freq(hd, 1e6)
    for pos in (0, 1, 63, 64, 65, 255, 256, 300, 1000, 2049, 6143):
        k = rng.standard_normal((pos + 1, row)).astype(np.float32)
        v = rng.standard_normal((pos + 1, row)).astype(np.float32)
        if pos:
            plan.kv_write(0, 0, k[:pos], v[:pos])
        qkv = rng.standard_normal((nh + 2 * nkv) * hd).astype(np.float32)
        cs = O.rope_table(pos, inv)
        att, _ = plan.step(pos, qkv, cs)

        kc, vc = cuda(np.concatenate([k, np.zeros((1, row), np.float32)])), cuda(np.concatenate([v, np.zeros((1, row), np.float32)]))
        q_ref, k_ref, v_ref = torch.zeros(nh * hd, device="cuda"), torch.zeros(row, device="cuda"), torch.zeros(row, device="cuda")
        sp = torch.tensor([pos, pos, 1, 0], dtype=torch.int32, device="cuda")
        O.ref_qk_rope(ref, cuda(qkv), q_ref, kc, vc, k_ref, v_ref, None, None, cuda(cs), sp, nh, nkv, hd, hd // 2, True, 1e-6)
        out = torch.zeros(nh * hd, device="cuda")
        O.ref_attend(ref, q_ref, kc, vc, out, sp, nh, nkv, hd, hd ** -0.5)
        r = out.cpu().numpy().astype(np.float64)
        assert np.isfinite(att).all()
        assert row_err(att[None], r[None]) < 1e-5, pos
    plan.close()


@pytest.mark.parametrize("gelu", [False, True])
def test_glu_matches_reference_dglu(backend, ref, gelu):
    n = 14336
    rng = np.random.default_rng(3)
    gu = (rng.standard_normal(2 * n) * 2).astype(np.float32)
    g = D.Graph()
    bi, bo = g.buf(2 * n), g.buf(n)
    g.glu(bi, bi.at(n), bo, n, gelu=gelu)
    g.input, g.n_input, g.hidden, g.n_hidden = bi, 2 * n, bo, n
    g.kv, g.rope_halves = [(1, 64)], [32]
    plan = D.decode_plan(backend, g, 64)
    assert plan is not None, backend.last_declined
    hid, _ = plan.step(0, gu, np.zeros(64, np.float32))
    d = cuda(gu)
    out = torch.zeros(n, device="cuda")
    O.ref_glu(ref, d[:n], d[n:], out, gelu)
    assert row_err(hid[None], out.cpu().numpy().astype(np.float64)[None]) < 1e-6
    plan.close()


@pytest.mark.parametrize("shape", [(128, 1024, 2048), (512, 4096, 1024)])
def test_mlx4_prefill_product_against_reference_gemm(backend, ref, shape):
    """The tensor-core product rounds activations and dequantized weights to bf16 (bound 1e-3 of the row maximum against
    the f64 definition); the reference's kernel multiplies in f32 (1e-5). The two must sit within 1e-3 of each other."""
    t, n_out, n_in = shape
    w = synth.mlx4(n_out, n_in, 11)
    m = oracle_matrix(w, n_out, n_in)
    dev = backend.upload(w, n_out, n_in)
    x = synth.activations(t, n_in, 12)
    xd = cuda(x)
    y_ref = torch.zeros(t, n_out, device="cuda")
    O.ref_gemm_q4a(ref, m, xd, y_ref)
    y = torch.zeros(t, n_out, device="cuda")
    assert backend.matmul_dev(dev, xd, y)
    torch.cuda.synchronize()
    exact = m.matmul_f64(x)
    assert row_err(y_ref.cpu().numpy(), exact) < 1e-5
    assert row_err(y.cpu().numpy(), exact) < 1e-3
    assert row_err(y.cpu().numpy(), y_ref.cpu().numpy().astype(np.float64)) < 1e-3
