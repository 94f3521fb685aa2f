"""Routed experts (MoE) on the GPU against the pinned CPU oracle, through the C ABI.

The reference defines the layer as y[i] += sum_j w_ij down_e(silu(gate_e x_i) * up_e x_i) with the axpy in
route order (src/moe.rs:625-828) and tests its CUDA path against the f64 definition at 1e-4 with f32
kernels (src/cuda.rs:2178-2186). Here the two projections run on f16 tensor-core operands. With 128-row token
tiles the activations of both projections enter as two f16 terms (22 bits), so what is left is the rounding of
the expanded weights to f16; every row is scaled by a power of two before its conversion, so the bound holds at
any input magnitude. Bound for the layer: 1e-3 max relative error per output row, for MLX-4 and for the synthetic
Q4_K blocks (random 6-bit scales and mins, heavy cancellation: the worst case).
"""
import numpy as np
import pytest
import torch

import oxinfer_b200 as ob
from oracle import oracle as O
from oxinfer_b200 import synth

from util import oracle_matrix, row_err

pytestmark = pytest.mark.gpu
TOL = 1e-3


def make_experts(backend, fmt, n_experts, h, inter, seed):
    refs_gu = [synth.make(fmt, 2 * inter, h, seed + 2 * e) for e in range(n_experts)]
    refs_dn = [synth.make(fmt, h, inter, seed + 2 * e + 1) for e in range(n_experts)]
    gu = [backend.upload(r, 2 * inter, h) for r in refs_gu]
    dn = [backend.upload(r, h, inter) for r in refs_dn]
    moe = backend.upload_moe(gu, dn, h, inter)
    assert moe is not None
    for d in gu + dn:  # the stacked copies are independent of the per-expert uploads
        d.free()
    return moe, [oracle_matrix(r, 2 * inter, h) for r in refs_gu], [oracle_matrix(r, h, inter) for r in refs_dn]


def routes(t, n_experts, k, seed):
    """Router logits N(0,1) plus a per-expert bias N(0,1) (a skewed load), top-k by the oracle's route_top_k."""
    rng = np.random.default_rng(seed)
    logits = (rng.standard_normal((t, n_experts)) + rng.standard_normal(n_experts)).astype(np.float32)
    ids, w = np.zeros((t, k), np.int32), np.zeros((t, k), np.float32)
    for i in range(t):
        ids[i], w[i] = O.route_top_k(logits[i], k)
    return logits, ids, w


@pytest.mark.parametrize("fmt", ["mlx4", "q4_k"])
@pytest.mark.parametrize("t", [1, 5, 64, 300])
def test_moe_matches_oracle(backend, fmt, t):
    n_experts, k, h, inter = 16, 4, 512, 256
    moe, gu, dn = make_experts(backend, fmt, n_experts, h, inter, 700)
    _, ids, w = routes(t, n_experts, k, 701 + t)
    x = synth.activations(t, h, 702)
    y0 = np.random.default_rng(703).standard_normal((t, h)).astype(np.float32)  # moe ADDS into y
    y = y0.copy()
    assert backend.moe(x, ids, w, moe, y)
    want = O.moe_forward(gu, dn, h, inter, x, ids, w, y=y0, exact=True)
    assert row_err(y - y0, want.astype(np.float64) - y0) < TOL
    assert row_err(y, want) < TOL


def test_moe_config_shape_one_token_and_batch(backend):
    """The benchmark's expert shape (h 2048, inter 768, top-8) with 32 of its 128 experts."""
    n_experts, k, h, inter = 32, 8, 2048, 768
    moe, gu, dn = make_experts(backend, "mlx4", n_experts, h, inter, 710)
    for t in (1, 64):
        _, ids, w = routes(t, n_experts, k, 711 + t)
        x = synth.activations(t, h, 712)
        y = np.zeros((t, h), np.float32)
        assert backend.moe(x, ids, w, moe, y)
        want = O.moe_forward(gu, dn, h, inter, x, ids, w, exact=True)
        assert row_err(y, want) < TOL
    # every token to the same experts (one long segment, several token tiles of one expert)
    t = 200
    ids = np.tile(np.arange(k, dtype=np.int32), (t, 1))
    w = np.full((t, k), 1.0 / k, np.float32)
    x = synth.activations(t, h, 713)
    y = np.zeros((t, h), np.float32)
    assert backend.moe(x, ids, w, moe, y)
    assert row_err(y, O.moe_forward(gu, dn, h, inter, x, ids, w, exact=True)) < TOL


@pytest.mark.parametrize("fmt", ["mlx4", "q4_k"])
def test_moe_rows_of_very_different_magnitude(backend, fmt):
    """Token rows scaled by 1e-3, 1, 300 and 2e5 (the magnitudes of the reference's own input(), src/cuda.rs:1579-1700): the
    per-row power-of-two factors keep every row inside f16's range and out of its subnormals, in both projections."""
    n_experts, k, h, inter, t = 8, 2, 512, 256, 70
    moe, gu, dn = make_experts(backend, fmt, n_experts, h, inter, 740)
    _, ids, w = routes(t, n_experts, k, 741)
    x = synth.activations(t, h, 742) * np.array([1e-3, 1.0, 300.0, 2e5], np.float32)[np.arange(t) % 4, None]
    y = np.zeros((t, h), np.float32)
    assert backend.moe(x, ids, w, moe, y)
    assert np.isfinite(y).all()
    assert row_err(y, O.moe_forward(gu, dn, h, inter, x, ids, w, exact=True)) < TOL


def _layer_f64(gate, up, down, x, ids, w, act, limit):
    """y[i] = sum_j w_ij down_e(act(gate_e x_i) * up_e x_i) in f64 over the bit-exact dequantized weights (MoeAct, src/gpu.rs:36-54)."""
    t, k = ids.shape
    y = np.zeros((t, down[0].n_out), np.float64)
    for i in range(t):
        for j in range(k):
            e = int(ids[i, j])
            g, u = gate[e].matmul_f64(x[i : i + 1])[0], up[e].matmul_f64(x[i : i + 1])[0]
            if act == 1:
                a = g / (1.0 + np.exp(-1.5957692 * (g + 0.044715 * g**3))) * u
            else:
                if act == 2:
                    g, u = np.minimum(g, limit), np.clip(u, -limit, limit)
                a = g / (1.0 + np.exp(-g)) * u
            y[i] += float(w[i, j]) * (down[e].dequantize_rows().astype(np.float64) @ a)
    return y


@pytest.mark.parametrize("act,limit", [(0, 0.0), (1, 0.0), (2, 7.0)])
@pytest.mark.parametrize("t", [3, 90])
def test_separate_up_matrices_and_the_other_activations(backend, act, limit, t):
    """upload_moe with the gate and up projections apart (GGUF checkpoints store them so, src/gpu.rs:200-215) and the gated
    activations the reference's CUDA backend runs besides SiLU: tanh GELU and the clamped SiLU (src/cuda.rs:300-316, 896-906)."""
    n_experts, k, h, inter = 6, 2, 512, 256
    refs = [(synth.mlx4(inter, h, 760 + 3 * e), synth.mlx4(inter, h, 761 + 3 * e), synth.mlx4(h, inter, 762 + 3 * e)) for e in range(n_experts)]
    devs = [[backend.upload(r[i], *(s)) for r in refs] for i, s in enumerate([(inter, h), (inter, h), (h, inter)])]
    moe = backend.upload_moe(devs[0], devs[2], h, inter, up=devs[1], act=act, act_limit=limit)
    assert moe is not None, backend.last_declined
    mats = [[oracle_matrix(r[i], *(s)) for r in refs] for i, s in enumerate([(inter, h), (inter, h), (h, inter)])]
    _, ids, w = routes(t, n_experts, k, 763 + t)
    x = synth.activations(t, h, 764) * np.float32(0.25)    # gate values around the clamp, not far beyond it
    y = np.zeros((t, h), np.float32)
    assert backend.moe(x, ids, w, moe, y)
    assert row_err(y, _layer_f64(mats[0], mats[1], mats[2], x, ids, w, act, limit)) < TOL
    # an activation the device does not run is declined, as the reference's backend declines it
    assert backend.upload_moe(devs[0], devs[2], h, inter, up=devs[1], act=3) is None


def test_route_topk_matches_oracle(backend):
    t, n, k = 70, 128, 8
    logits, ids, w = routes(t, n, k, 720)
    logits[3, 5] = logits[3, 9] = logits[3].max() + 1.0  # a tie at the top: the lower index wins
    ids[3], w[3] = O.route_top_k(logits[3], k)
    ld = torch.from_numpy(logits).cuda()
    idd = torch.zeros((t, k), dtype=torch.int32, device="cuda")
    wd = torch.zeros((t, k), dtype=torch.float32, device="cuda")
    assert backend.route_topk_dev(ld, k, idd, wd)
    torch.cuda.synchronize()
    assert np.array_equal(idd.cpu().numpy(), ids)
    assert np.allclose(wd.cpu().numpy(), w, rtol=2e-6, atol=1e-9)


def test_moe_rejects_bad_routes(backend):
    moe, _, _ = make_experts(backend, "q4_k", 4, 256, 256, 730)
    x = np.zeros((2, 256), np.float32)
    y = np.zeros((2, 256), np.float32)
    with pytest.raises(ob.BackendError):
        backend.moe(x, np.array([[0, 9], [1, 2]], np.int32), np.ones((2, 2), np.float32), moe, y)
