"""The routed-expert layer at the benchmark's full size: 128 experts, top-8 routing, hidden 2048, expert
intermediate 768, MLX affine 4-bit weights (group 64), at token batches of 512 and 4096 with a skewed load
(router logits N(0,1) plus a per-expert bias N(0,1)).

At these sizes the grouped tensor-core GEMM runs with its large-batch launch shapes (256-row token tiles, the
tile width chosen by the wave model), which the small cases of test_moe_gpu.py never reach. The oracle
(f64 products over the bit-exact dequantized weights, the reference's own CUDA test bar at
src/cuda.rs:2178-2186) is evaluated on a sample of token rows, since a token's result depends only on its own
row and routes. Bound: 1e-3 max relative error per output row.
"""
import numpy as np
import pytest

from oracle import oracle as O
from oxinfer_b200 import synth

from util import oracle_matrix, row_err

pytestmark = pytest.mark.gpu
TOL = 1e-3
E, K, H, I = 128, 8, 2048, 768


@pytest.fixture(scope="module")
def experts(backend):
    refs_gu = [synth.mlx4(2 * I, H, 3000 + 2 * e) for e in range(E)]
    refs_dn = [synth.mlx4(H, I, 3001 + 2 * e) for e in range(E)]
    gu = [backend.upload(r, 2 * I, H) for r in refs_gu]
    dn = [backend.upload(r, H, I) for r in refs_dn]
    moe = backend.upload_moe(gu, dn, H, I)
    assert moe is not None, backend.last_declined
    for d in gu + dn:
        d.free()
    yield moe, [oracle_matrix(r, 2 * I, H) for r in refs_gu], [oracle_matrix(r, H, I) for r in refs_dn]
    moe.free()


def skewed_routes(t, seed):
    rng = np.random.default_rng(seed)
    logits = (rng.standard_normal((t, E)) + rng.standard_normal(E)).astype(np.float32)
    ids, w = np.zeros((t, K), np.int32), np.zeros((t, K), np.float32)
    for i in range(t):
        ids[i], w[i] = O.route_top_k(logits[i], K)
    return ids, w


@pytest.mark.parametrize("t,sample", [(512, 32), (4096, 16)])
def test_moe_full_size_matches_oracle_on_sampled_rows(backend, experts, t, sample):
    moe, gu, dn = experts
    ids, w = skewed_routes(t, 3100 + t)
    x = synth.activations(t, H, 3200 + t)
    y0 = np.random.default_rng(3300 + t).standard_normal((t, H)).astype(np.float32)  # the layer ADDS into y
    y = y0.copy()
    assert backend.moe(x, ids, w, moe, y)
    rows = np.sort(np.random.default_rng(3400 + t).choice(t, size=sample, replace=False))
    rows[0], rows[-1] = 0, t - 1  # the first and the last token of the batch are always in the sample
    want = O.moe_forward(gu, dn, H, I, x[rows], ids[rows], w[rows], y=y0[rows], exact=True)
    err_layer = row_err(y[rows] - y0[rows], want.astype(np.float64) - y0[rows])
    print(f"moe config 3, t = {t}: row error of the layer's contribution {err_layer:.3e} over {sample} sampled rows")
    assert err_layer < TOL
    assert row_err(y[rows], want) < TOL
    # rows that were not sampled were written too (no token dropped by the segment building)
    assert np.all(np.any(y != y0, axis=1))
