"""The reference's OWN CUDA kernel (dmv_q4a of src/cuda_decode.cu, compiled into oracle/_ref by oracle/build_ref.py where
the reference's tree is present) as a second oracle for the MLX-4 matrix-vector product: both kernels multiply the same
repacked matrix by the same vector on the GPU. The reference kernel rounds per 32-block in f32 (its result sits within
1e-5 of the f64 definition, src/cuda.rs:2285-2307), so the two agree to about 1e-5 of the row maximum."""
import numpy as np
import pytest
import torch

import oxinfer_b200 as ob
from oracle import oracle as O
from oxinfer_b200 import synth

from util import oracle_matrix, row_err

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("shape", [(4096, 4096), (1000, 2048), (37, 512)])
def test_mlx4_matvec_agrees_with_the_reference_cuda_kernel(backend, shape):
    L = O.ref_cuda()
    if L is None:
        pytest.skip("oracle/_ref/libref_cuda.so was not built (the reference's tree is not on this machine)")
    n_out, n_in = shape
    ref = synth.mlx4(n_out, n_in, 42)
    m = oracle_matrix(ref, n_out, n_in)
    dev = backend.upload(ref, n_out, n_in)
    x = synth.activations(1, n_in, 43)
    xd = torch.from_numpy(x[0]).cuda()
    y_ref = torch.zeros(n_out, device="cuda")
    O.ref_dmv_q4a(L, m, xd, y_ref)
    y = torch.zeros(n_out, device="cuda")
    assert backend.matvec_dev(dev, xd, y)
    torch.cuda.synchronize()
    exact = m.matmul_f64(x)
    assert row_err(y_ref.cpu().numpy()[None], exact) < 1e-5      # the reference kernel against the definition
    assert row_err(y.cpu().numpy()[None], exact) < 2e-5          # this repository's kernel against the definition
    assert row_err(y.cpu().numpy()[None], y_ref.cpu().numpy().astype(np.float64)[None]) < 2e-5
