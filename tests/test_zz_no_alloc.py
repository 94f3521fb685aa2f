"""The allocation-free Q4_K matrix-vector entry point (b2_matvec_q4k_noalloc).

It exists for hosts that cannot allocate device memory when they need a product (their own arena
owns the GPU, or the decode loop must not enter the allocator): its scratch is a fixed array inside
the library. The test calls it through the C ABI twice in a row, with different inputs, and checks
each result against the regular entry point (b2_matvec_dev) on the same weights, and that sizes
beyond the built-in scratch are refused with a message. This file sorts last on purpose, so that a
run that stops at the first failure has already run every other test.
"""
import ctypes as C

import numpy as np
import pytest
import torch

import oxinfer_b200 as ob
from oracle import oracle as O
from oxinfer_b200 import synth

pytestmark = pytest.mark.gpu
TOL = 2e-5  # the GEMV tests' bound; both entry points run the same kernels, so equality is expected


def _call(w_dev, n_out, n_in, x, y):
    err = C.create_string_buffer(256)
    rc = ob.lib().b2_matvec_q4k_noalloc(w_dev.data_ptr(), n_out, n_in, x.data_ptr(), y.data_ptr(), torch.cuda.current_stream().cuda_stream,
                                        err, len(err))
    return rc, err.value.decode()


def test_noalloc_matches_regular_entry_point_twice_in_a_row(backend):
    n_out, n_in = 1000, 4096
    ref = synth.q4_k(n_out, n_in, 900)
    dev = backend.upload(ref, n_out, n_in)
    w_dev = torch.from_numpy(ref.data).cuda()
    backend.set_stream(torch.cuda.current_stream().cuda_stream)
    try:
        for seed in (901, 902):
            x = torch.from_numpy(synth.activations(1, n_in, seed)[0] * np.float32(1.37)).cuda()
            want = torch.zeros(n_out, device="cuda")
            assert backend.matvec_dev(dev, x, want)
            got = torch.full((n_out,), float("nan"), device="cuda")
            rc, msg = _call(w_dev, n_out, n_in, x, got)
            assert rc == ob.OK, msg
            torch.cuda.synchronize()
            w, g = want.cpu().numpy().astype(np.float64), got.cpu().numpy().astype(np.float64)
            assert np.isfinite(g).all()
            assert np.abs(g - w).max() <= TOL * np.abs(w).max()
        # a different, smaller shape right after: stale planes of the longer vector must not leak in
        n2_out, n2_in = 96, 512
        ref2 = synth.q4_k(n2_out, n2_in, 903)
        dev2 = backend.upload(ref2, n2_out, n2_in)
        w2 = torch.from_numpy(ref2.data).cuda()
        x2 = torch.from_numpy(synth.activations(1, n2_in, 904)[0]).cuda()
        want2, got2 = torch.zeros(n2_out, device="cuda"), torch.zeros(n2_out, device="cuda")
        assert backend.matvec_dev(dev2, x2, want2)
        rc, msg = _call(w2, n2_out, n2_in, x2, got2)
        assert rc == ob.OK, msg
        torch.cuda.synchronize()
        assert np.abs(got2.cpu().numpy() - want2.cpu().numpy()).max() <= TOL * np.abs(want2.cpu().numpy()).max()
    finally:
        backend.set_stream(0)


@pytest.mark.parametrize("n_out,n_in", [(1000, 4096), (515, 14336), (259, 16384)])
def test_noalloc_matches_the_cpu_oracle_and_leaves_device_memory_alone(n_out, n_in):
    """Against the f64 product over the bit-exact dequantized weights (not against this library's other entry point),
    with a ragged row count, up to the largest n_in the built-in scratch takes; from 14080 inputs on the kernel needs
    more than the default 48 KB of shared memory. Free device memory, as the driver reports it, is the same before
    and after two calls: nothing was allocated on the way (what the callers of this entry point rely on)."""
    ref = synth.q4_k(n_out, n_in, 910 + n_out)
    m = O.Matrix.gguf(O.Q4_K, ref.data, n_out, n_in)
    w_dev = torch.from_numpy(ref.data).cuda()
    xs = [synth.activations(1, n_in, 920 + i) for i in range(2)]
    xd = [torch.from_numpy(x[0]).cuda() for x in xs]
    got = [torch.full((n_out,), float("nan"), device="cuda") for _ in range(2)]
    rc, msg = _call(w_dev, n_out, n_in, xd[0], got[0])   # the first call on a device does the one-time set-up
    assert rc == ob.OK, msg
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    for i in range(2):
        rc, msg = _call(w_dev, n_out, n_in, xd[i], got[i])
        assert rc == ob.OK, msg
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before
    for i in range(2):
        want = m.matmul_f64(xs[i])
        assert O.row_err(got[i].cpu().numpy()[None], want) < TOL


def test_noalloc_refuses_sizes_beyond_its_scratch():
    n_out, n_in = 4, 16384 + 256
    w = torch.zeros(n_out * (n_in // 256) * 144, dtype=torch.uint8, device="cuda")
    x = torch.zeros(n_in, device="cuda")
    y = torch.full((n_out,), 7.0, device="cuda")
    rc, msg = _call(w, n_out, n_in, x, y)
    assert rc == -2 and "exceeds the built-in scratch" in msg
    rc, msg = _call(w, n_out, 300, x, y)
    assert rc == -2 and "multiple of 256" in msg
    torch.cuda.synchronize()
    assert (y == 7.0).all()  # refused: nothing was launched
