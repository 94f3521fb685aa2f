"""The boundary is process-wide and `Sync` in the reference (src/gpu.rs:151, src/cuda.rs:430-442): every entry point binds
the device on the calling thread and calls on one context serialize. The reference's own tests for that
(works_from_another_thread, concurrent_calls_do_not_mix: src/cuda.rs:2048-2075, 2411-2440) restated against the C ABI:
ctypes releases the interpreter lock during a call, so the threads below really are inside the library at once."""
import threading

import numpy as np
import pytest

import oxinfer_b200 as ob
from oxinfer_b200 import synth

from util import make_pair, row_err

pytestmark = pytest.mark.gpu


def test_works_from_another_thread(backend):
    n_out, n_in, t = 256, 512, 64
    ref, m = make_pair("q4_k", n_out, n_in, 970)
    x = synth.activations(t, n_in, 971)
    want = m.matmul_f64(x)
    out = {}

    def there():
        dev = backend.upload(ref, n_out, n_in)           # uploaded on the other thread
        y = np.zeros((t, n_out), np.float32)
        out["ok"] = backend.matmul(x, [ob.Job(dev, y)])
        out["y"], out["dev"] = y, dev

    th = threading.Thread(target=there)
    th.start()
    th.join()
    assert out["ok"] and row_err(out["y"], want) < 1e-3
    y2 = np.zeros((t, n_out), np.float32)                # weights uploaded there, used here
    assert backend.matmul(x, [ob.Job(out["dev"], y2)])
    assert np.array_equal(y2, out["y"])


def test_concurrent_calls_do_not_mix(backend):
    n_out, n_in = 320, 1024
    ref, m = make_pair("q4_k", n_out, n_in, 980)
    dev = backend.upload(ref, n_out, n_in)
    inputs = [synth.activations(t, n_in, 981 + i) for i, t in enumerate((1, 3, 12, 64, 130, 4, 40, 200))]   # GEMV, multi-row and GEMM paths
    wants = [m.matmul_f64(x) for x in inputs]
    errors = []

    def worker(x, want):
        try:
            first = None
            for _ in range(8):
                y = np.full((x.shape[0], n_out), np.nan, np.float32)
                if x.shape[0] <= 4:
                    assert backend.matvec_rows(x, [ob.RowsJob(dev, y)])
                else:
                    assert backend.matmul(x, [ob.Job(dev, y)])
                assert row_err(y, want) < 1e-3
                if first is None:
                    first = y.copy()
                assert np.array_equal(y, first)       # the same call gives the same bits whatever ran in between
        except Exception as e:   # noqa: BLE001 - reported by the main thread
            errors.append(repr(e))

    threads = [threading.Thread(target=worker, args=(x, w)) for x, w in zip(inputs, wants)]
    for th in threads:
        th.start()
    for th in threads:
        th.join()
    assert not errors, errors
