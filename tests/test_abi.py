"""The C-ABI library loads without a GPU and exports every symbol the public header declares."""
import ctypes as C

import oxinfer_b200 as ob


def test_library_exports_every_declared_symbol():
    ob.build()
    L = ob.lib()
    names = ob.exported_names()
    assert len(names) >= 20
    for n in names:
        assert hasattr(L, n), f"{n} is declared in include/b200qmm.h but not exported"


def test_no_load_time_cuda_dependency():
    """The host program links nothing: the library must not need libcuda / libcudart to load."""
    import subprocess

    out = subprocess.run(["ldd", str(ob.LIB_PATH)], capture_output=True, text=True).stdout
    assert "libcuda" not in out and "libcudart" not in out and "libtorch" not in out


def test_open_reports_instead_of_crashing_without_a_device():
    import torch

    if torch.cuda.is_available():
        return  # covered by the GPU tests
    ctx = C.c_void_p()
    rc = ob.lib().b2_open(0, C.byref(ctx))
    assert rc == ob.DECLINED and not ctx.value
    assert b"no CUDA device" in ob.lib().b2_open_error()
    try:
        ob.Backend(0)
    except ob.BackendError as e:
        assert e.code == ob.DECLINED
    else:
        raise AssertionError("Backend() must fail loudly without a GPU: there is no CPU fallback")


def test_null_context_is_an_error_not_a_crash():
    L = ob.lib()
    assert L.b2_wants(None, 64, 64, 1) == 0
    assert L.b2_free_weight(None, 1) == -2
    assert L.b2_launch_count(None) == 0
