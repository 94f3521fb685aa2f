"""ctypes binding of ``libb200qmm.so``, the C-ABI engine declared in ``include/b200qmm.h``.

There is no CPU fallback anywhere in this package: if the library is missing, or no sm_100 GPU is
present, the calls raise. Building is explicit (``oxinfer_b200.build()`` or ``make`` in ``csrc``).
"""
from __future__ import annotations

import ctypes as C
import subprocess
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
LIB_PATH = PKG_DIR / "libb200qmm.so"
CSRC = PKG_DIR / "csrc"
HEADER = PKG_DIR.parent / "include" / "b200qmm.h"

OK, DECLINED, ERR_CUDA, ERR_ARG, ERR_NOMEM, ERR_TIMEOUT = 0, 1, -1, -2, -3, -4
FMT_MLX4, FMT_Q8_0, FMT_Q4_K, FMT_Q6_K, FMT_F8E4M3 = 1, 8, 12, 14, 4096
# the other GGUF block formats (raw rows on the device, one generic matrix-vector kernel)
FMT_Q4_0, FMT_Q4_1, FMT_Q5_0, FMT_Q5_1, FMT_Q2_K, FMT_Q3_K, FMT_Q5_K, FMT_IQ4_NL, FMT_IQ4_XS, FMT_MXFP4 = 2, 3, 6, 7, 10, 11, 13, 20, 23, 39
OTHER_FORMATS = (FMT_Q4_0, FMT_Q4_1, FMT_Q5_0, FMT_Q5_1, FMT_Q2_K, FMT_Q3_K, FMT_Q5_K, FMT_IQ4_NL, FMT_IQ4_XS, FMT_MXFP4)
F32, BF16, F16 = 0, 1, 2
MODE_STORE, MODE_ADD, MODE_SILU_PAIR, MODE_GELU_PAIR, MODE_ADD_GATED = 0, 1, 2, 3, 4


class Job(C.Structure):
    _fields_ = [("w", C.c_uint64), ("n_out", C.c_size_t), ("y", C.c_void_p)]


class RowsJob(C.Structure):
    _fields_ = [("w", C.c_uint64), ("up", C.c_uint64), ("n_out", C.c_size_t), ("y", C.c_void_p)]


class View(C.Structure):
    _fields_ = [("buf", C.c_uint32), ("off", C.c_uint32)]


OP_NORM, OP_LINEAR, OP_QK_ROPE, OP_ATTEND, OP_GLU, OP_EXCHANGE = 1, 2, 3, 4, 5, 6
PLAN_HANDLE_BYTES = 128
COMM_ID_BYTES = 128


class Op(C.Structure):
    """``b2_op`` of ``include/b200qmm.h`` (field order is the ABI)."""

    _fields_ = [
        ("kind", C.c_uint32),
        ("x", View), ("y", View), ("z", View),
        ("w", C.c_uint64), ("w2", C.c_uint64),
        ("mode", C.c_uint32), ("n_out", C.c_uint32), ("n_in", C.c_uint32),
        ("p0", C.c_void_p), ("p1", C.c_void_p),
        ("n", C.c_uint32), ("rows", C.c_uint32), ("x_stride", C.c_uint32), ("out_stride", C.c_uint32), ("add", C.c_uint32),
        ("pre", C.c_float), ("eps", C.c_float),
        ("kv", C.c_uint32), ("nh", C.c_uint32), ("nkv", C.c_uint32), ("hd", C.c_uint32),
        ("half_rot", C.c_uint32), ("q_stride", C.c_uint32), ("k_off", C.c_uint32), ("v_off", C.c_uint32),
        ("interleaved", C.c_uint32), ("rope", C.c_uint32), ("v_norm", C.c_uint32), ("v_from_k", C.c_uint32),
        ("scale", C.c_float), ("window", C.c_uint32), ("gelu", C.c_uint32),
    ]


class GraphDesc(C.Structure):
    """``b2_graph``."""

    _fields_ = [
        ("bufs", C.POINTER(C.c_uint64)), ("n_bufs", C.c_uint32),
        ("ops", C.POINTER(Op)), ("n_ops", C.c_uint32),
        ("input", View), ("n_input", C.c_uint32),
        ("hidden", View), ("n_hidden", C.c_uint32),
        ("logits", View), ("n_logits", C.c_uint32),
        ("kv_nkv", C.POINTER(C.c_uint32)), ("kv_hd", C.POINTER(C.c_uint32)), ("n_kv", C.c_uint32),
        ("rope_halves", C.POINTER(C.c_uint32)), ("n_rope", C.c_uint32),
        ("max_len", C.c_uint32), ("kv_f16", C.c_uint32),
    ]


def build(verbose: bool = False) -> Path:
    """Compiles every CUDA source for sm_100a into ``libb200qmm.so`` (nvcc cross-compiles without a GPU)."""
    r = subprocess.run(["make", "-C", str(CSRC), "-j8"], capture_output=True, text=True)
    if verbose or r.returncode != 0:
        print(r.stdout[-4000:], r.stderr[-4000:])
    if r.returncode != 0:
        raise RuntimeError("building libb200qmm.so failed")
    return LIB_PATH


_SIGNATURES = {
    # name: (restype, argtypes)
    "b2_open": (C.c_int, [C.c_int, C.POINTER(C.c_void_p)]),
    "b2_close": (None, [C.c_void_p]),
    "b2_last_error": (C.c_char_p, [C.c_void_p]),
    "b2_open_error": (C.c_char_p, []),
    "b2_set_stream": (C.c_int, [C.c_void_p, C.c_void_p]),
    "b2_set_exact": (C.c_int, [C.c_void_p, C.c_int]),
    "b2_set_fast_planes": (C.c_int, [C.c_void_p, C.c_int]),
    "b2_set_fp8_activations": (C.c_int, [C.c_void_p, C.c_int]),
    "b2_set_chained": (C.c_int, [C.c_void_p, C.c_int]),
    "b2_stats": (C.c_char_p, [C.c_void_p]),
    "b2_launch_count": (C.c_uint64, [C.c_void_p]),
    "b2_wants": (C.c_int, [C.c_void_p, C.c_size_t, C.c_size_t, C.c_size_t]),
    "b2_upload_mlx4": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t, C.c_size_t, C.c_size_t, C.POINTER(C.c_uint64)]),
    "b2_upload_q4": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t, C.c_size_t, C.c_size_t, C.POINTER(C.c_uint64)]),
    "b2_upload_gguf": (C.c_int, [C.c_void_p, C.c_int, C.c_void_p, C.c_size_t, C.c_size_t, C.c_void_p, C.c_size_t, C.c_size_t, C.POINTER(C.c_uint64)]),
    "b2_shard_rows": (C.c_int, [C.c_void_p, C.c_uint64, C.c_size_t, C.c_size_t, C.POINTER(C.c_uint64)]),
    "b2_free_weight": (C.c_int, [C.c_void_p, C.c_uint64]),
    "b2_weight_bytes": (C.c_size_t, [C.c_void_p, C.c_uint64]),
    "b2_dequantize_rows": (C.c_int, [C.c_void_p, C.c_uint64, C.c_size_t, C.c_size_t, C.c_void_p]),
    "b2_dequantize_rows_dev": (C.c_int, [C.c_void_p, C.c_uint64, C.c_size_t, C.c_size_t, C.c_void_p]),
    "b2_matmul": (C.c_int, [C.c_void_p, C.c_void_p, C.c_size_t, C.c_size_t, C.POINTER(Job), C.c_size_t]),
    "b2_matvec_rows": (C.c_int, [C.c_void_p, C.c_void_p, C.c_size_t, C.c_size_t, C.POINTER(RowsJob), C.c_size_t]),
    "b2_matmul_dev": (C.c_int, [C.c_void_p, C.c_uint64, C.c_void_p, C.c_int, C.c_size_t, C.c_void_p, C.c_int]),
    "b2_matvec_dev": (C.c_int, [C.c_void_p, C.c_uint64, C.c_uint64, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p]),
    "b2_check_status": (C.c_int, [C.c_void_p]),
    "b2_upload_moe": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t, C.c_size_t, C.c_size_t, C.POINTER(C.c_uint64)]),
    "b2_upload_moe_ex": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t, C.c_size_t, C.c_size_t, C.c_int, C.c_float,
                         C.POINTER(C.c_uint64)]),
    "b2_free_moe": (C.c_int, [C.c_void_p, C.c_uint64]),
    "b2_moe": (C.c_int, [C.c_void_p, C.c_uint64, C.c_void_p, C.c_size_t, C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p]),
    "b2_moe_dev": (C.c_int, [C.c_void_p, C.c_uint64, C.c_void_p, C.c_size_t, C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p]),
    "b2_route_topk_dev": (C.c_int, [C.c_void_p, C.c_void_p, C.c_size_t, C.c_size_t, C.c_size_t, C.c_void_p, C.c_void_p]),
    "b2_prepare_x_dev": (C.c_int, [C.c_void_p, C.c_void_p, C.c_size_t]),
    "b2_matvec_prepared_dev": (C.c_int, [C.c_void_p, C.c_uint64, C.c_uint64, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p]),
    "b2_decode_plan": (C.c_int, [C.c_void_p, C.POINTER(GraphDesc), C.POINTER(C.c_uint64)]),
    "b2_decode_plan_multi": (C.c_int, [C.c_void_p, C.POINTER(GraphDesc), C.c_size_t, C.POINTER(C.c_uint64)]),
    "b2_plan_tokens": (C.c_int, [C.c_void_p, C.c_uint64, C.POINTER(C.c_size_t)]),
    "b2_decode_plan_prefill": (C.c_int, [C.c_void_p, C.POINTER(GraphDesc), C.c_size_t, C.POINTER(C.c_uint64)]),
    "b2_plan_last_step_ms": (C.c_int, [C.c_void_p, C.c_uint64, C.POINTER(C.c_float)]),
    "b2_plan_step_multi": (C.c_int, [C.c_void_p, C.c_uint64, C.c_size_t, C.c_size_t, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
    "b2_plan_free": (C.c_int, [C.c_void_p, C.c_uint64]),
    "b2_plan_step": (C.c_int, [C.c_void_p, C.c_uint64, C.c_size_t, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
    "b2_plan_kv_write": (C.c_int, [C.c_void_p, C.c_uint64, C.c_uint32, C.c_size_t, C.c_size_t, C.c_void_p, C.c_void_p]),
    "b2_plan_kv_read": (C.c_int, [C.c_void_p, C.c_uint64, C.c_uint32, C.c_size_t, C.c_size_t, C.c_void_p, C.c_void_p]),
    "b2_plan_generate": (C.c_int, [C.c_void_p, C.c_uint64, C.c_uint64, C.c_int32, C.c_size_t, C.c_size_t, C.c_void_p, C.c_void_p,
                                   C.POINTER(C.c_float)]),
    "b2_plan_launches": (C.c_int, [C.c_void_p, C.c_uint64, C.POINTER(C.c_uint64)]),
    "b2_plan_export": (C.c_int, [C.c_void_p, C.c_uint64, C.c_void_p]),
    "b2_plan_attach_peers": (C.c_int, [C.c_void_p, C.c_uint64, C.c_uint32, C.c_uint32, C.c_void_p]),
    "b2_comm_unique_id": (C.c_int, [C.c_void_p]),
    "b2_comm_init": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_void_p]),
    "b2_comm_free": (C.c_int, [C.c_void_p]),
    "b2_matmul_sharded": (C.c_int, [C.c_void_p, C.c_uint64, C.c_void_p, C.c_int, C.c_size_t, C.c_void_p]),
    "b2_matmul_sharded_peer": (C.c_int, [C.c_void_p, C.c_uint64, C.c_void_p, C.c_int, C.c_size_t, C.POINTER(C.c_void_p)]),
    "b2_moe_ep": (C.c_int, [C.c_void_p, C.c_uint64, C.c_size_t, C.c_void_p, C.c_size_t, C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p]),
    "b2_matvec_q4k_noalloc": (C.c_int, [C.c_void_p, C.c_size_t, C.c_size_t, C.c_void_p, C.c_void_p, C.c_void_p, C.c_char_p, C.c_size_t]),
}

_lib = None


def exported_names() -> list[str]:
    """Every function ``include/b200qmm.h`` declares (parsed from the header text)."""
    import re

    text = HEADER.read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(b2_[a-z0-9_]+)\s*\(", text)))


def lib() -> C.CDLL:
    """Loads the engine. Raises if it has not been built: nothing in this package computes without it."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise RuntimeError(f"{LIB_PATH} is missing: run oxinfer_b200.build() (or make -C {CSRC}); there is no CPU fallback")
        L = C.CDLL(str(LIB_PATH))
        for name, (res, args) in _SIGNATURES.items():
            fn = getattr(L, name)
            fn.restype, fn.argtypes = res, args
        _lib = L
    return _lib
