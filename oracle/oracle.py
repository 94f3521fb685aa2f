"""ctypes binding of the CPU oracle (``liboracle.so``): TEST INFRASTRUCTURE, NOT PRODUCT CODE.

Only the test suite, the smoke check and the CPU-baseline / reference legs of the benchmark import
this module. The CUDA engine (``oxinfer_b200``) never does.

The oracle restates oxinfer's CPU arithmetic (see ``oracle.cpp`` for the per-function citations).
Parity is pinned against the reference's own known-answer hashes: ``REF_HASHES`` below is the
table of ``src/ggml.rs:1547-1577`` for the kinds this oracle implements.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from pathlib import Path

import numpy as np

_HERE = Path(__file__).resolve().parent
_LIB_PATH = _HERE / "liboracle.so"

# GGUF type ids (src/ggml.rs:42-93)
F32, F16, Q8_0, Q4_K, Q6_K, BF16, F8E4M3 = 0, 1, 8, 12, 14, 30, 0x1000
Q4_0, Q4_1, Q5_0, Q5_1, Q2_K, Q3_K, Q5_K, IQ4_NL, IQ4_XS, MXFP4 = 2, 3, 6, 7, 10, 11, 13, 20, 23, 39
NVFP4 = 40  # no known-answer hash in the reference (src/ggml.rs:1547-1577 has none): pinned to the closed form in the tests
OTHER_KINDS = (Q4_0, Q4_1, Q5_0, Q5_1, Q2_K, Q3_K, Q5_K, IQ4_NL, IQ4_XS, MXFP4)
KIND_NAMES = {Q4_0: "q4_0", Q4_1: "q4_1", Q5_0: "q5_0", Q5_1: "q5_1", Q2_K: "q2_k", Q3_K: "q3_k", Q5_K: "q5_k", IQ4_NL: "iq4_nl",
              IQ4_XS: "iq4_xs", MXFP4: "mxfp4", NVFP4: "nvfp4", Q8_0: "q8_0", Q4_K: "q4_k", Q6_K: "q6_k"}

# FNV-1a-64 of the f32 bits of dequantize_row(kind, fixture(kind)), from src/ggml.rs:1547-1577.
REF_HASHES = {
    BF16: 0x767E77C423088E31,
    F16: 0xD03C69EE7934955F,
    F32: 0x8C4157552256808B,
    Q4_K: 0xDE4DA39C1D9096B2,
    Q6_K: 0x20A51CC0FEAAE638,
    Q8_0: 0x3199BE3DEDDF5C1A,
    Q4_0: 0xC2AC60F0D9D22BC8,
    Q4_1: 0x8A49B60459C03FA2,
    Q5_0: 0x46640E791FEAF19F,
    Q5_1: 0xB0FD98E61B74D61D,
    Q2_K: 0x44B0A081C4B9C71C,
    Q3_K: 0x0C8FA80FD8589B8A,
    Q5_K: 0x4BE2F59B66CC7042,
    IQ4_NL: 0x9DE348F3E6E39671,
    IQ4_XS: 0xF26FD3824913AF96,
    MXFP4: 0xF64D0292F050737D,
}
FIXTURE_ELEMS = 1024  # src/ggml.rs:1535


def build(force: bool = False) -> Path:
    """Compiles ``liboracle.so`` next to this file if it is missing or older than its source."""
    src = _HERE / "oracle.cpp"
    if force or not _LIB_PATH.exists() or _LIB_PATH.stat().st_mtime < src.stat().st_mtime:
        subprocess.run(["make", "-C", str(_HERE), "-B", "liboracle.so"], check=True, capture_output=True)
    return _LIB_PATH


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        build()
        L = C.CDLL(str(_LIB_PATH))
        sz, vp, i32, u64, f32 = C.c_size_t, C.c_void_p, C.c_int, C.c_uint64, C.c_float
        sig = {
            "orc_lcg": (u64, [C.POINTER(u64)]),
            "orc_block_size": (sz, [i32]),
            "orc_type_size": (sz, [i32]),
            "orc_f16_to_f32": (f32, [C.c_uint16]),
            "orc_f32_to_f16": (C.c_uint16, [f32]),
            "orc_f32_to_bf16": (C.c_uint16, [f32]),
            "orc_e4m3_to_f32": (f32, [C.c_uint8]),
            "orc_f32_to_e4m3": (C.c_uint8, [f32]),
            "orc_fast_exp": (f32, [f32]),
            "orc_fnv_f32": (u64, [vp, sz]),
            "orc_random_blocks": (None, [i32, sz, C.POINTER(u64), vp]),
            "orc_dequantize_row": (None, [i32, vp, vp, sz]),
            "orc_matrix_from_mlx_q4": (vp, [vp, vp, vp, sz, sz, sz]),
            "orc_matrix_gguf": (vp, [i32, vp, sz, sz, vp, sz, sz]),
            "orc_matrix_free": (None, [vp]),
            "orc_matrix_bytes": (sz, [vp]),
            "orc_matrix_q4_parts": (i32, [vp, C.POINTER(vp), C.POINTER(sz), C.POINTER(vp), C.POINTER(sz), C.POINTER(vp), C.POINTER(sz), C.POINTER(sz)]),
            "orc_matrix_dequantize_rows": (None, [vp, sz, sz, vp]),
            "orc_mlx_dequant_row": (None, [vp, vp, vp, sz, vp, sz]),
            "orc_set_decode_scalar": (None, [i32]),
            "orc_matmul_cpu": (None, [vp, vp, sz, vp, i32]),
            "orc_matmul_prefill": (None, [vp, vp, sz, vp, i32]),
            "orc_matmul_f64": (None, [vp, vp, sz, vp, i32]),
            "orc_quantize_act": (None, [vp, sz, sz, vp, vp, vp, vp, vp]),
            "orc_route_top_k": (None, [vp, sz, sz, vp, vp]),
            "orc_moe_forward": (None, [vp, vp, sz, sz, sz, vp, sz, vp, vp, sz, vp, i32, i32]),
            "orc_quantize_act_e4m3": (None, [vp, sz, sz, sz, vp, vp]),
            "orc_encode_q8_0": (None, [vp, sz, vp]),
            "orc_encode_q4_k": (None, [vp, sz, vp]),
            "orc_encode_q6_k": (None, [vp, sz, vp]),
            "orc_rmsnorm_f32w": (None, [vp, vp, sz, f32, vp]),
            "orc_rope_inv_freq": (None, [sz, C.c_double, C.c_double, vp]),
            "orc_rope_table": (None, [sz, vp, sz, vp]),
            "orc_apply_rope": (None, [vp, vp, sz, i32]),
            "orc_softmax_inplace": (None, [vp, sz]),
            "orc_attention": (None, [vp, vp, vp, sz, sz, sz, sz, sz, vp, i32]),
            "orc_llama_step": (None, [vp, vp, vp, vp, vp, sz, sz, vp, vp, vp, vp, i32, i32]),
        }
        for name, (res, args) in sig.items():
            fn = getattr(L, name)
            fn.restype, fn.argtypes = res, args
        _lib = L
    return _lib


def _p(a: np.ndarray) -> int:
    assert a.flags["C_CONTIGUOUS"]
    return a.ctypes.data


def cpu_threads() -> int:
    return len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)


def block_size(kind: int) -> int:
    return lib().orc_block_size(kind)


def type_size(kind: int) -> int:
    return lib().orc_type_size(kind)


def row_bytes(kind: int, n: int) -> int:
    return n // block_size(kind) * type_size(kind)


def random_blocks(kind: int, nb: int, seed: int) -> tuple[np.ndarray, int]:
    """``random_blocks`` of src/ggml.rs:1446: returns (bytes, advanced seed)."""
    out = np.zeros(nb * type_size(kind), dtype=np.uint8)
    s = C.c_uint64(seed)
    lib().orc_random_blocks(kind, nb, C.byref(s), _p(out))
    return out, s.value


def fixture(kind: int) -> np.ndarray:
    """``fixture(kind)`` of src/ggml.rs:1537-1541."""
    return random_blocks(kind, FIXTURE_ELEMS // block_size(kind), 1000 + kind)[0]


def dequantize_row(kind: int, src: np.ndarray, n: int) -> np.ndarray:
    out = np.zeros(n, dtype=np.float32)
    assert src.dtype == np.uint8 and src.size == row_bytes(kind, n)
    lib().orc_dequantize_row(kind, _p(src), _p(out), n)
    return out


def fnv_f32(v: np.ndarray) -> int:
    v = np.ascontiguousarray(v, dtype=np.float32)
    return lib().orc_fnv_f32(_p(v), v.size)


class Matrix:
    """A weight matrix as the reference's CPU path holds it (Q4 + offsets, or raw GGUF rows)."""

    def __init__(self, handle: int, n_out: int, n_in: int, keep=()):
        self.h, self.n_out, self.n_in, self._keep = handle, n_out, n_in, keep

    @classmethod
    def from_mlx_q4(cls, w: np.ndarray, scales: np.ndarray, biases: np.ndarray, n_out: int, n_in: int, group: int = 64) -> "Matrix":
        assert w.dtype == np.uint32 and scales.dtype == np.uint16 and biases.dtype == np.uint16
        assert w.size == n_out * n_in // 8 and scales.size == n_out * n_in // group == biases.size
        return cls(lib().orc_matrix_from_mlx_q4(_p(w), _p(scales), _p(biases), n_out, n_in, group), n_out, n_in)

    @classmethod
    def gguf(cls, kind: int, data: np.ndarray, n_out: int, n_in: int, block_scales: np.ndarray | None = None, bs_rows: int = 128,
             bs_cols: int = 128) -> "Matrix":
        assert data.dtype == np.uint8 and data.size == n_out * row_bytes(kind, n_in)
        bs = None if block_scales is None else np.ascontiguousarray(block_scales, dtype=np.float32)
        return cls(lib().orc_matrix_gguf(kind, _p(data), n_out, n_in, None if bs is None else _p(bs), bs_rows, bs_cols), n_out, n_in)

    def __del__(self):
        if getattr(self, "h", None):
            lib().orc_matrix_free(self.h)
            self.h = None

    def bytes(self) -> int:
        return lib().orc_matrix_bytes(self.h)

    def q4_parts(self):
        """(nibbles u8, f16 scale bits u16, bf16 offset bits u16, group) of a matrix made by ``from_mlx_q4``: the arrays
        the reference's kernels take (copies)."""
        q, s, o = C.c_void_p(), C.c_void_p(), C.c_void_p()
        nq, ns, no, g = C.c_size_t(), C.c_size_t(), C.c_size_t(), C.c_size_t()
        if lib().orc_matrix_q4_parts(self.h, C.byref(q), C.byref(nq), C.byref(s), C.byref(ns), C.byref(o), C.byref(no), C.byref(g)) != 0:
            raise ValueError("not a Q4 matrix")
        qa = np.ctypeslib.as_array(C.cast(q, C.POINTER(C.c_uint8)), (nq.value,)).copy()
        sa = np.ctypeslib.as_array(C.cast(s, C.POINTER(C.c_uint16)), (ns.value,)).copy()
        oa = np.ctypeslib.as_array(C.cast(o, C.POINTER(C.c_uint16)), (no.value,)).copy()
        return qa, sa, oa, g.value

    def dequantize_rows(self, r0: int = 0, r1: int | None = None) -> np.ndarray:
        r1 = self.n_out if r1 is None else r1
        out = np.zeros((r1 - r0, self.n_in), dtype=np.float32)
        lib().orc_matrix_dequantize_rows(self.h, r0, r1, _p(out))
        return out

    def matmul_cpu(self, x: np.ndarray, threads: int | None = None) -> np.ndarray:
        """The CPU path's own result (int8-activation decode kernels up to 7 rows, f32 GEMM above)."""
        x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1, self.n_in)
        y = np.zeros((x.shape[0], self.n_out), dtype=np.float32)
        lib().orc_matmul_cpu(self.h, _p(x), x.shape[0], _p(y), threads or cpu_threads())
        return y

    def matmul_prefill(self, x: np.ndarray, threads: int | None = None) -> np.ndarray:
        """The f32 prefill-GEMM arithmetic (sequential FMA over k) at any number of rows."""
        x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1, self.n_in)
        y = np.zeros((x.shape[0], self.n_out), dtype=np.float32)
        lib().orc_matmul_prefill(self.h, _p(x), x.shape[0], _p(y), threads or cpu_threads())
        return y

    def matmul_f64(self, x: np.ndarray, threads: int | None = None) -> np.ndarray:
        """f64 product of the bit-exact dequantized weights with x (the definition)."""
        x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1, self.n_in)
        y = np.zeros((x.shape[0], self.n_out), dtype=np.float64)
        lib().orc_matmul_f64(self.h, _p(x), x.shape[0], _p(y), threads or cpu_threads())
        return y


def matrix_of(ref, n_out: int, n_in: int) -> Matrix:
    """The oracle's matrix for a synthetic weight reference: an MLX triple (fields ``w scales biases group``) or raw GGUF
    rows (fields ``kind data block_scales bs_rows bs_cols``)."""
    if hasattr(ref, "w"):
        return Matrix.from_mlx_q4(ref.w.reshape(-1), ref.scales.reshape(-1), ref.biases.reshape(-1), n_out, n_in, ref.group)
    return Matrix.gguf(ref.kind, ref.data, n_out, n_in, ref.block_scales, ref.bs_rows, ref.bs_cols)


def set_decode_scalar(on: bool) -> None:
    """``matmul_cpu`` at up to 7 rows: the scalar restatements of the decode kernels instead of the AVX2 ones (same bits)."""
    lib().orc_set_decode_scalar(int(on))


def decode_kernel_name() -> str:
    """Which restatement of the reference's int8-activation decode kernels ``matmul_cpu`` runs at up to 7 rows."""
    return "AVX2 int8-activation decode kernels (maddubs / madd; src/kernels_x86.rs:476-536, src/kernels_ggml_x86.rs:120-431)"


def mlx_dequant_row(w: np.ndarray, scales: np.ndarray, biases: np.ndarray, group: int, n: int) -> np.ndarray:
    out = np.zeros(n, dtype=np.float32)
    lib().orc_mlx_dequant_row(_p(w), _p(scales), _p(biases), group, _p(out), n)
    return out


def quantize_act(x: np.ndarray):
    x = np.ascontiguousarray(x, dtype=np.float32)
    t, n_in = x.shape
    bpr = n_in // 32
    q = np.zeros((t, n_in), np.int8)
    scales, fsums = np.zeros((t, bpr), np.float32), np.zeros((t, bpr), np.float32)
    sums, hsums = np.zeros((t, bpr), np.int32), np.zeros((t, 2 * bpr), np.float32)
    lib().orc_quantize_act(_p(x), t, n_in, _p(q), _p(scales), _p(sums), _p(fsums), _p(hsums))
    return q, scales, sums, fsums, hsums


def route_top_k(logits: np.ndarray, k: int):
    logits = np.ascontiguousarray(logits, dtype=np.float32)
    ids, w = np.zeros(k, np.int32), np.zeros(k, np.float32)
    lib().orc_route_top_k(_p(logits), logits.size, k, _p(ids), _p(w))
    return ids, w


def moe_forward(gate_up: list[Matrix], down: list[Matrix], h: int, inter: int, x: np.ndarray, route_ids: np.ndarray, route_w: np.ndarray,
                y: np.ndarray | None = None, exact: bool = True, threads: int | None = None) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    t, k = route_ids.shape
    ids = np.ascontiguousarray(route_ids, dtype=np.int32)
    w = np.ascontiguousarray(route_w, dtype=np.float32)
    y = np.zeros((t, h), np.float32) if y is None else np.ascontiguousarray(y, dtype=np.float32).copy()
    n = len(gate_up)
    gu = (C.c_void_p * n)(*[m.h for m in gate_up])
    dn = (C.c_void_p * n)(*[m.h for m in down])
    lib().orc_moe_forward(C.cast(gu, C.c_void_p), C.cast(dn, C.c_void_p), n, h, inter, _p(x), t, _p(ids), _p(w), k, _p(y),
                          threads or cpu_threads(), 1 if exact else 0)
    return y


def quantize_act_e4m3(x: np.ndarray, blk: int = 128):
    x = np.ascontiguousarray(x, dtype=np.float32)
    t, n_in = x.shape
    nb = (n_in + blk - 1) // blk
    q, s = np.zeros((t, n_in), np.uint8), np.zeros((t, nb), np.float32)
    lib().orc_quantize_act_e4m3(_p(x), t, n_in, blk, _p(q), _p(s))
    return q, s


def e4m3_table() -> np.ndarray:
    return np.array([lib().orc_e4m3_to_f32(b) for b in range(256)], dtype=np.float32)


def encode(kind: int, w: np.ndarray) -> np.ndarray:
    """Synthetic-data encoders (not from the reference, which has no K-quant encoder)."""
    w = np.ascontiguousarray(w, dtype=np.float32).reshape(-1)
    out = np.zeros(row_bytes(kind, w.size), dtype=np.uint8)
    {Q8_0: lib().orc_encode_q8_0, Q4_K: lib().orc_encode_q4_k, Q6_K: lib().orc_encode_q6_k}[kind](_p(w), w.size, _p(out))
    return out


def row_err(y: np.ndarray, r: np.ndarray) -> float:
    """Worst per-row ``max|y - r| / max|r|`` (src/cuda.rs:1582-1592); rows are the leading axis."""
    y = np.asarray(y, dtype=np.float64).reshape(r.shape)
    r = np.asarray(r, dtype=np.float64)
    num = np.abs(y - r).reshape(r.shape[0], -1).max(axis=1)
    den = np.maximum(np.abs(r).reshape(r.shape[0], -1).max(axis=1), 1e-30)
    return float((num / den).max())


# ---- one decode token (src/kernels.rs rmsnorm / rope / softmax, src/model.rs attention_ext, src/qwen.rs layer order) ----
def rmsnorm_f32w(x: np.ndarray, w: np.ndarray, eps: float) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    w = np.ascontiguousarray(w, dtype=np.float32)
    out = np.empty_like(x)
    lib().orc_rmsnorm_f32w(_p(x), _p(w), x.size, eps, _p(out))
    return out


def rope_inv_freq(dim: int, theta: float, proportion: float = 1.0) -> np.ndarray:
    out = np.empty(dim // 2, dtype=np.float32)
    lib().orc_rope_inv_freq(dim, theta, proportion, _p(out))
    return out


def rope_table(pos: int, inv_freq: np.ndarray) -> np.ndarray:
    """cos[half] then sin[half] of one position."""
    f = np.ascontiguousarray(inv_freq, dtype=np.float32)
    cs = np.empty(2 * f.size, dtype=np.float32)
    lib().orc_rope_table(pos, _p(f), f.size, _p(cs))
    return cs


def apply_rope(v: np.ndarray, cs: np.ndarray, interleaved: bool) -> np.ndarray:
    v = np.array(v, dtype=np.float32)
    cs = np.ascontiguousarray(cs, dtype=np.float32)
    lib().orc_apply_rope(_p(v), _p(cs), cs.size // 2, int(interleaved))
    return v


def softmax(x: np.ndarray) -> np.ndarray:
    x = np.array(x, dtype=np.float32)
    lib().orc_softmax_inplace(_p(x), x.size)
    return x


def attention(q: np.ndarray, kc: np.ndarray, vc: np.ndarray, length: int, nh: int, nkv: int, hd: int, lo: int = 0,
              threads: int | None = None) -> np.ndarray:
    """q [nh][hd] already scaled; kc / vc [>= length][nkv][hd]; keys lo .. length - 1."""
    q = np.ascontiguousarray(q, dtype=np.float32)
    kc = np.ascontiguousarray(kc, dtype=np.float32)
    vc = np.ascontiguousarray(vc, dtype=np.float32)
    out = np.empty(nh * hd, dtype=np.float32)
    lib().orc_attention(_p(q), _p(kc), _p(vc), length, lo, nh, nkv, hd, _p(out), threads or cpu_threads())
    return out


class LlamaCfg(C.Structure):
    _fields_ = [(n, C.c_uint32) for n in ("n_layers", "h", "nh", "nkv", "hd", "inter", "vocab", "interleaved")] + [("eps", C.c_float),
                                                                                                                  ("scale", C.c_float)]


class Llama:
    """The CPU decoder: per layer matrices q k v o gate up down, norms ln_pre ln_post; final norm; head.
    Keeps its own KV caches [n_layers][max_len][nkv][hd]."""

    def __init__(self, cfg: LlamaCfg, layers: list[dict], final_norm: np.ndarray, head: Matrix, max_len: int):
        self.cfg, self.layers, self.head, self.max_len = cfg, layers, head, max_len
        mats = []
        norms = []
        for L in layers:
            mats += [L[k].h for k in ("q", "k", "v", "o", "gate", "up", "down")]
            norms += [np.ascontiguousarray(L["ln_pre"], dtype=np.float32), np.ascontiguousarray(L["ln_post"], dtype=np.float32)]
        mats.append(head.h)
        norms.append(np.ascontiguousarray(final_norm, dtype=np.float32))
        self._norms = norms
        self._mats = (C.c_void_p * len(mats))(*mats)
        self._normp = (C.c_void_p * len(norms))(*[_p(n) for n in norms])
        row = cfg.nkv * cfg.hd
        self.kc = np.zeros((cfg.n_layers, max_len, row), dtype=np.float32)
        self.vc = np.zeros((cfg.n_layers, max_len, row), dtype=np.float32)

    def step(self, pos: int, x: np.ndarray, rope_cs: np.ndarray, exact: bool, want_logits: bool = True, threads: int | None = None):
        """`exact`: matrix-vector products as f64 sums over the dequantized weights; else the CPU decode kernels."""
        x = np.ascontiguousarray(x, dtype=np.float32)
        cs = np.ascontiguousarray(rope_cs, dtype=np.float32)
        hidden = np.empty(self.cfg.h, dtype=np.float32)
        logits = np.empty(self.cfg.vocab, dtype=np.float32) if want_logits else None
        lib().orc_llama_step(C.byref(self.cfg), self._mats, self._normp, _p(self.kc), _p(self.vc), self.max_len, pos, _p(x), _p(cs), _p(hidden),
                             _p(logits) if logits is not None else None, int(exact), threads or cpu_threads())
        return hidden, logits


# ---- the reference's own CUDA kernels (oracle/_ref/libref_cuda.so, built by build_ref.py where the reference's tree is) ----
def ref_cuda():
    """The harness library around the reference's CUDA decode kernels, or None when it was not built."""
    from . import build_ref

    path = build_ref.build()
    if path is None or not Path(path).exists():
        return None
    L = C.CDLL(str(path))
    L.ref_dmv_q4a.restype = C.c_int
    L.ref_dmv_q4a.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint, C.c_uint, C.c_void_p, C.c_void_p, C.c_uint, C.c_uint, C.c_int,
                              C.POINTER(C.c_float), C.c_void_p]
    vp, u, f = C.c_void_p, C.c_uint, C.c_float
    for name, args in (("ref_norm", [vp, vp, vp, u, u, f, f, u, vp]),
                       ("ref_qk_rope", [vp] * 10 + [u] * 5 + [f, vp]),
                       ("ref_attend", [vp] * 6 + [u, u, u, f, u, C.c_int, C.POINTER(f), vp]),
                       ("ref_glu", [vp, vp, vp, u, u, vp]),
                       ("ref_gemm_q4a", [vp, vp, vp, u, u, vp, vp, u, u, u, C.c_int, C.POINTER(f), vp]),
                       ("ref_moe_q4a", [vp] * 6 + [u, u, u, u, vp, u, u, vp, vp, vp, vp, u, vp, vp, vp, vp, vp, C.c_int, C.POINTER(f), vp])):
        fn = getattr(L, name)
        fn.restype, fn.argtypes = C.c_int, args
    return L


def _ref_rc(rc: int) -> None:
    if rc != 0:
        raise RuntimeError(f"the reference kernel failed with CUDA error {rc}")


def ref_norm(L, x, out, w, eps: float, pre: float = 1.0, add: bool = False) -> None:
    """dnorm (src/cuda_decode.cu) over the rows of the torch CUDA tensor ``x`` [rows][n]; ``w`` a tensor or None."""
    rows, n = x.shape
    _ref_rc(L.ref_norm(x.data_ptr(), out.data_ptr(), w.data_ptr() if w is not None else None, n, rows, eps, pre, int(add), None))


def ref_qk_rope(L, qkv, q_out, kc, vc, k_out, v_out, qn, kn, cs, sp, nh: int, nkv: int, hd: int, half_rot: int, interleaved: bool,
                eps: float) -> None:
    """dqk_rope: caches ``kc`` / ``vc`` are [max_len][nkv][hd] f32 tensors, ``sp`` an int32 tensor of 4 with sp[0] = position."""
    _ref_rc(L.ref_qk_rope(qkv.data_ptr(), q_out.data_ptr(), kc.data_ptr(), vc.data_ptr(), k_out.data_ptr(), v_out.data_ptr(),
                          qn.data_ptr() if qn is not None else None, kn.data_ptr() if kn is not None else None, cs.data_ptr(), sp.data_ptr(),
                          nh, nkv, hd, half_rot, int(interleaved), eps, None))


def ref_attend(L, q, kc, vc, out, sp, nh: int, nkv: int, hd: int, scale: float, window: int = 0, iters: int = 0) -> float:
    """dattn_* + dattn_combine over positions 0 .. sp[0]; returns the mean device milliseconds of the pair (``iters`` > 0)."""
    import torch

    part = torch.zeros(nh * 64 * (hd + 2), device=q.device)
    ms = C.c_float()
    _ref_rc(L.ref_attend(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), out.data_ptr(), part.data_ptr(), sp.data_ptr(), nh, nkv, hd, scale, window,
                         iters, C.byref(ms), None))
    return ms.value


def ref_glu(L, g, u, out, gelu: bool = False) -> None:
    _ref_rc(L.ref_glu(g.data_ptr(), u.data_ptr(), out.data_ptr(), g.numel(), int(gelu), None))


def ref_gemm_q4a(L, m: Matrix, x, y, iters: int = 0) -> float:
    """The reference's prefill kernel gemm_q4a: ``x`` [tokens][n_in], ``y`` [tokens][n_out] torch CUDA f32 tensors, tokens and
    n_out multiples of 64. Returns the mean device milliseconds of a launch (``iters`` > 0)."""
    import torch

    q, s, o, group = m.q4_parts()
    dq, ds, do = (torch.from_numpy(a).cuda() for a in (q, s.view(np.int16), o.view(np.int16)))
    ms = C.c_float()
    _ref_rc(L.ref_gemm_q4a(dq.data_ptr(), ds.data_ptr(), do.data_ptr(), m.n_in // group, group // 32, x.data_ptr(), y.data_ptr(), m.n_out, m.n_in,
                           x.shape[0], iters, C.byref(ms), None))
    return ms.value


def ref_dmv_q4a(L, m: Matrix, x, y, iters: int = 1, stream: int = 0) -> float:
    """The reference's one-token affine-Q4 matvec (src/cuda_decode.cu dmv_q4a) on the current CUDA device: ``m`` from
    ``Matrix.from_mlx_q4``, ``x`` / ``y`` torch CUDA tensors. Returns the mean device milliseconds of a launch."""
    import torch

    q, s, o, group = m.q4_parts()
    dq, ds, do = (torch.from_numpy(a).cuda() for a in (q, s.view(np.int16), o.view(np.int16)))
    ms = C.c_float()
    rc = L.ref_dmv_q4a(dq.data_ptr(), ds.data_ptr(), do.data_ptr(), m.n_in // group, group // 32, x.data_ptr(), y.data_ptr(), m.n_out, m.n_in, iters,
                       C.byref(ms), stream)
    if rc != 0:
        raise RuntimeError(f"the reference kernel failed with CUDA error {rc}")
    return ms.value


class RefMoe:
    """The experts of one MoE layer as the reference's CUDA backend holds them (per expert the Q4Matrix arrays of the fused
    gate_up and of the down projection on the device), for ``ref_moe_q4a``. ``gate_up`` / ``down``: oracle matrices made by
    ``Matrix.from_mlx_q4``."""

    def __init__(self, gate_up: list, down: list, h: int, inter: int):
        import torch

        self.h, self.inter, self.n = h, inter, len(gate_up)
        self.keep, tabs = [], [[] for _ in range(6)]
        self.group = None
        for e in range(self.n):
            for base, m in ((0, gate_up[e]), (3, down[e])):
                q, s, o, group = m.q4_parts()
                self.group = group
                for j, a in enumerate((q, s.view(np.int16), o.view(np.int16))):
                    d = torch.from_numpy(a).cuda()
                    self.keep.append(d)
                    tabs[base + j].append(d.data_ptr())
        self.tabs = [(C.c_void_p * self.n)(*t) for t in tabs]


def ref_moe_q4a(L, rm: RefMoe, x, route_ids: np.ndarray, route_w: np.ndarray, y, iters: int = 0) -> float:
    """One routed-expert layer with the reference's own kernels in the sequence of CudaBackend::moe_run
    (src/cuda.rs:798-966): segments per expert padded to its 64-row GEMM tile, built here on the host as moe_run builds
    them. ``x``, ``y``: torch CUDA f32 [t][h]; y is added to once per run of the sequence (1 + iters runs). Returns the
    mean device milliseconds of one sequence."""
    import torch

    t, k = route_ids.shape
    TILE = 64
    count = np.bincount(route_ids.reshape(-1), minlength=rm.n)
    seg_len = ((count + TILE - 1) // TILE * TILE).astype(np.uint32)
    seg_start = np.concatenate([[0], np.cumsum(seg_len)[:-1]]).astype(np.uint32)
    rows = int(seg_len.sum())
    src = np.full(rows, t, np.uint32)
    slots = np.zeros(2 * t * k, np.uint32)
    fill = seg_start.astype(np.int64).copy()
    wbits = np.ascontiguousarray(route_w, dtype=np.float32).view(np.uint32)
    for i in range(t):
        for j in range(k):
            e = int(route_ids[i, j])
            r = fill[e]
            fill[e] += 1
            src[r] = i
            slots[2 * (i * k + j)] = r
            slots[2 * (i * k + j) + 1] = wbits[i, j]
    dsrc, dslots = torch.from_numpy(src.view(np.int32)).cuda(), torch.from_numpy(slots.view(np.int32)).cuda()
    xs = torch.empty((rows, rm.h), device="cuda")
    gu = torch.empty((rows, 2 * rm.inter), device="cuda")
    a = torch.empty((rows, rm.inter), device="cuda")
    o = torch.empty((rows, rm.h), device="cuda")
    ms = C.c_float()
    _ref_rc(L.ref_moe_q4a(*rm.tabs, rm.n, rm.h, rm.inter, rm.group, x.data_ptr(), t, k, dsrc.data_ptr(), dslots.data_ptr(),
                          seg_start.ctypes.data, seg_len.ctypes.data, rows, xs.data_ptr(), gu.data_ptr(), a.data_ptr(), o.data_ptr(), y.data_ptr(),
                          iters, C.byref(ms), None))
    return ms.value
