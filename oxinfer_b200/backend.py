"""Host-side mirror of oxinfer's accelerator boundary for this engine.

The names follow the reference's ``gpu::Backend`` trait (``src/gpu.rs:151-294``) and its CUDA
implementation (``src/cuda.rs``): ``wants``, ``upload``, ``matmul`` with ``Job`` s, ``matvec_rows``
with ``RowsJob`` s, ``stats``. Results follow the same convention: ``False`` / ``None`` means
"declined, nothing was computed" (the reference's caller then runs the batch on the CPU,
``src/model.rs:875-886``); errors raise ``BackendError``. Everything goes through the C ABI of
``include/b200qmm.h``; there is no other compute path.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, field

import numpy as np

from . import _lib
from ._lib import (BF16, DECLINED, F16, F32, FMT_F8E4M3, FMT_MLX4, FMT_Q4_K, FMT_Q6_K, FMT_Q8_0, MODE_ADD, MODE_ADD_GATED, MODE_GELU_PAIR,
                   MODE_SILU_PAIR, MODE_STORE, OK)


class BackendError(RuntimeError):
    def __init__(self, code: int, text: str):
        super().__init__(f"{text} (code {code})")
        self.code = code


@dataclass
class MlxQ4:
    """``WeightRef::Q4`` with offsets in its on-disk MLX form: u32 words, bf16 scales and biases."""
    w: np.ndarray        # uint32 [n_out, n_in/8]
    scales: np.ndarray   # uint16 (bf16 bits) [n_out, n_in/group]
    biases: np.ndarray   # uint16 (bf16 bits) [n_out, n_in/group]
    group: int = 64


@dataclass
class Q4Matrix:
    """``WeightRef::Q4(&Q4Matrix)`` as a backend receives it (``src/gpu.rs:15-21``, ``src/quant.rs:427-440``): Q4_0-order
    nibbles, an f16 scale per 32 weights and, for MLX checkpoints, a bf16 offset per group."""
    q: np.ndarray               # uint8 [n_out, n_in/2]
    scales: np.ndarray          # uint16 (f16 bits) [n_out, n_in/32]
    offsets: np.ndarray | None  # uint16 (bf16 bits) [n_out, n_in/group]
    group: int = 64


@dataclass
class Gguf:
    """``WeightRef::Gguf``: raw rows of a GGUF block format, FP8 with its block scales."""
    kind: int            # FMT_Q4_K / FMT_Q6_K / FMT_Q8_0 / FMT_F8E4M3
    data: np.ndarray     # uint8, row-major
    block_scales: np.ndarray | None = None  # float32 [ceil(n_out/rows), ceil(n_in/cols)]
    bs_rows: int = 128
    bs_cols: int = 128


class DeviceWeight:
    """Device-side state of one matrix, owned by the layer that uploaded it (``src/gpu.rs:57``)."""

    def __init__(self, backend: "Backend", handle: int, n_out: int, n_in: int, fmt: int):
        self.backend, self.handle, self.n_out, self.n_in, self.fmt = backend, handle, n_out, n_in, fmt

    def bytes(self) -> int:
        return _lib.lib().b2_weight_bytes(self.backend._ctx, self.handle)

    def free(self) -> None:
        if self.handle and self.backend._ctx:
            _lib.lib().b2_free_weight(self.backend._ctx, self.handle)
        self.handle = 0

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


class MoeWeights:
    """Device state of one MoE layer's routed experts (stacked gate/up and down matrices)."""

    def __init__(self, backend: "Backend", handle: int, experts: int, h: int, inter: int):
        self.backend, self.handle, self.experts, self.h, self.inter = backend, handle, experts, h, inter

    def free(self) -> None:
        if self.handle and self.backend._ctx:
            _lib.lib().b2_free_moe(self.backend._ctx, self.handle)
        self.handle = 0

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


@dataclass
class Job:
    """One matmul of a batch sharing the input (``src/gpu.rs:60-65``): ``y[t][n_out] = x W^T``."""
    dev: DeviceWeight
    y: np.ndarray  # float32 [t, n_out], written in place


@dataclass
class RowsJob:
    """``src/gpu.rs:69-75``: ``y = W x`` or, with ``up``, ``y = silu(W x) * (U x)``."""
    dev: DeviceWeight
    y: np.ndarray
    up: DeviceWeight | None = None


def _ptr(a) -> int:
    """Address of a numpy array or of a torch tensor (host or device)."""
    if isinstance(a, np.ndarray):
        assert a.flags["C_CONTIGUOUS"]
        return a.ctypes.data
    assert a.is_contiguous()
    return a.data_ptr()


class _DeviceArray:
    """A raw device pointer with a shape, as torch reads it (``__cuda_array_interface__``)."""

    def __init__(self, ptr: int, shape: tuple):
        self.__cuda_array_interface__ = {"shape": shape, "typestr": "<f4", "data": (ptr, False), "version": 2}


def _device_f32_tensor(ptr: int, shape: tuple, device):
    """An f32 torch tensor over device memory the library owns (no copy)."""
    import torch

    return torch.as_tensor(_DeviceArray(ptr, shape), device=device)


_TORCH_DTYPES = None


def _dtype_code(t) -> int:
    global _TORCH_DTYPES
    if _TORCH_DTYPES is None:
        import torch

        _TORCH_DTYPES = {torch.float32: F32, torch.bfloat16: BF16, torch.float16: F16}
    return _TORCH_DTYPES[t.dtype]


class Backend:
    """One B200 bound through ``b2_open`` (``CudaBackend::new``, ``src/cuda.rs:448-570``)."""

    def __init__(self, ordinal: int = 0):
        self._L = _lib.lib()
        ctx = C.c_void_p()
        rc = self._L.b2_open(ordinal, C.byref(ctx))
        if rc != OK:
            raise BackendError(rc, self._L.b2_open_error().decode())
        self._ctx = ctx
        self.ordinal = ordinal

    def close(self) -> None:
        if getattr(self, "_ctx", None):
            self._L.b2_close(self._ctx)
            self._ctx = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # -- helpers ------------------------------------------------------------------------------
    def _check(self, rc: int) -> bool:
        """True = done, False = declined, raises on error."""
        if rc == OK:
            return True
        if rc == DECLINED:
            self.last_declined = self._L.b2_last_error(self._ctx).decode()
            return False
        raise BackendError(rc, self._L.b2_last_error(self._ctx).decode())

    def name(self) -> str:
        return "b200"

    def set_stream(self, cuda_stream: int) -> None:
        self._check(self._L.b2_set_stream(self._ctx, cuda_stream))

    def launch_count(self) -> int:
        return self._L.b2_launch_count(self._ctx)

    def stats(self) -> str:
        return self._L.b2_stats(self._ctx).decode()

    def set_chained(self, on: bool) -> None:
        """Device-resident matrix-vector calls launch as a dependent chain (each kernel may start while the one ahead drains)."""
        self._check(self._L.b2_set_chained(self._ctx, int(on)))

    def set_fast_planes(self, on: bool) -> None:
        """Matrix-vector products over 16 of the activations' 21 bits (no counterpart in the reference; off by default)."""
        self._check(self._L.b2_set_fast_planes(self._ctx, int(on)))

    def set_exact(self, on: bool) -> None:
        """``gpu::set_exact`` (``src/gpu.rs:313-338``): many-token matmuls with two-term f16 operands, within 1e-4 per row."""
        self._check(self._L.b2_set_exact(self._ctx, int(on)))

    def set_fp8_activations(self, on: bool) -> None:
        """FP8 weights x FP8 activations (``b2_set_fp8_activations``): activations quantized per token and per 128 k to e4m3."""
        self._check(self._L.b2_set_fp8_activations(self._ctx, int(on)))

    def check_status(self) -> None:
        self._check(self._L.b2_check_status(self._ctx))

    # -- the trait ----------------------------------------------------------------------------
    def wants(self, n_out: int, n_in: int, t: int) -> bool:
        return bool(self._L.b2_wants(self._ctx, n_out, n_in, t))

    def upload(self, w: "MlxQ4 | Q4Matrix | Gguf", n_out: int, n_in: int) -> DeviceWeight | None:
        h = C.c_uint64()
        if isinstance(w, Q4Matrix):
            assert w.q.dtype == np.uint8 and w.scales.dtype == np.uint16 and w.q.size == n_out * n_in // 2 and w.scales.size == n_out * n_in // 32
            assert w.offsets is None or (w.offsets.dtype == np.uint16 and w.offsets.size == n_out * n_in // w.group)
            rc = self._L.b2_upload_q4(self._ctx, _ptr(w.q), _ptr(w.scales), None if w.offsets is None else _ptr(w.offsets), w.group, n_out, n_in,
                                      C.byref(h))
            fmt = FMT_MLX4 if w.offsets is not None else 2  # plain Q4 becomes a Q4_0 weight
        elif isinstance(w, MlxQ4):
            assert w.w.dtype == np.uint32 and w.scales.dtype == np.uint16 and w.biases.dtype == np.uint16
            assert w.w.size == n_out * n_in // 8 and w.scales.size == n_out * n_in // w.group == w.biases.size
            rc = self._L.b2_upload_mlx4(self._ctx, _ptr(w.w), _ptr(w.scales), _ptr(w.biases), n_out, n_in, w.group, C.byref(h))
            fmt = FMT_MLX4
        else:
            assert w.data.dtype == np.uint8
            bs = None if w.block_scales is None else np.ascontiguousarray(w.block_scales, dtype=np.float32)
            rc = self._L.b2_upload_gguf(self._ctx, w.kind, _ptr(w.data), n_out, n_in, None if bs is None else _ptr(bs), w.bs_rows,
                                        w.bs_cols, C.byref(h))
            fmt = w.kind
        if not self._check(rc):
            return None
        return DeviceWeight(self, h.value, n_out, n_in, fmt)

    def shard_rows(self, dev: DeviceWeight, r0: int, r1: int) -> DeviceWeight:
        """Rows ``[r0, r1)`` as their own weight sharing ``dev``'s memory (``dev`` must outlive it)."""
        h = C.c_uint64()
        self._check(self._L.b2_shard_rows(self._ctx, dev.handle, r0, r1, C.byref(h)))
        s = DeviceWeight(self, h.value, r1 - r0, dev.n_in, dev.fmt)
        s._parent = dev
        return s

    def dequantize_rows(self, dev: DeviceWeight, r0: int = 0, r1: int | None = None) -> np.ndarray:
        r1 = dev.n_out if r1 is None else r1
        out = np.zeros((r1 - r0, dev.n_in), dtype=np.float32)
        self._check(self._L.b2_dequantize_rows(self._ctx, dev.handle, r0, r1, _ptr(out)))
        return out

    def matmul(self, x: np.ndarray, jobs: list[Job]) -> bool:
        x = np.ascontiguousarray(x, dtype=np.float32)
        t, n_in = x.shape
        arr = (_lib.Job * len(jobs))()
        for i, j in enumerate(jobs):
            assert j.y.dtype == np.float32 and j.y.shape == (t, j.dev.n_out) and j.y.flags["C_CONTIGUOUS"]
            arr[i] = _lib.Job(j.dev.handle, j.dev.n_out, _ptr(j.y))
        return self._check(self._L.b2_matmul(self._ctx, _ptr(x), t, n_in, arr, len(jobs)))

    def matvec_rows(self, x: np.ndarray, jobs: list[RowsJob]) -> bool:
        x = np.ascontiguousarray(x, dtype=np.float32)
        t, n_in = x.shape
        arr = (_lib.RowsJob * len(jobs))()
        for i, j in enumerate(jobs):
            assert j.y.dtype == np.float32 and j.y.shape == (t, j.dev.n_out) and j.y.flags["C_CONTIGUOUS"]
            arr[i] = _lib.RowsJob(j.dev.handle, j.up.handle if j.up else 0, j.dev.n_out, _ptr(j.y))
        return self._check(self._L.b2_matvec_rows(self._ctx, _ptr(x), t, n_in, arr, len(jobs)))

    # -- device-resident calls (torch tensors carry the device memory) ---------------------------
    def matmul_dev(self, dev: DeviceWeight, x, y) -> bool:
        """``y[t][n_out] = x[t][n_in] W^T`` on device tensors, no copies, no synchronization."""
        t = x.shape[0]
        assert x.shape[1] == dev.n_in and tuple(y.shape) == (t, dev.n_out) and x.is_cuda and y.is_cuda
        return self._check(self._L.b2_matmul_dev(self._ctx, dev.handle, _ptr(x), _dtype_code(x), t, _ptr(y), _dtype_code(y)))

    def matvec_dev(self, dev: DeviceWeight, x, y, mode: int = MODE_STORE, up: DeviceWeight | None = None, gate=None) -> bool:
        assert x.numel() == dev.n_in and y.numel() == dev.n_out and x.is_cuda and y.is_cuda
        return self._check(self._L.b2_matvec_dev(self._ctx, dev.handle, up.handle if up else 0, _ptr(x), _ptr(y), mode,
                                                 _ptr(gate) if gate is not None else None))

    # -- routed experts ---------------------------------------------------------------------------
    def upload_moe(self, gate_up: list, down: list, h: int, inter: int, up: list | None = None, act: int = 0, act_limit: float = 0.0) -> "MoeWeights | None":
        """``Backend::upload_moe`` (``src/gpu.rs:200-215``): per-expert weights already uploaded with ``upload``. With ``up`` the gate
        and up projections come apart; ``act``: 0 SiLU, 1 tanh GELU, 2 SiLU clamped at ``act_limit`` (``MoeAct``)."""
        n = len(gate_up)
        gu = (C.c_uint64 * n)(*[d.handle for d in gate_up])
        dn = (C.c_uint64 * n)(*[d.handle for d in down])
        up_arr = (C.c_uint64 * n)(*[d.handle for d in up]) if up is not None else None
        hd = C.c_uint64()
        if not self._check(self._L.b2_upload_moe_ex(self._ctx, C.cast(gu, C.c_void_p), C.cast(up_arr, C.c_void_p) if up_arr is not None else None,
                                                    C.cast(dn, C.c_void_p), n, h, inter, act, act_limit, C.byref(hd))):
            return None
        return MoeWeights(self, hd.value, n, h, inter)

    def moe(self, x: np.ndarray, routes_ids: np.ndarray, routes_w: np.ndarray, dev: "MoeWeights", y: np.ndarray) -> bool:
        """``Backend::moe`` (``src/gpu.rs:232-248``): ``y[i] += sum_j w_ij down(silu(gate x_i) * up x_i)``, y in place."""
        x = np.ascontiguousarray(x, dtype=np.float32)
        ids = np.ascontiguousarray(routes_ids, dtype=np.int32)
        w = np.ascontiguousarray(routes_w, dtype=np.float32)
        t, k = ids.shape
        assert x.shape == (t, dev.h) and y.shape == (t, dev.h) and y.dtype == np.float32 and y.flags["C_CONTIGUOUS"]
        return self._check(self._L.b2_moe(self._ctx, dev.handle, _ptr(x), t, _ptr(ids), _ptr(w), k, _ptr(y)))

    def moe_dev(self, x, routes_ids: np.ndarray, routes_w: np.ndarray, dev: "MoeWeights", y) -> bool:
        """``moe`` with x and y resident on the device (torch tensors); the routes stay host arrays. Not synchronized."""
        ids = np.ascontiguousarray(routes_ids, dtype=np.int32)
        w = np.ascontiguousarray(routes_w, dtype=np.float32)
        t, k = ids.shape
        return self._check(self._L.b2_moe_dev(self._ctx, dev.handle, _ptr(x), t, _ptr(ids), _ptr(w), k, _ptr(y)))

    def route_topk_dev(self, logits, k: int, ids, w) -> bool:
        t, n = logits.shape
        return self._check(self._L.b2_route_topk_dev(self._ctx, _ptr(logits), t, n, k, _ptr(ids), _ptr(w)))

    # -- several GPUs (one process per GPU; collectives over NCCL, opened by the library itself) ----------------------
    @staticmethod
    def comm_unique_id() -> bytes:
        """Rank 0 makes the id; the other processes receive its bytes by any host channel."""
        buf = C.create_string_buffer(_lib.COMM_ID_BYTES)
        rc = _lib.lib().b2_comm_unique_id(buf)
        if rc != OK:
            raise BackendError(rc, "b2_comm_unique_id: NCCL is not available")
        return buf.raw

    def comm_init(self, world: int, rank: int, comm_id: bytes) -> bool:
        assert len(comm_id) == _lib.COMM_ID_BYTES
        self.world, self.rank = world, rank
        return self._check(self._L.b2_comm_init(self._ctx, world, rank, comm_id))

    def comm_free(self) -> None:
        self._check(self._L.b2_comm_free(self._ctx))

    def matmul_sharded(self, shard: DeviceWeight, x, y) -> bool:
        """``y[t][world * n_local]`` (f32, full on every rank) from this rank's row shard; collective."""
        t = x.shape[0]
        assert x.shape[1] == shard.n_in and y.shape[0] == t and y.is_cuda and x.is_cuda
        return self._check(self._L.b2_matmul_sharded(self._ctx, shard.handle, _ptr(x), _dtype_code(x), t, _ptr(y)))

    def matmul_sharded_peer(self, shard: DeviceWeight, x):
        """The same with the gather done by the GEMM's epilogue (peer stores over NVLink): returns this rank's full ``y`` as a
        torch tensor over the library's buffer (valid until the call after the next one), or None when declined; collective."""
        import torch

        t = x.shape[0]
        assert x.shape[1] == shard.n_in and x.is_cuda
        out = C.c_void_p()
        if not self._check(self._L.b2_matmul_sharded_peer(self._ctx, shard.handle, _ptr(x), _dtype_code(x), t, C.byref(out))):
            return None
        return _device_f32_tensor(out.value, (t, shard.n_out * self.world), x.device)

    def moe_ep(self, x, routes_ids: np.ndarray, routes_w: np.ndarray, dev: "MoeWeights", n_experts_global: int, y) -> bool:
        """Expert-parallel ``moe``: ``dev`` holds this rank's experts, the routes name global experts; collective."""
        ids = np.ascontiguousarray(routes_ids, dtype=np.int32)
        w = np.ascontiguousarray(routes_w, dtype=np.float32)
        t, k = ids.shape
        return self._check(self._L.b2_moe_ep(self._ctx, dev.handle, n_experts_global, _ptr(x), t, _ptr(ids), _ptr(w), k, _ptr(y)))

    def prepare_x_dev(self, x) -> bool:
        """Splits a device vector into the integer planes the GEMV kernels read (once per vector)."""
        return self._check(self._L.b2_prepare_x_dev(self._ctx, _ptr(x), x.numel()))

    def matvec_prepared_dev(self, dev: DeviceWeight, x, y, mode: int = MODE_STORE, up: DeviceWeight | None = None, gate=None) -> bool:
        """One product over the planes prepared last by ``prepare_x_dev`` (same vector length)."""
        return self._check(self._L.b2_matvec_prepared_dev(self._ctx, dev.handle, up.handle if up else 0, _ptr(x), _ptr(y), mode,
                                                          _ptr(gate) if gate is not None else None))

    def dequantize_rows_dev(self, dev: DeviceWeight, out, r0: int = 0, r1: int | None = None) -> bool:
        r1 = dev.n_out if r1 is None else r1
        return self._check(self._L.b2_dequantize_rows_dev(self._ctx, dev.handle, r0, r1, _ptr(out)))
