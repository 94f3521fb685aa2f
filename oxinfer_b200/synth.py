"""Seeded synthetic weights and activations with the shapes and value distributions of the
benchmark configurations (no checkpoints or datasets are read anywhere in this repository).

Formats are produced directly in their on-disk byte layouts: the MLX triple
(``src/safetensors.rs:767-853``), GGUF Q4_K / Q6_K / Q8_0 blocks (``src/ggml.rs:750-793,707-712``) and
FP8 e4m3 with 128 x 128 block scales (``src/ggml.rs:240-256``).
"""
from __future__ import annotations

import numpy as np

from ._lib import FMT_F8E4M3, FMT_Q4_K, FMT_Q6_K, FMT_Q8_0
from .backend import Gguf, MlxQ4


def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even bf16 bit patterns of finite f32 values."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


def bf16_bits_to_f32(h: np.ndarray) -> np.ndarray:
    return (h.astype(np.uint32) << 16).view(np.float32)


def bf16_round(x: np.ndarray) -> np.ndarray:
    """f32 values rounded to the nearest bf16 (still stored as f32)."""
    return bf16_bits_to_f32(f32_to_bf16_bits(x)).reshape(np.shape(x))


def activations(t: int, n_in: int, seed: int) -> np.ndarray:
    """``[t, n_in]`` N(0,1) values that are exactly representable in bf16, as f32."""
    rng = np.random.default_rng(seed)
    return bf16_round(rng.standard_normal((t, n_in), dtype=np.float32))


def mlx4(n_out: int, n_in: int, seed: int, group: int = 64) -> MlxQ4:
    """Uniform nibbles; scale ~ U(0.005, 0.02) and bias = -8 scale + N(0, 1e-3), both bf16."""
    rng = np.random.default_rng(seed)
    w = rng.integers(0, 2**32, size=(n_out, n_in // 8), dtype=np.uint64).astype(np.uint32)
    s = bf16_round(rng.uniform(0.005, 0.02, size=(n_out, n_in // group)).astype(np.float32))
    b = (-8.0 * s + 1e-3 * rng.standard_normal(s.shape, dtype=np.float32)).astype(np.float32)
    return MlxQ4(np.ascontiguousarray(w), f32_to_bf16_bits(s).reshape(s.shape), f32_to_bf16_bits(b).reshape(s.shape), group)


def _f16_bits(x: np.ndarray) -> np.ndarray:
    return np.ascontiguousarray(x, dtype=np.float32).astype(np.float16).view(np.uint16)


def q4_k(n_out: int, n_in: int, seed: int) -> Gguf:
    """d, dmin ~ |N(0, 0.01)| as f16; the 12 scale bytes and 128 quant bytes uniform."""
    rng = np.random.default_rng(seed)
    nb = n_out * (n_in // 256)
    blk = rng.integers(0, 256, size=(nb, 144), dtype=np.uint16).astype(np.uint8)
    d = _f16_bits(np.abs(0.01 * rng.standard_normal(nb)))
    dm = _f16_bits(np.abs(0.01 * rng.standard_normal(nb)))
    blk[:, 0], blk[:, 1] = d & 0xFF, d >> 8
    blk[:, 2], blk[:, 3] = dm & 0xFF, dm >> 8
    return Gguf(FMT_Q4_K, np.ascontiguousarray(blk.reshape(-1)))


def q6_k(n_out: int, n_in: int, seed: int) -> Gguf:
    rng = np.random.default_rng(seed)
    nb = n_out * (n_in // 256)
    blk = rng.integers(0, 256, size=(nb, 210), dtype=np.uint16).astype(np.uint8)
    d = _f16_bits(0.002 * rng.standard_normal(nb))
    blk[:, 208], blk[:, 209] = d & 0xFF, d >> 8
    return Gguf(FMT_Q6_K, np.ascontiguousarray(blk.reshape(-1)))


def q8_0(n_out: int, n_in: int, seed: int) -> Gguf:
    rng = np.random.default_rng(seed)
    nb = n_out * (n_in // 32)
    blk = rng.integers(0, 256, size=(nb, 34), dtype=np.uint16).astype(np.uint8)
    d = _f16_bits(0.01 * rng.standard_normal(nb))
    blk[:, 0], blk[:, 1] = d & 0xFF, d >> 8
    return Gguf(FMT_Q8_0, np.ascontiguousarray(blk.reshape(-1)))


def f8_e4m3(n_out: int, n_in: int, seed: int, bs_rows: int = 128, bs_cols: int = 128) -> Gguf:
    """W ~ N(0, 0.02), one scale ~ U(1e-4, 1e-3) per block, q = e4m3(W / scale) saturated at 448."""
    import torch

    rng = np.random.default_rng(seed)
    nrb, ncb = -(-n_out // bs_rows), -(-n_in // bs_cols)
    scales = rng.uniform(1e-4, 1e-3, size=(nrb, ncb)).astype(np.float32)
    out = np.empty((n_out, n_in), dtype=np.uint8)
    step = max(1, (1 << 24) // n_in)
    for r0 in range(0, n_out, step):  # bounded working set for the 28672 x 12288 case
        r1 = min(n_out, r0 + step)
        w = 0.02 * rng.standard_normal((r1 - r0, n_in), dtype=np.float32)
        s = np.repeat(np.repeat(scales[r0 // bs_rows : -(-r1 // bs_rows)], bs_rows, axis=0)[(r0 % bs_rows) : (r0 % bs_rows) + r1 - r0],
                      bs_cols, axis=1)[:, :n_in]
        q = torch.from_numpy(np.clip(w / s, -448.0, 448.0)).to(torch.float8_e4m3fn)
        out[r0:r1] = q.view(torch.uint8).numpy()
    return Gguf(FMT_F8E4M3, np.ascontiguousarray(out.reshape(-1)), scales, bs_rows, bs_cols)


def make(fmt: str, n_out: int, n_in: int, seed: int):
    return {"mlx4": mlx4, "q4_k": q4_k, "q6_k": q6_k, "q8_0": q8_0, "f8_e4m3": f8_e4m3}[fmt](n_out, n_in, seed)
