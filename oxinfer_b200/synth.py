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


# The other GGUF block formats: (block elements, block bytes, [(offset of an f16 field, magnitude, signed)]); MXFP4's first
# byte is an E8M0 exponent instead (src/ggml.rs:173-215 for the sizes, src/ggml.rs:665-773, 915-960 for the fields).
OTHER_BLOCKS = {
    2: (32, 18, [(0, 0.01, True)]),                      # Q4_0
    3: (32, 20, [(0, 0.01, False), (2, 0.05, True)]),    # Q4_1
    6: (32, 22, [(0, 0.01, True)]),                      # Q5_0
    7: (32, 24, [(0, 0.01, False), (2, 0.05, True)]),    # Q5_1
    10: (256, 84, [(80, 0.01, False), (82, 0.01, False)]),   # Q2_K
    11: (256, 110, [(108, 0.002, True)]),                # Q3_K
    13: (256, 176, [(0, 0.01, False), (2, 0.01, False)]),    # Q5_K
    20: (32, 18, [(0, 0.001, True)]),                    # IQ4_NL
    23: (256, 136, [(0, 0.0001, True)]),                 # IQ4_XS
    39: (32, 17, []),                                    # MXFP4
}
OTHER_NAMES = {2: "q4_0", 3: "q4_1", 6: "q5_0", 7: "q5_1", 10: "q2_k", 11: "q3_k", 13: "q5_k", 20: "iq4_nl", 23: "iq4_xs", 39: "mxfp4"}


def other_blocks(kind: int, n_out: int, n_in: int, seed: int) -> Gguf:
    """Uniform random block bytes of one of the other GGUF formats with its f16 scale fields drawn as |N(0, magnitude)|
    (signed where the format's scale is) and MXFP4's exponent byte in 118 .. 124."""
    bs, ts, fields = OTHER_BLOCKS[kind]
    rng = np.random.default_rng(seed)
    nb = n_out * (n_in // bs)
    blk = rng.integers(0, 256, size=(nb, ts), dtype=np.uint16).astype(np.uint8)
    for off, mag, signed in fields:
        v = mag * rng.standard_normal(nb)
        d = _f16_bits(v if signed else np.abs(v))
        blk[:, off], blk[:, off + 1] = d & 0xFF, d >> 8
    if kind == 39:
        blk[:, 0] = rng.integers(118, 125, size=nb, dtype=np.uint16).astype(np.uint8)
    return Gguf(kind, np.ascontiguousarray(blk.reshape(-1)))


def make(fmt: str, n_out: int, n_in: int, seed: int):
    return {"mlx4": mlx4, "q4_k": q4_k, "q6_k": q6_k, "q8_0": q8_0, "f8_e4m3": f8_e4m3}[fmt](n_out, n_in, seed)


# ---- weights of a random-init model: zero mean, a chosen standard deviation --------------------------
# The block generators above draw every byte uniformly, which exercises every code path of the decoders but
# gives matrices with a large mean; a decoder stack needs y = W x to stay O(|x|). These keep the random
# bytes and choose the block constants so that the decoded weights are zero-mean with std `sigma`.

def q4_k_model(n_out: int, n_in: int, seed: int, sigma: float) -> Gguf:
    """Sub-block scales and mins uniform in 0..15, quants uniform, dmin = 7.5 d: w = d (sc q - 7.5 m) has mean 0 and
    std 63.5 d (from the moments of the three uniforms); d = sigma / 63.5 with a +-10 % spread per block."""
    rng = np.random.default_rng(seed)
    nb = n_out * (n_in // 256)
    blk = rng.integers(0, 256, size=(nb, 144), dtype=np.uint16).astype(np.uint8)
    blk[:, 4:12] &= 0x0F          # sc_j, m_j of sub-blocks 0..3 (bytes 4..11); bytes 12..15 hold sub-blocks 4..7 as nibbles
    d = (sigma / 63.5) * (1.0 + 0.1 * rng.uniform(-1, 1, nb))
    db, mb = _f16_bits(d), _f16_bits(7.5 * d)
    blk[:, 0], blk[:, 1] = db & 0xFF, db >> 8
    blk[:, 2], blk[:, 3] = mb & 0xFF, mb >> 8
    return Gguf(FMT_Q4_K, np.ascontiguousarray(blk.reshape(-1)))


def q6_k_model(n_out: int, n_in: int, seed: int, sigma: float) -> Gguf:
    """Sub-block scales uniform in -8..7, quants uniform: w = d sc (q - 32) has mean ~0 and std about 4.6 * 18.5 d."""
    rng = np.random.default_rng(seed)
    nb = n_out * (n_in // 256)
    blk = rng.integers(0, 256, size=(nb, 210), dtype=np.uint16).astype(np.uint8)
    blk[:, 192:208] = rng.integers(-8, 8, size=(nb, 16)).astype(np.int8).view(np.uint8)
    d = _f16_bits((sigma / (4.63 * 18.48)) * (1.0 + 0.1 * rng.uniform(-1, 1, nb)))
    blk[:, 208], blk[:, 209] = d & 0xFF, d >> 8
    return Gguf(FMT_Q6_K, np.ascontiguousarray(blk.reshape(-1)))


def q8_0_model(n_out: int, n_in: int, seed: int, sigma: float) -> Gguf:
    """Quants uniform in -128..127: w = d q has std 73.9 d."""
    rng = np.random.default_rng(seed)
    nb = n_out * (n_in // 32)
    blk = rng.integers(0, 256, size=(nb, 34), dtype=np.uint16).astype(np.uint8)
    d = _f16_bits((sigma / 73.9) * (1.0 + 0.1 * rng.uniform(-1, 1, nb)))
    blk[:, 0], blk[:, 1] = d & 0xFF, d >> 8
    return Gguf(FMT_Q8_0, np.ascontiguousarray(blk.reshape(-1)))


def llama_weights(n_layers: int, h: int, nh: int, nkv: int, hd: int, inter: int, vocab: int, seed: int, same_layers: bool = False,
                  mixed: bool = False):
    """Random-init weights of a Llama-style decoder in the formats of a GGUF Q4_K_M-like checkpoint: Q4_K body,
    Q6_K head, Q8_0 embeddings, f32 norms. Returns (layers, final_norm, head, embed); each layer is a dict of
    ``Gguf`` refs ``q k v o gate up down`` plus f32 ``ln_pre ln_post``. ``same_layers`` reuses layer 0's bytes for
    every layer (each still uploads to its own device memory): generation time only, the work per token is unchanged.
    ``mixed``: v and down in Q6_K (as Q4_K_M checkpoints keep them in half of their layers) and o in Q8_0."""
    rng = np.random.default_rng(seed)
    shapes = {"q": (nh * hd, h), "k": (nkv * hd, h), "v": (nkv * hd, h), "o": (h, nh * hd), "gate": (inter, h), "up": (inter, h),
              "down": (h, inter)}
    layers = []
    for li in range(n_layers):
        if same_layers and li > 0:
            layers.append(dict(layers[0]))
            continue
        L = {}
        for j, (name, (n_out, n_in)) in enumerate(shapes.items()):
            make = q4_k_model
            if mixed:
                make = {"v": q6_k_model, "down": q6_k_model, "o": q8_0_model}.get(name, q4_k_model)
            L[name] = make(n_out, n_in, seed + 100 * li + j + 1, 1.0 / np.sqrt(n_in))
        L["ln_pre"] = (1.0 + 0.1 * rng.standard_normal(h)).astype(np.float32)
        L["ln_post"] = (1.0 + 0.1 * rng.standard_normal(h)).astype(np.float32)
        layers.append(L)
    final_norm = (1.0 + 0.1 * rng.standard_normal(h)).astype(np.float32)
    head = q6_k_model(vocab, h, seed + 7001, 1.0 / np.sqrt(h))
    embed = q8_0_model(vocab, h, seed + 7002, 1.0)
    return layers, final_norm, head, embed, shapes
