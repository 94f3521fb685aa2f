// CPU oracle for the quantized-matmul path: TEST INFRASTRUCTURE, NOT PRODUCT CODE.
//
// A plain C++ restatement of oxinfer's CPU arithmetic for the formats and operators the CUDA
// engine implements. Only the test suite, the smoke check and the CPU-baseline leg of the
// benchmark may load this library; the CUDA product path never calls into it.
//
// Every function cites the reference source (path inside the oxinfer tree : line) it restates.
// Parity is PINNED: oracle/pin.py and tests/test_oracle_pins.py check the dequantizers against the
// reference's own known-answer hashes (src/ggml.rs:1547-1577, REF_HASHES) computed on the
// reference's own fixtures (src/ggml.rs:1437-1496, random_blocks), and the e4m3 decoder against the
// closed form of src/ggml.rs:258-271 for all 256 bytes.
//
// Third-party arithmetic restated here: crate `half` 2.7.1 (f16/bf16 <-> f32, IEEE round to
// nearest even), which the reference uses through src/quant.rs:449-455,580-583.

#include <algorithm>
#include <atomic>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <functional>
#include <thread>
#include <vector>

#if defined(__AVX2__) && defined(__FMA__)
#include <immintrin.h>
#define ORC_AVX2 1
#else
#define ORC_AVX2 0
#endif

#define ORC_API extern "C" __attribute__((visibility("default")))

namespace {

// ---------------------------------------------------------------------------------------------
// half / bf16 conversions (crate `half`: IEEE, round to nearest even).
// ---------------------------------------------------------------------------------------------
inline float bits_f32(uint32_t u) {
    float f;
    std::memcpy(&f, &u, 4);
    return f;
}
inline uint32_t f32_bits(float f) {
    uint32_t u;
    std::memcpy(&u, &f, 4);
    return u;
}

inline float f16_to_f32(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000) << 16;
    uint32_t e = (h >> 10) & 0x1f, m = h & 0x3ff;
    if (e == 0) {
        if (m == 0) return bits_f32(sign);
        // subnormal: m * 2^-24, exact in f32
        float v = (float)m * 5.9604644775390625e-8f;
        return bits_f32(f32_bits(v) | sign);
    }
    if (e == 31) return bits_f32(sign | 0x7f800000u | (m << 13));
    return bits_f32(sign | ((e + 112) << 23) | (m << 13));
}

inline uint16_t f32_to_f16(float f) {
    uint32_t x = f32_bits(f);
    uint32_t sign = (x >> 16) & 0x8000;
    uint32_t ax = x & 0x7fffffffu;
    if (ax >= 0x7f800000u) {  // inf / nan
        return (uint16_t)(sign | 0x7c00 | ((ax > 0x7f800000u) ? (0x200 | ((ax >> 13) & 0x3ff)) : 0));
    }
    if (ax >= 0x477ff000u) {  // rounds to >= 65520 -> inf
        return (uint16_t)(sign | 0x7c00);
    }
    if (ax < 0x38800000u) {  // below 2^-14: subnormal half
        if (ax < 0x33000000u) return (uint16_t)sign;  // < 2^-25 -> 0 (2^-25 itself ties to even = 0)
        uint32_t e = ax >> 23;
        uint32_t m = (ax & 0x7fffffu) | 0x800000u;
        uint32_t shift = 126 - e;  // 14..24
        uint32_t r = m >> shift;
        uint32_t rem = m & ((1u << shift) - 1), half = 1u << (shift - 1);
        if (rem > half || (rem == half && (r & 1))) r++;
        return (uint16_t)(sign | r);
    }
    uint32_t r = ((ax >> 13) - (112u << 10));
    uint32_t rem = ax & 0x1fffu;
    if (rem > 0x1000u || (rem == 0x1000u && (r & 1))) r++;
    return (uint16_t)(sign | r);
}

inline float bf16_to_f32(uint16_t h) { return bits_f32((uint32_t)h << 16); }
inline uint16_t f32_to_bf16(float f) {
    uint32_t x = f32_bits(f);
    if ((x & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((x >> 16) | 0x40);
    uint32_t lsb = (x >> 16) & 1;
    x += 0x7fffu + lsb;
    return (uint16_t)(x >> 16);
}

// ---------------------------------------------------------------------------------------------
// A small parallel-for over work items claimed from an atomic counter, like the reference's
// spin pool (src/pool.rs:262-310) but with plain threads.
// ---------------------------------------------------------------------------------------------
void parallel_for(size_t n, int threads, const std::function<void(size_t)>& f) {
    if (threads <= 1 || n <= 1) {
        for (size_t i = 0; i < n; i++) f(i);
        return;
    }
    std::atomic<size_t> next{0};
    auto body = [&] {
        for (;;) {
            size_t i = next.fetch_add(1, std::memory_order_relaxed);
            if (i >= n) break;
            f(i);
        }
    };
    std::vector<std::thread> ts;
    int nt = (int)std::min<size_t>((size_t)threads, n);
    for (int i = 1; i < nt; i++) ts.emplace_back(body);
    body();
    for (auto& t : ts) t.join();
}

// ---------------------------------------------------------------------------------------------
// GGUF kinds (ids of src/ggml.rs:42-93).
// ---------------------------------------------------------------------------------------------
enum Kind : int {
    K_F32 = 0, K_F16 = 1, K_Q4_0 = 2, K_Q4_1 = 3, K_Q5_0 = 6, K_Q5_1 = 7, K_Q8_0 = 8, K_Q2_K = 10, K_Q3_K = 11, K_Q4_K = 12, K_Q5_K = 13,
    K_Q6_K = 14, K_IQ4_NL = 20, K_IQ4_XS = 23, K_BF16 = 30, K_MXFP4 = 39, K_NVFP4 = 40, K_F8E4M3 = 0x1000
};
// The block kinds whose matrix products this file runs through the f32 route only (decoded bit-exactly here).
inline bool other_block_kind(int kind) {
    switch (kind) {
        case K_Q4_0: case K_Q4_1: case K_Q5_0: case K_Q5_1: case K_Q2_K: case K_Q3_K: case K_Q5_K: case K_IQ4_NL: case K_IQ4_XS: case K_MXFP4: case K_NVFP4: return true;
        default: return false;
    }
}

inline size_t block_size(int kind) {  // src/ggml.rs:173-185
    switch (kind) {
        case K_Q4_0: case K_Q4_1: case K_Q5_0: case K_Q5_1: case K_IQ4_NL: case K_MXFP4:
        case K_Q8_0: return 32;
        case K_NVFP4: return 64;
        case K_Q2_K: case K_Q3_K: case K_Q5_K: case K_IQ4_XS:
        case K_Q4_K:
        case K_Q6_K: return 256;
        default: return 1;
    }
}
inline size_t type_size(int kind) {  // src/ggml.rs:187-215
    switch (kind) {
        case K_F32: return 4;
        case K_F16:
        case K_BF16: return 2;
        case K_Q8_0: return 34;
        case K_Q4_0: case K_IQ4_NL: return 18;
        case K_Q4_1: return 20;
        case K_Q5_0: return 22;
        case K_Q5_1: return 24;
        case K_Q2_K: return 84;
        case K_Q3_K: return 110;
        case K_Q5_K: return 176;
        case K_IQ4_XS: return 136;
        case K_MXFP4: return 17;
        case K_NVFP4: return 36;
        case K_Q4_K: return 144;
        case K_Q6_K: return 210;
        case K_F8E4M3: return 1;
        default: return 0;
    }
}
inline size_t row_bytes(int kind, size_t n) { return n / block_size(kind) * type_size(kind); }

inline float f16at(const uint8_t* b, size_t i) { return f16_to_f32((uint16_t)(b[i] | (b[i + 1] << 8))); }

// src/ggml.rs:501-509 (get_scale_min_k4)
inline void scale_min_k4(int j, const uint8_t* q, uint8_t* sc, uint8_t* m) {
    if (j < 4) {
        *sc = q[j] & 63;
        *m = q[j + 4] & 63;
    } else {
        *sc = (uint8_t)((q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4));
        *m = (uint8_t)((q[j + 4] >> 4) | ((q[j] >> 6) << 4));
    }
}

inline uint32_t u32at(const uint8_t* b, size_t i) { return (uint32_t)b[i] | ((uint32_t)b[i + 1] << 8) | ((uint32_t)b[i + 2] << 16) | ((uint32_t)b[i + 3] << 24); }

// src/ggml.rs:466-474 (e8m0_half): 2^(e - 128), the subnormal cases from their bit patterns.
inline float e8m0_half(uint8_t e) { return bits_f32(e < 2 ? (0x00200000u << e) : (((uint32_t)e - 1) << 23)); }

// src/ggml.rs:477-491 (ue4m3_half): half the value of an unsigned E4M3 scale byte; 0 and 0x7f give 0.
inline float ue4m3_half(uint8_t x) {
    if (x == 0 || x == 0x7F) return 0.0f;
    const int e = (x >> 3) & 0xF;
    const float m = (float)(x & 7);
    const float raw = e == 0 ? m * std::ldexp(1.0f, -9) : (1.0f + m / 8.0f) * std::ldexp(1.0f, e - 7);
    return raw * 0.5f;
}

// src/ggml.rs:511-530 (q3k_scales): sixteen 6-bit scales from 12 bytes, still offset by 32.
inline void q3k_scales(const uint8_t* s, int8_t* out) {
    const uint32_t k1 = 0x03030303u, k2 = 0x0f0f0f0fu;
    const uint32_t a0 = u32at(s, 0), a1 = u32at(s, 4), tmp = u32at(s, 8);
    const uint32_t aux[4] = {(a0 & k2) | ((tmp & k1) << 4), (a1 & k2) | (((tmp >> 2) & k1) << 4), ((a0 >> 4) & k2) | (((tmp >> 4) & k1) << 4),
                             ((a1 >> 4) & k2) | (((tmp >> 6) & k1) << 4)};
    for (int i = 0; i < 4; i++)
        for (int j = 0; j < 4; j++) out[4 * i + j] = (int8_t)(uint8_t)(aux[i] >> (8 * j));
}

// src/ggml.rs:544-547 (iq4xs_scale)
inline int iq4xs_scale(const uint8_t* b, int ib) {
    const uint32_t sh = (uint32_t)b[2] | ((uint32_t)b[3] << 8);
    return (int)(((b[4 + ib / 2] >> (4 * (ib % 2))) & 0xF) | (((sh >> (2 * ib)) & 3) << 4)) - 32;
}

// ggml's published code books: the non-linear 4-bit values of IQ4_NL / IQ4_XS and the doubled E2M1 values of MXFP4.
const int8_t KV_IQ4NL[16] = {-127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113};
const int8_t KV_MXFP4[16] = {0, 1, 2, 3, 4, 6, 8, 12, 0, -1, -2, -3, -4, -6, -8, -12};

// src/ggml.rs:258-271
inline float e4m3_to_f32(uint8_t b) {
    float sign = (b & 0x80) ? -1.0f : 1.0f;
    int e = (b >> 3) & 0xF, m = b & 7;
    if (e == 0xF && m == 7) return std::nanf("");
    float v = e == 0 ? (float)m / 8.0f * std::ldexp(1.0f, -6) : (1.0f + (float)m / 8.0f) * std::ldexp(1.0f, e - 7);
    return sign * v;
}

// src/ggml.rs:630-793: one row of `kind` from its raw bytes. The products are written unfused and
// in the reference's order (this file is compiled with -ffp-contract=off).
void dequantize_row(int kind, const uint8_t* src, float* out, size_t n) {
    size_t bs = block_size(kind), ts = type_size(kind);
    if (kind == K_F32) {
        std::memcpy(out, src, n * 4);
        return;
    }
    if (kind == K_F16) {
        for (size_t i = 0; i < n; i++) out[i] = f16at(src, 2 * i);
        return;
    }
    if (kind == K_BF16) {
        for (size_t i = 0; i < n; i++) out[i] = bf16_to_f32((uint16_t)(src[2 * i] | (src[2 * i + 1] << 8)));
        return;
    }
    if (kind == K_F8E4M3) {
        for (size_t i = 0; i < n; i++) out[i] = e4m3_to_f32(src[i]);
        return;
    }
    for (size_t bi = 0; bi < n / bs; bi++) {
        const uint8_t* b = src + bi * ts;
        float* y = out + bi * bs;
        if (kind == K_Q8_0) {  // src/ggml.rs:707-712
            float d = f16at(b, 0);
            for (int j = 0; j < 32; j++) y[j] = (float)(int8_t)b[2 + j] * d;
        } else if (kind == K_Q4_0) {  // src/ggml.rs:673-679
            float d = f16at(b, 0);
            for (int j = 0; j < 16; j++) {
                y[j] = (float)((int)(b[2 + j] & 0xF) - 8) * d;
                y[j + 16] = (float)((int)(b[2 + j] >> 4) - 8) * d;
            }
        } else if (kind == K_Q4_1) {  // src/ggml.rs:680-686
            float d = f16at(b, 0), m = f16at(b, 2);
            for (int j = 0; j < 16; j++) {
                float p0 = (float)(b[4 + j] & 0xF) * d, p1 = (float)(b[4 + j] >> 4) * d;
                y[j] = p0 + m;
                y[j + 16] = p1 + m;
            }
        } else if (kind == K_Q5_0 || kind == K_Q5_1) {  // src/ggml.rs:687-706
            const bool one = kind == K_Q5_1;
            float d = f16at(b, 0), m = one ? f16at(b, 2) : 0.0f;
            const uint32_t qh = u32at(b, one ? 4 : 2);
            const uint8_t* qs = b + (one ? 8 : 6);
            for (int j = 0; j < 16; j++) {
                const uint32_t h0 = ((qh >> j) << 4) & 0x10, h1 = (qh >> (j + 12)) & 0x10;
                const int v0 = (int)((qs[j] & 0xF) | h0), v1 = (int)((qs[j] >> 4) | h1);
                if (one) {
                    float p0 = (float)v0 * d, p1 = (float)v1 * d;
                    y[j] = p0 + m;
                    y[j + 16] = p1 + m;
                } else {
                    y[j] = (float)(v0 - 16) * d;
                    y[j + 16] = (float)(v1 - 16) * d;
                }
            }
        } else if (kind == K_Q2_K) {  // src/ggml.rs:713-729
            float d = f16at(b, 80), mn = f16at(b, 82);
            const uint8_t* sc = b;
            const uint8_t* qs = b + 16;
            for (int nn = 0; nn < 2; nn++) {
                const uint8_t* q = qs + 32 * nn;
                for (int j = 0; j < 4; j++)
                    for (int h = 0; h < 2; h++) {
                        const uint8_t s = sc[8 * nn + 2 * j + h];
                        float dl = d * (float)(s & 0xF), ml = mn * (float)(s >> 4);
                        float* o = y + 128 * nn + 32 * j + 16 * h;
                        for (int l = 0; l < 16; l++) {
                            float p = dl * (float)((q[16 * h + l] >> (2 * j)) & 3);
                            o[l] = p - ml;
                        }
                    }
            }
        } else if (kind == K_Q3_K) {  // src/ggml.rs:730-749
            float d = f16at(b, 108);
            const uint8_t* hm = b;
            const uint8_t* qs = b + 32;
            int8_t sc[16];
            q3k_scales(b + 96, sc);
            for (int nn = 0; nn < 2; nn++) {
                const uint8_t* q = qs + 32 * nn;
                for (int j = 0; j < 4; j++) {
                    const uint8_t msk = (uint8_t)(1u << (4 * nn + j));
                    for (int h = 0; h < 2; h++) {
                        float dl = d * (float)((int)sc[8 * nn + 2 * j + h] - 32);
                        float* o = y + 128 * nn + 32 * j + 16 * h;
                        for (int l = 0; l < 16; l++) {
                            const int i = 16 * h + l;
                            const int v = (int)((q[i] >> (2 * j)) & 3) - ((hm[i] & msk) ? 0 : 4);
                            o[l] = dl * (float)v;
                        }
                    }
                }
            }
        } else if (kind == K_IQ4_NL) {  // src/ggml.rs:915-921
            float d = f16at(b, 0);
            for (int j = 0; j < 16; j++) {
                y[j] = d * (float)KV_IQ4NL[b[2 + j] & 0xF];
                y[j + 16] = d * (float)KV_IQ4NL[b[2 + j] >> 4];
            }
        } else if (kind == K_MXFP4) {  // src/ggml.rs:922-928
            float d = e8m0_half(b[0]);
            for (int j = 0; j < 16; j++) {
                y[j] = d * (float)KV_MXFP4[b[1 + j] & 0xF];
                y[j + 16] = d * (float)KV_MXFP4[b[1 + j] >> 4];
            }
        } else if (kind == K_NVFP4) {  // src/ggml.rs:936-947
            for (int sb = 0; sb < 4; sb++) {
                float d = ue4m3_half(b[sb]);
                const uint8_t* q = b + 4 + 8 * sb;
                for (int j = 0; j < 8; j++) {
                    y[16 * sb + j] = d * (float)KV_MXFP4[q[j] & 0xF];
                    y[16 * sb + j + 8] = d * (float)KV_MXFP4[q[j] >> 4];
                }
            }
        } else if (kind == K_IQ4_XS) {  // src/ggml.rs:948-958
            float d = f16at(b, 0);
            for (int ib = 0; ib < 8; ib++) {
                float dl = d * (float)iq4xs_scale(b, ib);
                const uint8_t* q = b + 8 + 16 * ib;
                for (int j = 0; j < 16; j++) {
                    y[32 * ib + j] = dl * (float)KV_IQ4NL[q[j] & 0xF];
                    y[32 * ib + j + 16] = dl * (float)KV_IQ4NL[q[j] >> 4];
                }
            }
        } else if (kind == K_Q4_K || kind == K_Q5_K) {  // src/ggml.rs:750-773
            const bool five = kind == K_Q5_K;
            float d = f16at(b, 0), mn = f16at(b, 2);
            const uint8_t* sc = b + 4;
            const uint8_t* qh = b + 16;
            const uint8_t* qs = b + (five ? 48 : 16);
            for (int j = 0; j < 4; j++) {
                const uint8_t* q = qs + 32 * j;
                for (int h = 0; h < 2; h++) {
                    uint8_t s, m;
                    scale_min_k4(2 * j + h, sc, &s, &m);
                    float d1 = d * (float)s, m1 = mn * (float)m;
                    float* o = y + 64 * j + 32 * h;
                    for (int l = 0; l < 32; l++) {
                        uint8_t v = (q[l] >> (4 * h)) & 0xF;
                        if (five && (qh[l] & (1 << (2 * j + h)))) v += 16;
                        float p = d1 * (float)v;
                        o[l] = p - m1;
                    }
                }
            }
        } else if (kind == K_Q6_K) {  // src/ggml.rs:774-793
            float d = f16at(b, 208);
            for (int nn = 0; nn < 2; nn++) {
                const uint8_t* ql = b + 64 * nn;
                const uint8_t* qh = b + 128 + 32 * nn;
                const uint8_t* sc = b + 192 + 8 * nn;
                float* o = y + 128 * nn;
                for (int l = 0; l < 32; l++) {
                    int is = l / 16;
                    int q1 = (int)((ql[l] & 0xF) | ((qh[l] & 3) << 4)) - 32;
                    int q2 = (int)((ql[l + 32] & 0xF) | (((qh[l] >> 2) & 3) << 4)) - 32;
                    int q3 = (int)((ql[l] >> 4) | (((qh[l] >> 4) & 3) << 4)) - 32;
                    int q4 = (int)((ql[l + 32] >> 4) | (((qh[l] >> 6) & 3) << 4)) - 32;
                    float a;
                    a = d * (float)(int8_t)sc[is];
                    o[l] = a * (float)q1;
                    a = d * (float)(int8_t)sc[is + 2];
                    o[l + 32] = a * (float)q2;
                    a = d * (float)(int8_t)sc[is + 4];
                    o[l + 64] = a * (float)q3;
                    a = d * (float)(int8_t)sc[is + 6];
                    o[l + 96] = a * (float)q4;
                }
            }
        }
    }
}

// src/ggml.rs:1437-1440
inline uint64_t lcg(uint64_t* s) {
    *s = *s * 6364136223846793005ull + 1442695040888963407ull;
    return *s >> 33;
}

// A weight matrix as the CPU path sees it: MLX affine 4-bit repacked to Q4_0 layout with per-group
// offsets (src/quant.rs:427-440), or raw GGUF rows with optional FP8 block scales
// (src/ggml.rs:240-256).
struct Matrix {
    int format = 0;  // 0 = Q4 (+offsets), 1 = GGUF
    int kind = 0;
    size_t n_out = 0, n_in = 0;
    // Q4
    std::vector<uint8_t> q;
    std::vector<uint16_t> scales;
    std::vector<uint16_t> offsets;
    size_t group = 0;
    // GGUF
    std::vector<uint8_t> data;
    std::vector<float> bscales;
    size_t bs_rows = 0, bs_cols = 0;

    size_t bytes() const {
        return format == 0 ? q.size() + scales.size() * 2 + offsets.size() * 2 : data.size();
    }
    // "dense" formats take the f32 path at every token count (src/ggml.rs:220-225).
    // The other block kinds also take it here: the reference multiplies them through an int8 block decode
    // (src/ggml.rs:965-1130) that this file does not restate; their products are checked against the f64 product of the
    // bit-exactly decoded weights.
    bool dense() const { return format == 1 && (kind == K_F8E4M3 || kind == K_F32 || kind == K_F16 || kind == K_BF16 || other_block_kind(kind)); }
};

// src/quant.rs:586-606
void dequantize_rows_q4(const Matrix& m, size_t r0, size_t r1, float* out) {
    size_t n_in = m.n_in, bpr = n_in / 32;
    for (size_t r = r0; r < r1; r++) {
        const uint8_t* qrow = m.q.data() + r * n_in / 2;
        const uint16_t* srow = m.scales.data() + r * bpr;
        float* orow = out + (r - r0) * n_in;
        for (size_t b = 0; b < bpr; b++) {
            float d = f16_to_f32(srow[b]);
            float off = m.offsets.empty() ? 0.0f : bf16_to_f32(m.offsets[r * (n_in / m.group) + b * 32 / m.group]);
            for (int j = 0; j < 16; j++) {
                uint8_t byte = qrow[b * 16 + j];
                float p0 = (float)((int)(byte & 0x0F) - 8) * d;
                float p1 = (float)((int)(byte >> 4) - 8) * d;
                orow[b * 32 + j] = p0 + off;
                orow[b * 32 + j + 16] = p1 + off;
            }
        }
    }
}

// src/ggml.rs:409-460 (GgufMatrix::dequantize_rows): FP8 rows take the block scale per `cols`
// chunk as `e4m3 * s` (src/ggml.rs:273-293); the other kinds go through dequantize_row.
void dequantize_rows_gguf(const Matrix& m, size_t r0, size_t r1, float* out) {
    size_t n = m.n_in, rb = row_bytes(m.kind, n);
    for (size_t r = r0; r < r1; r++) {
        float* o = out + (r - r0) * n;
        const uint8_t* w = m.data.data() + r * rb;
        if (m.kind == K_F8E4M3 && !m.bscales.empty()) {
            size_t ncb = (n + m.bs_cols - 1) / m.bs_cols;
            const float* srow = m.bscales.data() + (r / m.bs_rows) * ncb;
            for (size_t c = 0; c < n; c++) {
                float v = e4m3_to_f32(w[c]);
                o[c] = v * srow[c / m.bs_cols];
            }
        } else {
            dequantize_row(m.kind, w, o, n);
            if (!m.bscales.empty()) {  // scales on top of what the kind decodes (NVFP4's global scale), src/ggml.rs:420-432
                size_t ncb = (n + m.bs_cols - 1) / m.bs_cols;
                const float* srow = m.bscales.data() + (r / m.bs_rows) * ncb;
                for (size_t c = 0; c < n; c++) o[c] *= srow[c / m.bs_cols];
            }
        }
    }
}

void dequantize_rows(const Matrix& m, size_t r0, size_t r1, float* out) {
    if (m.format == 0)
        dequantize_rows_q4(m, r0, r1, out);
    else
        dequantize_rows_gguf(m, r0, r1, out);
}

// ---------------------------------------------------------------------------------------------
// Activation quantization for the decode kernels: src/quant.rs:240-343 (portable arm).
// ---------------------------------------------------------------------------------------------
struct QAct {
    std::vector<int8_t> q;
    std::vector<float> scales;
    std::vector<int32_t> sums;
    std::vector<float> fsums;
    std::vector<float> hsums;
    size_t t = 0, n_in = 0;
};

void quantize_act(const float* x, size_t t, size_t n_in, QAct& a) {
    size_t bpr = n_in / 32;
    a.t = t;
    a.n_in = n_in;
    a.q.assign(t * n_in, 0);
    a.scales.assign(t * bpr, 0);
    a.sums.assign(t * bpr, 0);
    a.fsums.assign(t * bpr, 0);
    a.hsums.assign(t * bpr * 2, 0);
    for (size_t ti = 0; ti < t; ti++) {
        for (size_t b = 0; b < bpr; b++) {
            const float* blk = x + ti * n_in + b * 32;
            float amax = 0.0f;
            for (int i = 0; i < 32; i++) amax = std::max(amax, std::fabs(blk[i]));
            float inv = amax > 0.0f ? 127.0f / amax : 0.0f;
            int32_t s = 0;
            for (int i = 0; i < 32; i++) {
                float v = blk[i] * inv;
                int8_t o = (int8_t)std::round(v);  // half away from zero, like f32::round
                a.q[ti * n_in + b * 32 + i] = o;
                s += o;
            }
            a.scales[ti * bpr + b] = amax / 127.0f;
            a.sums[ti * bpr + b] = s;
            float h0 = 0.0f, h1 = 0.0f, fs = 0.0f;
            for (int i = 0; i < 16; i++) h0 += blk[i];
            for (int i = 16; i < 32; i++) h1 += blk[i];
            for (int i = 0; i < 32; i++) fs += blk[i];
            a.hsums[2 * (ti * bpr + b)] = h0;
            a.hsums[2 * (ti * bpr + b) + 1] = h1;
            a.fsums[ti * bpr + b] = fs;
        }
    }
}

// ---------------------------------------------------------------------------------------------
// Decode (t <= 7) kernels: int8 activations.
// ---------------------------------------------------------------------------------------------

// src/ggml.rs:967-1091 (decode_i8), arms Q8_0 / Q4_K / Q6_K.
bool decode_i8(int kind, const uint8_t* b, int8_t* q, float* s, float* m) {
    if (kind == K_Q8_0) {
        for (int j = 0; j < 32; j++) q[j] = (int8_t)b[2 + j];
        s[0] = s[1] = f16at(b, 0);
        return false;
    }
    if (kind == K_Q4_K) {
        float d = f16at(b, 0), mn = f16at(b, 2);
        const uint8_t* qs = b + 16;
        for (int j = 0; j < 4; j++)
            for (int h = 0; h < 2; h++) {
                uint8_t sc, mm;
                scale_min_k4(2 * j + h, b + 4, &sc, &mm);
                int g = 2 * (2 * j + h);
                s[g] = d * (float)sc;
                s[g + 1] = s[g];
                float a = 8.0f * s[g];
                float c = mn * (float)mm;
                m[g] = a - c;
                m[g + 1] = m[g];
                for (int l = 0; l < 32; l++) {
                    uint8_t v = (qs[32 * j + l] >> (4 * h)) & 0xF;
                    q[64 * j + 32 * h + l] = (int8_t)((int)v - 8);
                }
            }
        return true;
    }
    // Q6_K
    float d = f16at(b, 208);
    for (int g = 0; g < 16; g++) s[g] = d * (float)(int8_t)b[192 + g];
    for (int n = 0; n < 2; n++) {
        const uint8_t* ql = b + 64 * n;
        const uint8_t* qh = b + 128 + 32 * n;
        int8_t* o = q + 128 * n;
        for (int l = 0; l < 32; l++) {
            o[l] = (int8_t)((int)((ql[l] & 0xF) | ((qh[l] & 3) << 4)) - 32);
            o[l + 32] = (int8_t)((int)((ql[l + 32] & 0xF) | (((qh[l] >> 2) & 3) << 4)) - 32);
            o[l + 64] = (int8_t)((int)((ql[l] >> 4) | (((qh[l] >> 4) & 3) << 4)) - 32);
            o[l + 96] = (int8_t)((int)((ql[l + 32] >> 4) | (((qh[l] >> 6) & 3) << 4)) - 32);
        }
    }
    return false;
}

// src/ggml.rs:1288-1315 (dot_row_generic): one row against one activation row. The reference's
// AVX2 kernel (src/kernels_ggml_x86.rs:389-417) gives the same bits
// (src/kernels_ggml_x86.rs:576-624), so this is also the AVX2 path's result.
float dot_row_gguf(int kind, const uint8_t* row, size_t n_in, const QAct& x, size_t c) {
    size_t bs = block_size(kind), ts = type_size(kind);
    int8_t q[256];
    float s[16], m[16];
    float acc = 0.0f;
    for (size_t bi = 0; bi < n_in / bs; bi++) {
        bool has_min = decode_i8(kind, row + bi * ts, q, s, m);
        size_t e0 = bi * bs;
        const int8_t* xq = x.q.data() + c * n_in + e0;
        const float* xs = x.scales.data() + c * n_in / 32 + e0 / 32;
        float sum = 0.0f;
        for (size_t g = 0; g < bs / 16; g++) {
            int isum = 0;
            for (int i = 0; i < 16; i++) isum += (int)q[16 * g + i] * (int)xq[16 * g + i];
            float a = s[g] * xs[g / 2];
            sum += a * (float)isum;
        }
        if (has_min) {
            const float* xh = x.hsums.data() + c * n_in / 16 + e0 / 16;
            for (size_t g = 0; g < bs / 16; g++) sum += m[g] * xh[g];
        }
        acc += sum;
    }
    return acc;
}

// src/kernels_x86.rs:476-519 (q4_dot_rows_tc_avx2, R = 1, TC = 1) + hsum (:96-103), then the
// affine offsets of src/kernels.rs:1284-1297 (dot of bf16 offsets with group sums; the offset dot
// is taken here in 8 lanes then summed, as the portable arm of dot_bf16 does).
float dot_row_q4(const Matrix& m, size_t r, const QAct& x, size_t c, const float* gsums) {
    size_t n_in = m.n_in, bpr = n_in / 32;
    const uint8_t* q = m.q.data() + r * n_in / 2;
    const uint16_t* s = m.scales.data() + r * bpr;
    const int8_t* xq = x.q.data() + c * n_in;
    const float* xs = x.scales.data() + c * bpr;
    const int32_t* xsums = x.sums.data() + c * bpr;
    float lanes[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    float corr = 0.0f;
    for (size_t b = 0; b < bpr; b++) {
        int w[32];
        for (int j = 0; j < 16; j++) {
            w[j] = q[b * 16 + j] & 0x0F;
            w[j + 16] = q[b * 16 + j] >> 4;
        }
        float d = f16_to_f32(s[b]);
        float sc = d * xs[b];
        // maddubs + madd: lane i holds the sum of elements 4i..4i+3
        for (int i = 0; i < 8; i++) {
            int p = 0;
            for (int e = 0; e < 4; e++) p += w[4 * i + e] * (int)xq[b * 32 + 4 * i + e];
            lanes[i] = std::fmaf((float)p, sc, lanes[i]);
        }
        corr += sc * (float)xsums[b];
    }
    // hsum: (lo + hi) -> pairs -> scalar
    float s4[4] = {lanes[0] + lanes[4], lanes[1] + lanes[5], lanes[2] + lanes[6], lanes[3] + lanes[7]};
    float s2[2] = {s4[0] + s4[2], s4[1] + s4[3]};
    float y = (s2[0] + s2[1]) - 8.0f * corr;
    if (!m.offsets.empty()) {
        size_t gpr = n_in / m.group;
        const uint16_t* o = m.offsets.data() + r * gpr;
        float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        for (size_t g = 0; g < gpr; g++) acc[g % 8] = std::fmaf(bf16_to_f32(o[g]), gsums[g], acc[g % 8]);
        float t = 0.0f;
        for (int i = 0; i < 8; i++) t += acc[i];
        y += t;
    }
    return y;
}

// ---------------------------------------------------------------------------------------------
// The same two decode kernels with the reference's AVX2 instructions (the form the reference runs on x86 and the one timed
// as its CPU baseline): src/kernels_x86.rs:476-519 (q4_dot_rows_tc_avx2: maddubs of unsigned nibbles with int8 x, madd to
// eight i32 lanes, one FMA per block into eight f32 lanes, hsum, the -8 * sum correction) and src/kernels_ggml_x86.rs:120-431
// (unpack a block to int8 in registers, maddubs / madd for the 16-element integer sums). The reference's own invariant is
// that these give the bits of the portable kernels (src/kernels_ggml_x86.rs:576-624); tests/test_oracle_pins.py holds
// these to the scalar restatements above bit for bit. The float arithmetic over a block's 16 sums stays in the portable
// kernel's order, which is what makes the bits equal.
// ---------------------------------------------------------------------------------------------
static bool g_decode_scalar = false;  // orc_set_decode_scalar: force the scalar restatements (the bit-identity tests)

static inline float hsum256(__m256 v) {  // src/kernels_x86.rs:96-103
    __m128 lo = _mm256_castps256_ps128(v), hi = _mm256_extractf128_ps(v, 1);
    __m128 t = _mm_add_ps(lo, hi);
    t = _mm_add_ps(t, _mm_movehl_ps(t, t));
    t = _mm_add_ss(t, _mm_shuffle_ps(t, t, 1));
    return _mm_cvtss_f32(t);
}

// R = 2 rows against one activation row, as q4_rows_t1 pairs them (src/kernels_x86.rs:522-536): y[0], y[1]; rows == 1 for
// the last row of an odd range.
void dot_rows_q4_avx2(const Matrix& m, size_t r, int rows, const QAct& x, size_t c, const float* gsums, float* y) {
    const size_t n_in = m.n_in, bpr = n_in / 32;
    const int8_t* xq = x.q.data() + c * n_in;
    const float* xs = x.scales.data() + c * bpr;
    const int32_t* xsums = x.sums.data() + c * bpr;
    const __m256i ones = _mm256_set1_epi16(1);
    const __m128i m0f = _mm_set1_epi8(0x0F);
    __m256 acc[2] = {_mm256_setzero_ps(), _mm256_setzero_ps()};
    float corr[2] = {0.0f, 0.0f};
    for (size_t b = 0; b < bpr; b++) {
        const __m256i xv = _mm256_loadu_si256((const __m256i*)(xq + b * 32));
        for (int i = 0; i < rows; i++) {
            const __m128i bytes = _mm_loadu_si128((const __m128i*)(m.q.data() + (r + i) * n_in / 2 + b * 16));
            const __m128i lo = _mm_and_si128(bytes, m0f), hi = _mm_and_si128(_mm_srli_epi16(bytes, 4), m0f);
            const __m256i wv = _mm256_set_m128i(hi, lo);
            const float d = f16_to_f32(m.scales[(r + i) * bpr + b]);
            const __m256i p32 = _mm256_madd_epi16(_mm256_maddubs_epi16(wv, xv), ones);
            const float sc = d * xs[b];
            acc[i] = _mm256_fmadd_ps(_mm256_cvtepi32_ps(p32), _mm256_set1_ps(sc), acc[i]);
            corr[i] += sc * (float)xsums[b];
        }
    }
    for (int i = 0; i < rows; i++) {
        float v = hsum256(acc[i]) - 8.0f * corr[i];
        if (!m.offsets.empty()) {  // src/kernels.rs:1284-1297
            const size_t gpr = n_in / m.group;
            const uint16_t* o = m.offsets.data() + (r + i) * gpr;
            float a8[8] = {0, 0, 0, 0, 0, 0, 0, 0};
            for (size_t g = 0; g < gpr; g++) a8[g % 8] = std::fmaf(bf16_to_f32(o[g]), gsums[g], a8[g % 8]);
            float t = 0.0f;
            for (int k = 0; k < 8; k++) t += a8[k];
            v += t;
        }
        y[i] = v;
    }
}

// The int8 values of one block, unpacked with 256-bit operations into q (32-byte aligned); the scales / offsets come from
// the scalar decode_i8 arithmetic (16 values per block).
static inline void unpack_q_avx2(int kind, const uint8_t* b, int8_t* q) {
    const __m256i m4 = _mm256_set1_epi8(0x0F);
    if (kind == K_Q8_0) {
        _mm256_store_si256((__m256i*)q, _mm256_loadu_si256((const __m256i*)(b + 2)));
    } else if (kind == K_Q4_K) {
        const __m256i eight = _mm256_set1_epi8(8);
        for (int j = 0; j < 4; j++) {
            const __m256i v = _mm256_loadu_si256((const __m256i*)(b + 16 + 32 * j));
            _mm256_store_si256((__m256i*)(q + 64 * j), _mm256_sub_epi8(_mm256_and_si256(v, m4), eight));
            _mm256_store_si256((__m256i*)(q + 64 * j + 32), _mm256_sub_epi8(_mm256_and_si256(_mm256_srli_epi16(v, 4), m4), eight));
        }
    } else {  // Q6_K
        const __m256i m2 = _mm256_set1_epi8(3), off = _mm256_set1_epi8(32);
        for (int n = 0; n < 2; n++) {
            const __m256i la = _mm256_loadu_si256((const __m256i*)(b + 64 * n)), lb = _mm256_loadu_si256((const __m256i*)(b + 64 * n + 32));
            const __m256i h = _mm256_loadu_si256((const __m256i*)(b + 128 + 32 * n));
            const __m256i h0 = _mm256_slli_epi16(_mm256_and_si256(h, m2), 4);
            const __m256i h1 = _mm256_slli_epi16(_mm256_and_si256(_mm256_srli_epi16(h, 2), m2), 4);
            const __m256i h2 = _mm256_slli_epi16(_mm256_and_si256(_mm256_srli_epi16(h, 4), m2), 4);
            const __m256i h3 = _mm256_slli_epi16(_mm256_and_si256(_mm256_srli_epi16(h, 6), m2), 4);
            int8_t* o = q + 128 * n;
            _mm256_store_si256((__m256i*)o, _mm256_sub_epi8(_mm256_or_si256(_mm256_and_si256(la, m4), h0), off));
            _mm256_store_si256((__m256i*)(o + 32), _mm256_sub_epi8(_mm256_or_si256(_mm256_and_si256(lb, m4), h1), off));
            _mm256_store_si256((__m256i*)(o + 64), _mm256_sub_epi8(_mm256_or_si256(_mm256_and_si256(_mm256_srli_epi16(la, 4), m4), h2), off));
            _mm256_store_si256((__m256i*)(o + 96), _mm256_sub_epi8(_mm256_or_si256(_mm256_and_si256(_mm256_srli_epi16(lb, 4), m4), h3), off));
        }
    }
}

// The block's scales (and offsets) alone: decode_i8 without its element loop.
static inline bool block_scales(int kind, const uint8_t* b, float* s, float* m) {
    if (kind == K_Q8_0) {
        s[0] = s[1] = f16at(b, 0);
        return false;
    }
    if (kind == K_Q4_K) {
        const float d = f16at(b, 0), mn = f16at(b, 2);
        for (int i = 0; i < 8; i++) {
            uint8_t sc, mm;
            scale_min_k4(i, b + 4, &sc, &mm);
            s[2 * i] = s[2 * i + 1] = d * (float)sc;
            const float a = 8.0f * s[2 * i], c = mn * (float)mm;
            m[2 * i] = m[2 * i + 1] = a - c;
        }
        return true;
    }
    const float d = f16at(b, 208);
    for (int g = 0; g < 16; g++) s[g] = d * (float)(int8_t)b[192 + g];
    return false;
}

float dot_row_gguf_avx2(int kind, const uint8_t* row, size_t n_in, const QAct& x, size_t c) {
    const size_t bs = block_size(kind), ts = type_size(kind);
    alignas(32) int8_t q[256];
    alignas(32) int32_t lanes[8];
    float s[16], m[16];
    const __m256i ones = _mm256_set1_epi16(1);
    float acc = 0.0f;
    for (size_t bi = 0; bi < n_in / bs; bi++) {
        const uint8_t* b = row + bi * ts;
        unpack_q_avx2(kind, b, q);
        const bool has_min = block_scales(kind, b, s, m);
        const size_t e0 = bi * bs;
        const int8_t* xq = x.q.data() + c * n_in + e0;
        const float* xs = x.scales.data() + c * n_in / 32 + e0 / 32;
        float sum = 0.0f;
        for (size_t g2 = 0; g2 < bs / 32; g2++) {  // two 16-element groups per 256-bit step
            const __m256i qv = _mm256_load_si256((const __m256i*)(q + 32 * g2));
            const __m256i xv = _mm256_loadu_si256((const __m256i*)(xq + 32 * g2));
            // maddubs wants an unsigned first operand: |q| times x with q's sign (|q| <= 128, |x| <= 127: no saturation)
            const __m256i p32 = _mm256_madd_epi16(_mm256_maddubs_epi16(_mm256_abs_epi8(qv), _mm256_sign_epi8(xv, qv)), ones);
            _mm256_store_si256((__m256i*)lanes, p32);
            const int i0 = lanes[0] + lanes[1] + lanes[2] + lanes[3], i1 = lanes[4] + lanes[5] + lanes[6] + lanes[7];
            const float a0 = s[2 * g2] * xs[g2];
            sum += a0 * (float)i0;
            const float a1 = s[2 * g2 + 1] * xs[g2];
            sum += a1 * (float)i1;
        }
        if (has_min) {
            const float* xh = x.hsums.data() + c * n_in / 16 + e0 / 16;
            for (size_t g = 0; g < bs / 16; g++) sum += m[g] * xh[g];
        }
        acc += sum;
    }
    return acc;
}

// ---------------------------------------------------------------------------------------------
// Prefill (t > 7, and every t for dense formats): dequantize 8 rows, then an 8 x 8 outer-product
// FMA tile with ONE accumulator per output and k in ascending order
// (src/kernels.rs:1998-2038, src/kernels_x86.rs:296-324). The value of each output is therefore
// the sequential fused multiply-add chain, whatever the vector width.
// ---------------------------------------------------------------------------------------------
void pack_xt(const float* x, size_t t, size_t n_in, std::vector<float>& xt, int threads) {  // src/kernels.rs:297-316
    size_t tiles = (t + 7) / 8;
    xt.assign(tiles * n_in * 8, 0.0f);
    parallel_for(tiles, threads, [&](size_t tile) {
        float* dst = xt.data() + tile * n_in * 8;
        for (size_t c = 0; c < 8; c++) {
            size_t tok = tile * 8 + c;
            if (tok >= t) break;
            const float* src = x + tok * n_in;
            for (size_t k = 0; k < n_in; k++) dst[k * 8 + c] = src[k];
        }
    });
}

void gemm_8x8(const float* w, size_t rows, size_t n_in, const float* xt, float* y, size_t n_out, size_t rb, size_t c0,
              size_t c_valid) {
#if ORC_AVX2
    if (rows == 8) {
        __m256 acc[8];
        for (int r = 0; r < 8; r++) acc[r] = _mm256_setzero_ps();
        for (size_t k = 0; k < n_in; k++) {
            __m256 xv = _mm256_loadu_ps(xt + k * 8);
            for (int r = 0; r < 8; r++) acc[r] = _mm256_fmadd_ps(_mm256_broadcast_ss(w + r * n_in + k), xv, acc[r]);
        }
        float tmp[8];
        for (int r = 0; r < 8; r++) {
            _mm256_storeu_ps(tmp, acc[r]);
            for (size_t c = 0; c < c_valid; c++) y[(c0 + c) * n_out + rb + r] = tmp[c];
        }
        return;
    }
#endif
    for (size_t r = 0; r < rows; r++)
        for (size_t c = 0; c < c_valid; c++) {
            float acc = 0.0f;
            for (size_t k = 0; k < n_in; k++) acc = std::fmaf(w[r * n_in + k], xt[k * 8 + c], acc);
            y[(c0 + c) * n_out + rb + r] = acc;
        }
}

void block_prefill(const Matrix& m, const float* xt, size_t t, size_t r0, size_t r1, float* y) {
    size_t n_in = m.n_in, n_out = m.n_out;
    std::vector<float> scratch(8 * n_in);
    for (size_t r = r0; r < r1;) {
        size_t rows = std::min<size_t>(r1 - r, 8);
        dequantize_rows(m, r, r + rows, scratch.data());
        size_t tiles = (t + 7) / 8;
        for (size_t tile = 0; tile < tiles; tile++) {
            size_t c0 = tile * 8;
            gemm_8x8(scratch.data(), rows, n_in, xt + tile * n_in * 8, y, n_out, r, c0, std::min<size_t>(t - c0, 8));
        }
        r += rows;
    }
}

// The driver: src/kernels.rs:1731-1879. Row blocks of about total_bytes / (8 threads), at least
// 128 KiB, in multiples of 16 rows; decode kernels up to 7 tokens (src/kernels.rs:1422), the f32
// GEMM above that and for dense formats.
void matmul_quant(const Matrix& m, const float* x, size_t t, float* y, int threads) {
    if (t == 0) return;
    size_t n_in = m.n_in, n_out = m.n_out;
    size_t total = m.bytes();
    size_t bytes_per_row = std::max<size_t>(total / n_out, 1);
    size_t target = std::max<size_t>(total / ((size_t)threads * 8), 128 * 1024);
    size_t rpb = std::max<size_t>(target / bytes_per_row, 16) / 16 * 16;
    std::vector<std::pair<size_t, size_t>> blocks;
    for (size_t r = 0; r < n_out; r += rpb) blocks.emplace_back(r, std::min(r + rpb, n_out));
    bool gemm = t > 7 || m.dense();
    if (gemm) {
        std::vector<float> xt;
        pack_xt(x, t, n_in, xt, threads);
        parallel_for(blocks.size(), threads, [&](size_t b) { block_prefill(m, xt.data(), t, blocks[b].first, blocks[b].second, y); });
        return;
    }
    QAct xa;
    quantize_act(x, t, n_in, xa);
    std::vector<float> gs;
    size_t gpr = 0;
    if (m.format == 0 && !m.offsets.empty()) {
        gpr = n_in / m.group;
        size_t k = m.group / 32, bpr = n_in / 32;
        gs.assign(t * gpr, 0.0f);
        for (size_t c = 0; c < t; c++)
            for (size_t g = 0; g < gpr; g++) {
                float s = 0.0f;
                for (size_t i = 0; i < k; i++) s += xa.fsums[c * bpr + g * k + i];
                gs[c * gpr + g] = s;
            }
    }
    size_t rb = m.format == 1 ? row_bytes(m.kind, n_in) : 0;
    const bool scalar = g_decode_scalar;
    parallel_for(blocks.size(), threads, [&](size_t b) {
        const size_t r0 = blocks[b].first, r1 = blocks[b].second;
        if (scalar) {
            for (size_t r = r0; r < r1; r++)
                for (size_t c = 0; c < t; c++)
                    y[c * n_out + r] = m.format == 0 ? dot_row_q4(m, r, xa, c, gs.empty() ? nullptr : gs.data() + c * gpr)
                                                     : dot_row_gguf(m.kind, m.data.data() + r * rb, n_in, xa, c);
            return;
        }
        if (m.format == 0) {
            for (size_t r = r0; r < r1; r += 2) {
                const int rows = r + 2 <= r1 ? 2 : 1;
                for (size_t c = 0; c < t; c++) {
                    float o[2];
                    dot_rows_q4_avx2(m, r, rows, xa, c, gs.empty() ? nullptr : gs.data() + c * gpr, o);
                    for (int i = 0; i < rows; i++) y[c * n_out + r + i] = o[i];
                }
            }
        } else {
            for (size_t r = r0; r < r1; r++)
                for (size_t c = 0; c < t; c++) y[c * n_out + r] = dot_row_gguf_avx2(m.kind, m.data.data() + r * rb, n_in, xa, c);
        }
    });
}

// src/kernels.rs:2225-2231
inline float fast_exp(float x) {
    x = std::min(std::max(x, -87.0f), 88.0f);
    float fx = std::round(x * 1.44269504088896340736f);
    float a = fx * 0.6933594f;
    float b = fx * -2.1219444e-4f;
    float r = (x - a) - b;
    float p = 1.0f + r * (1.0f + r * (0.5f + r * (0.16666667f + r * (0.041666668f + r * (0.008333334f + r * 0.0013888889f)))));
    return bits_f32((uint32_t)(((int)fx + 127) << 23)) * p;
}

}  // namespace

// =============================================================================================
// C interface (ctypes).
// =============================================================================================

ORC_API uint64_t orc_lcg(uint64_t* seed) { return lcg(seed); }
ORC_API size_t orc_block_size(int kind) { return block_size(kind); }
ORC_API size_t orc_type_size(int kind) { return type_size(kind); }
ORC_API float orc_f16_to_f32(uint16_t h) { return f16_to_f32(h); }
ORC_API uint16_t orc_f32_to_f16(float f) { return f32_to_f16(f); }
ORC_API uint16_t orc_f32_to_bf16(float f) { return f32_to_bf16(f); }
ORC_API float orc_e4m3_to_f32(uint8_t b) { return e4m3_to_f32(b); }
ORC_API float orc_fast_exp(float x) { return fast_exp(x); }

// src/ggml.rs:1525-1533: FNV-1a 64 over the little-endian bytes of each f32.
ORC_API uint64_t orc_fnv_f32(const float* v, size_t n) {
    uint64_t h = 0xcbf29ce484222325ull;
    for (size_t i = 0; i < n; i++) {
        uint32_t u = f32_bits(v[i]);
        for (int b = 0; b < 4; b++) h = (h ^ ((u >> (8 * b)) & 0xff)) * 0x100000001b3ull;
    }
    return h;
}

// src/ggml.rs:1446-1496 (random_blocks), the arms of every kind this file decodes.
ORC_API void orc_random_blocks(int kind, size_t nb, uint64_t* seed, uint8_t* v) {
    size_t ts = type_size(kind);
    for (size_t i = 0; i < nb * ts; i++) v[i] = (uint8_t)lcg(seed);
    auto rnd = [&](bool sgn) {
        uint64_t e = 117 + lcg(seed) % 6;
        uint32_t mant = (uint32_t)lcg(seed) & 0x7fffffu;
        float mag = bits_f32((uint32_t)(e << 23) | mant);
        if (sgn && (lcg(seed) & 1) == 1) return -mag;
        return mag;
    };
    auto put_f16 = [&](uint8_t* b, size_t i, float x) {
        uint16_t h = f32_to_f16(x);
        b[i] = (uint8_t)(h & 0xff);
        b[i + 1] = (uint8_t)(h >> 8);
    };
    for (size_t bi = 0; bi < nb; bi++) {
        uint8_t* b = v + bi * ts;
        switch (kind) {
            case K_F32: {
                float x = rnd(true) * 64.0f;
                std::memcpy(b, &x, 4);
                break;
            }
            case K_F16: put_f16(b, 0, rnd(true) * 64.0f); break;
            case K_BF16: {
                uint16_t h = f32_to_bf16(rnd(true) * 64.0f);
                b[0] = (uint8_t)(h & 0xff);
                b[1] = (uint8_t)(h >> 8);
                break;
            }
            case K_Q4_1:
            case K_Q5_1: {
                put_f16(b, 0, rnd(false));
                put_f16(b, 2, rnd(true) * 8.0f);
                break;
            }
            case K_Q2_K: {
                put_f16(b, 80, rnd(false));
                put_f16(b, 82, rnd(false));
                break;
            }
            case K_Q3_K: put_f16(b, 108, rnd(true)); break;
            case K_Q5_K:
            case K_Q4_K: {
                put_f16(b, 0, rnd(false));
                put_f16(b, 2, rnd(false));
                break;
            }
            case K_Q6_K: put_f16(b, 208, rnd(true)); break;
            case K_MXFP4: b[0] = (uint8_t)(118 + lcg(seed) % 7); break;
            default: put_f16(b, 0, rnd(true)); break;  // Q8_0, Q4_0, Q5_0, IQ4_NL, IQ4_XS
        }
    }
}

ORC_API void orc_dequantize_row(int kind, const uint8_t* src, float* out, size_t n) { dequantize_row(kind, src, out, n); }

// ---- matrices --------------------------------------------------------------------------------

// src/quant.rs:518-563 (from_mlx_q4): MLX (u32 words, bf16 scales, bf16 biases) -> Q4_0 layout +
// bf16 offsets `bias + 8 scale`, f16 scale copied to each 32-block of a group.
ORC_API void* orc_matrix_from_mlx_q4(const uint32_t* w, const uint16_t* scales, const uint16_t* biases, size_t n_out, size_t n_in,
                                     size_t group) {
    auto* m = new Matrix();
    m->format = 0;
    m->n_out = n_out;
    m->n_in = n_in;
    m->group = group;
    size_t gpr = n_in / group, bpr = n_in / 32;
    m->q.assign(n_out * n_in / 2, 0);
    m->scales.assign(n_out * bpr, 0);
    m->offsets.assign(n_out * gpr, 0);
    for (size_t r = 0; r < n_out; r++) {
        const uint32_t* wrow = w + r * n_in / 8;
        for (size_t g = 0; g < gpr; g++) {
            float s = bf16_to_f32(scales[r * gpr + g]);
            float b = bf16_to_f32(biases[r * gpr + g]);
            float e = 8.0f * s;
            m->offsets[r * gpr + g] = f32_to_bf16(b + e);
            uint16_t d = f32_to_f16(s);
            for (size_t blk = g * group / 32; blk < (g + 1) * group / 32; blk++) m->scales[r * bpr + blk] = d;
        }
        for (size_t blk = 0; blk < bpr; blk++) {
            const uint32_t* words = wrow + blk * 4;
            auto nib = [&](size_t e) { return (uint8_t)((words[e / 8] >> (4 * (e % 8))) & 15); };
            for (size_t j = 0; j < 16; j++) m->q[r * n_in / 2 + blk * 16 + j] = (uint8_t)(nib(j) | (nib(j + 16) << 4));
        }
    }
    return m;
}

ORC_API void* orc_matrix_gguf(int kind, const uint8_t* data, size_t n_out, size_t n_in, const float* bscales, size_t bs_rows,
                              size_t bs_cols) {
    auto* m = new Matrix();
    m->format = 1;
    m->kind = kind;
    m->n_out = n_out;
    m->n_in = n_in;
    m->data.assign(data, data + n_out * row_bytes(kind, n_in));
    if (bscales) {
        size_t ncb = (n_in + bs_cols - 1) / bs_cols, nrb = (n_out + bs_rows - 1) / bs_rows;
        m->bscales.assign(bscales, bscales + ncb * nrb);
        m->bs_rows = bs_rows;
        m->bs_cols = bs_cols;
    }
    return m;
}

ORC_API void orc_matrix_free(void* m) { delete (Matrix*)m; }
// The Q4 + offsets arrays of a matrix built by orc_matrix_from_mlx_q4, as the reference's kernels take them
// (src/quant.rs:427-440): nibbles [n_out n_in / 2], f16 scales [n_out n_in / 32], bf16 offsets [n_out n_in / group].
ORC_API int orc_matrix_q4_parts(void* mp, const uint8_t** q, size_t* q_bytes, const uint16_t** scales, size_t* n_scales, const uint16_t** offsets,
                                size_t* n_offsets, size_t* group) {
    const Matrix& m = *(Matrix*)mp;
    if (m.format != 0) return -1;
    *q = m.q.data();
    *q_bytes = m.q.size();
    *scales = m.scales.data();
    *n_scales = m.scales.size();
    *offsets = m.offsets.data();
    *n_offsets = m.offsets.size();
    *group = m.group;
    return 0;
}
ORC_API size_t orc_matrix_bytes(void* m) { return ((Matrix*)m)->bytes(); }

ORC_API void orc_matrix_dequantize_rows(void* m, size_t r0, size_t r1, float* out) { dequantize_rows(*(Matrix*)m, r0, r1, out); }

// src/quant.rs:566-578 (mlx_dequant_row, bits = 4): the exact MLX value `s * q + b`.
ORC_API void orc_mlx_dequant_row(const uint32_t* w, const uint16_t* scales, const uint16_t* biases, size_t group, float* out, size_t n) {
    for (size_t e = 0; e < n; e++) {
        size_t g = e / group;
        float s = bf16_to_f32(scales[g]), b = bf16_to_f32(biases[g]);
        uint32_t q = (w[e / 8] >> (4 * (e % 8))) & 15;
        float p = s * (float)q;
        out[e] = p + b;
    }
}

// The CPU path's own result: decode kernels for t <= 7, f32 GEMM otherwise (matmul_quant above).
// 1: the decode path (t <= 7) runs the scalar restatements; 0 (default): the AVX2 kernels. Same bits either way.
ORC_API void orc_set_decode_scalar(int on) { g_decode_scalar = on != 0; }
ORC_API void orc_matmul_cpu(void* m, const float* x, size_t t, float* y, int threads) { matmul_quant(*(Matrix*)m, x, t, y, threads); }

// The prefill (f32 GEMM) arithmetic at any t (what a GPU GEMM result is compared with).
ORC_API void orc_matmul_prefill(void* mp, const float* x, size_t t, float* y, int threads) {
    const Matrix& m = *(Matrix*)mp;
    std::vector<float> xt;
    pack_xt(x, t, m.n_in, xt, threads);
    size_t rpb = 64;
    size_t nb = (m.n_out + rpb - 1) / rpb;
    parallel_for(nb, threads, [&](size_t b) { block_prefill(m, xt.data(), t, b * rpb, std::min((b + 1) * rpb, m.n_out), y); });
}

// f64 product of the bit-exact dequantized weights with x: the definition the reference's CUDA
// tests bind to (src/cuda.rs:1594-1602, gemm_ref). y is [t][n_out] in f64.
ORC_API void orc_matmul_f64(void* mp, const float* x, size_t t, double* y, int threads) {
    const Matrix& m = *(Matrix*)mp;
    size_t rpb = 16;
    size_t nb = (m.n_out + rpb - 1) / rpb;
    parallel_for(nb, threads, [&](size_t b) {
        size_t r0 = b * rpb, r1 = std::min((b + 1) * rpb, m.n_out);
        std::vector<float> w((r1 - r0) * m.n_in);
        dequantize_rows(m, r0, r1, w.data());
        for (size_t r = r0; r < r1; r++)
            for (size_t c = 0; c < t; c++) {
                double acc = 0.0;
                const float* wr = w.data() + (r - r0) * m.n_in;
                const float* xr = x + c * m.n_in;
                for (size_t k = 0; k < m.n_in; k++) acc += (double)wr[k] * (double)xr[k];
                y[c * m.n_out + r] = acc;
            }
    });
}

ORC_API void orc_quantize_act(const float* x, size_t t, size_t n_in, int8_t* q, float* scales, int32_t* sums, float* fsums, float* hsums) {
    QAct a;
    quantize_act(x, t, n_in, a);
    std::memcpy(q, a.q.data(), a.q.size());
    std::memcpy(scales, a.scales.data(), a.scales.size() * 4);
    std::memcpy(sums, a.sums.data(), a.sums.size() * 4);
    std::memcpy(fsums, a.fsums.data(), a.fsums.size() * 4);
    std::memcpy(hsums, a.hsums.data(), a.hsums.size() * 4);
}

// ---- MoE ------------------------------------------------------------------------------------

// src/moe.rs:180-193 (route_top_k): top k by value descending (total order, ties to the lower
// index), weights = exp(l - max) / sum over the k chosen.
ORC_API void orc_route_top_k(const float* logits, size_t n, size_t k, int32_t* ids, float* w) {
    std::vector<size_t> idx(n);
    for (size_t i = 0; i < n; i++) idx[i] = i;
    auto key = [&](size_t i) {  // f32::total_cmp order as a signed integer key
        int32_t b = (int32_t)f32_bits(logits[i]);
        return b ^ (int32_t)(((uint32_t)(b >> 31)) >> 1);
    };
    std::sort(idx.begin(), idx.end(), [&](size_t a, size_t b) {
        int32_t ka = key(a), kb = key(b);
        if (ka != kb) return ka > kb;
        return a < b;
    });
    k = std::min(k, n);
    float mx = logits[idx[0]];
    std::vector<float> e(k);
    float s = 0.0f;
    for (size_t j = 0; j < k; j++) {
        e[j] = std::exp(logits[idx[j]] - mx);
        s += e[j];
    }
    for (size_t j = 0; j < k; j++) {
        ids[j] = (int32_t)idx[j];
        w[j] = e[j] / s;
    }
}

// src/moe.rs:625-828 (Experts::forward), f32 arithmetic of the grouped-prefill arm: for token i and
// each of its routes (e, w) in order: h = act(gate_e x) * (up_e x) with SiLU through fast_exp
// (src/kernels.rs:2188-2198), o = down_e h, y[i] += w * o (axpy in route order). The expert
// matrices are `gate_up[e]` ([2 inter, h]: gate rows then up rows) and `down[e]` ([h, inter]).
// `exact_products` = 1 takes every dot product in f64 over the bit-exact dequantized weights (the
// definition); 0 uses the CPU path's own kernels (decode kernels for fewer than 8 rows per call).
ORC_API void orc_moe_forward(void* const* gate_up, void* const* down, size_t n_experts, size_t h, size_t inter, const float* x,
                             size_t t, const int32_t* route_ids, const float* route_w, size_t k, float* y, int threads,
                             int exact_products) {
    // Segment tokens per expert, in token order (like src/cuda.rs:810-857).
    std::vector<std::vector<std::pair<size_t, size_t>>> seg(n_experts);  // (token, slot)
    for (size_t i = 0; i < t; i++)
        for (size_t j = 0; j < k; j++) seg[(size_t)route_ids[i * k + j]].emplace_back(i, j);
    std::vector<float> outs(t * k * h, 0.0f);  // o per (token, slot)
    parallel_for(n_experts, threads, [&](size_t e) {
        size_t n = seg[e].size();
        if (n == 0) return;
        const Matrix& gu = *(const Matrix*)gate_up[e];
        const Matrix& dn = *(const Matrix*)down[e];
        std::vector<float> xs(n * h), gv(n * 2 * inter), act(n * inter), o(n * h);
        for (size_t s = 0; s < n; s++) std::memcpy(xs.data() + s * h, x + seg[e][s].first * h, h * 4);
        if (exact_products) {
            std::vector<double> tmp(n * 2 * inter);
            orc_matmul_f64((void*)&gu, xs.data(), n, tmp.data(), 1);
            for (size_t i = 0; i < tmp.size(); i++) gv[i] = (float)tmp[i];
        } else {
            matmul_quant(gu, xs.data(), n, gv.data(), 1);
        }
        for (size_t s = 0; s < n; s++)
            for (size_t c = 0; c < inter; c++) {
                float g = gv[s * 2 * inter + c], u = gv[s * 2 * inter + inter + c];
                float sg = exact_products ? (float)((double)g / (1.0 + std::exp(-(double)g))) : g / (1.0f + fast_exp(-g));
                act[s * inter + c] = sg * u;
            }
        if (exact_products) {
            std::vector<double> tmp(n * h);
            orc_matmul_f64((void*)&dn, act.data(), n, tmp.data(), 1);
            for (size_t i = 0; i < tmp.size(); i++) o[i] = (float)tmp[i];
        } else {
            matmul_quant(dn, act.data(), n, o.data(), 1);
        }
        for (size_t s = 0; s < n; s++) std::memcpy(outs.data() + (seg[e][s].first * k + seg[e][s].second) * h, o.data() + s * h, h * 4);
    });
    for (size_t i = 0; i < t; i++)
        for (size_t j = 0; j < k; j++) {
            float w = route_w[i * k + j];
            const float* o = outs.data() + (i * k + j) * h;
            for (size_t c = 0; c < h; c++) {
                float p = w * o[c];
                y[i * h + c] += p;
            }
        }
}

// ---- FP8 activation quantizer ------------------------------------------------------------------
// The reference has no f32 -> e4m3 encoder (its FP8 matrices take f32 activations,
// src/ggml.rs:433-443). This is the definition the CUDA FP8 GEMM is checked against: per token and
// per block of `blk` consecutive K values, scale = amax / 448 (1 when amax = 0), q = RNE(x / scale)
// to e4m3fn, saturating at +-448.
ORC_API uint8_t orc_f32_to_e4m3(float f) {
    uint32_t x = f32_bits(f);
    uint8_t sign = (uint8_t)((x >> 24) & 0x80);
    float a = std::fabs(f);
    if (!(a == a)) return (uint8_t)(sign | 0x7f);
    if (a >= 448.0f) return (uint8_t)(sign | 0x7e);
    if (a < 0.0009765625f) return sign;  // < 2^-10 (half the smallest subnormal 2^-9) -> 0; tie at 2^-10 -> even = 0
    int e;
    std::frexp(a, &e);  // a = m * 2^e, m in [0.5, 1)
    int ex = e - 1;     // a in [2^ex, 2^(ex+1))
    if (ex < -6) ex = -6;
    float ulp = std::ldexp(1.0f, ex - 3);
    float qf = a / ulp;  // exact: power-of-two division
    float r = std::nearbyint(qf);  // RNE (default rounding mode)
    float v = r * ulp;
    if (v >= 448.0f) return (uint8_t)(sign | 0x7e);
    // encode v
    if (v < 0.015625f) {  // subnormal: v = m * 2^-9
        return (uint8_t)(sign | (uint8_t)(v * 512.0f));
    }
    std::frexp(v, &e);
    int be = e - 1 + 7;
    int m = (int)(v / std::ldexp(1.0f, e - 1) * 8.0f) - 8;
    return (uint8_t)(sign | (be << 3) | m);
}

ORC_API void orc_quantize_act_e4m3(const float* x, size_t t, size_t n_in, size_t blk, uint8_t* q, float* scales) {
    size_t nb = (n_in + blk - 1) / blk;
    for (size_t i = 0; i < t; i++)
        for (size_t b = 0; b < nb; b++) {
            size_t k0 = b * blk, k1 = std::min(n_in, k0 + blk);
            float amax = 0.0f;
            for (size_t k = k0; k < k1; k++) amax = std::max(amax, std::fabs(x[i * n_in + k]));
            float s = amax > 0.0f ? amax / 448.0f : 1.0f;
            scales[i * nb + b] = s;
            for (size_t k = k0; k < k1; k++) q[i * n_in + k] = orc_f32_to_e4m3(x[i * n_in + k] / s);
        }
}

// ---- simple encoders (synthetic data only; the reference has no K-quant encoder) ---------------
// Quality is irrelevant: they only have to produce valid blocks whose DECODE the parity tests pin.
ORC_API void orc_encode_q8_0(const float* w, size_t n, uint8_t* out) {
    for (size_t b = 0; b < n / 32; b++) {
        const float* v = w + b * 32;
        float amax = 0.0f;
        for (int i = 0; i < 32; i++) amax = std::max(amax, std::fabs(v[i]));
        float d = amax / 127.0f;
        uint16_t dh = f32_to_f16(d);
        float dq = f16_to_f32(dh);
        uint8_t* o = out + b * 34;
        o[0] = (uint8_t)(dh & 0xff);
        o[1] = (uint8_t)(dh >> 8);
        for (int i = 0; i < 32; i++) {
            int q = dq > 0.0f ? (int)std::lround(v[i] / dq) : 0;
            o[2 + i] = (uint8_t)(int8_t)std::min(127, std::max(-127, q));
        }
    }
}

ORC_API void orc_encode_q4_k(const float* w, size_t n, uint8_t* out) {
    for (size_t b = 0; b < n / 256; b++) {
        const float* v = w + b * 256;
        uint8_t* o = out + b * 144;
        float mins[8], scs[8];
        float max_sc = 0.0f, max_min = 0.0f;
        for (int j = 0; j < 8; j++) {
            float lo = v[32 * j], hi = v[32 * j];
            for (int l = 1; l < 32; l++) {
                lo = std::min(lo, v[32 * j + l]);
                hi = std::max(hi, v[32 * j + l]);
            }
            if (lo > 0.0f) lo = 0.0f;
            scs[j] = (hi - lo) / 15.0f;
            mins[j] = -lo;
            max_sc = std::max(max_sc, scs[j]);
            max_min = std::max(max_min, mins[j]);
        }
        uint16_t dh = f32_to_f16(max_sc / 63.0f), mh = f32_to_f16(max_min / 63.0f);
        float d = f16_to_f32(dh), dm = f16_to_f32(mh);
        o[0] = (uint8_t)(dh & 0xff);
        o[1] = (uint8_t)(dh >> 8);
        o[2] = (uint8_t)(mh & 0xff);
        o[3] = (uint8_t)(mh >> 8);
        uint8_t ls[8], lm[8];
        for (int j = 0; j < 8; j++) {
            ls[j] = (uint8_t)std::min(63, std::max(0, d > 0 ? (int)std::lround(scs[j] / d) : 0));
            lm[j] = (uint8_t)std::min(63, std::max(0, dm > 0 ? (int)std::lround(mins[j] / dm) : 0));
        }
        std::memset(o + 4, 0, 12);
        for (int j = 0; j < 8; j++) {
            if (j < 4) {
                o[4 + j] |= ls[j] & 63;
                o[4 + j + 4] |= lm[j] & 63;
            } else {
                o[4 + j + 4] = (uint8_t)((ls[j] & 0xF) | ((lm[j] & 0xF) << 4));
                o[4 + j - 4] |= (uint8_t)((ls[j] >> 4) << 6);
                o[4 + j] |= (uint8_t)((lm[j] >> 4) << 6);
            }
        }
        for (int j = 0; j < 4; j++)
            for (int l = 0; l < 32; l++) {
                uint8_t qv[2];
                for (int hh = 0; hh < 2; hh++) {
                    int g = 2 * j + hh;
                    float d1 = d * (float)ls[g], m1 = dm * (float)lm[g];
                    int q = d1 > 0.0f ? (int)std::lround((v[64 * j + 32 * hh + l] + m1) / d1) : 0;
                    qv[hh] = (uint8_t)std::min(15, std::max(0, q));
                }
                o[16 + 32 * j + l] = (uint8_t)(qv[0] | (qv[1] << 4));
            }
    }
}

ORC_API void orc_encode_q6_k(const float* w, size_t n, uint8_t* out) {
    for (size_t b = 0; b < n / 256; b++) {
        const float* v = w + b * 256;
        uint8_t* o = out + b * 210;
        float sc[16], max_s = 0.0f;
        for (int g = 0; g < 16; g++) {
            float amax = 0.0f;
            for (int l = 0; l < 16; l++) amax = std::max(amax, std::fabs(v[16 * g + l]));
            sc[g] = amax / 31.0f;
            max_s = std::max(max_s, sc[g]);
        }
        uint16_t dh = f32_to_f16(max_s / 127.0f);
        float d = f16_to_f32(dh);
        int8_t ls[16];
        for (int g = 0; g < 16; g++) ls[g] = (int8_t)std::min(127, std::max(0, d > 0 ? (int)std::lround(sc[g] / d) : 0));
        std::memset(o, 0, 192);
        for (int g = 0; g < 16; g++) o[192 + g] = (uint8_t)ls[g];
        o[208] = (uint8_t)(dh & 0xff);
        o[209] = (uint8_t)(dh >> 8);
        for (int n2 = 0; n2 < 2; n2++)
            for (int k = 0; k < 4; k++)
                for (int l = 0; l < 32; l++) {
                    int e = 128 * n2 + 32 * k + l;
                    float dd = d * (float)ls[e / 16];
                    int q = dd > 0.0f ? (int)std::lround(v[e] / dd) : 0;
                    q = std::min(31, std::max(-32, q)) + 32;
                    // element 32k + l of half n2: nibble k/2 of ql[(k%2)*32 + l], bits 2k, 2k+1 of qh[l]
                    o[64 * n2 + (k % 2) * 32 + l] |= (uint8_t)((q & 0xF) << (4 * (k / 2)));
                    o[128 + 32 * n2 + l] |= (uint8_t)(((q >> 4) & 3) << (2 * k));
                }
    }
}

// ---- one decode token of a Llama-style decoder on the CPU path --------------------------------
// The per-op arithmetic follows the reference's CPU functions; the step strings them together in the
// order of QwenModel's dense layer (src/qwen.rs:2344-2522 attention, the SiLU MLP of src/qwen.rs's
// Mlp, final norm, head) which is also the op order of the decode graph (src/qwen.rs:1477-1528).

// src/kernels.rs:2157-2164 (rmsnorm_f32w): sequential f32 sum of squares, powf(-0.5), x * r * w.
ORC_API void orc_rmsnorm_f32w(const float* x, const float* w, size_t n, float eps, float* out) {
    float ss = 0.0f;
    for (size_t i = 0; i < n; i++) ss += x[i] * x[i];
    ss = ss / (float)n + eps;
    float r = std::pow(ss, -0.5f);
    for (size_t i = 0; i < n; i++) out[i] = x[i] * r * w[i];
}

// src/kernels.rs:2277-2289 (rope_inv_freq): f64 power, rounded to f32; zeros past the rotated part.
ORC_API void orc_rope_inv_freq(size_t dim, double theta, double proportion, float* out) {
    size_t half = dim / 2, rot = (size_t)(proportion * (double)dim) / 2;
    for (size_t i = 0; i < half; i++) out[i] = i < rot ? (float)(1.0 / std::pow(theta, (double)(2 * i) / (double)dim)) : 0.0f;
}

// src/kernels.rs:2291-2306 (rope_tables) for one position: the angle is an f32 product.
ORC_API void orc_rope_table(size_t pos, const float* inv_freq, size_t half, float* cs) {
    for (size_t i = 0; i < half; i++) {
        float a = (float)pos * inv_freq[i];
        cs[i] = std::cos(a);
        cs[half + i] = std::sin(a);
    }
}

// src/kernels.rs:2310-2331 (apply_rope, apply_rope_interleaved) on the first 2 * half values of v.
ORC_API void orc_apply_rope(float* v, const float* cs, size_t half, int interleaved) {
    const float *c = cs, *s = cs + half;
    for (size_t i = 0; i < half; i++) {
        float& a = interleaved ? v[2 * i] : v[i];
        float& b = interleaved ? v[2 * i + 1] : v[half + i];
        float x1 = a, x2 = b;
        a = x1 * c[i] - x2 * s[i];
        b = x2 * c[i] + x1 * s[i];
    }
}

namespace {

// src/kernels.rs:2076-2094 (dot): 8 accumulators over whole groups of 8, summed in order, then the tail.
float dot8(const float* a, const float* b, size_t n) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    size_t chunks = n / 8;
    for (size_t i = 0; i < chunks; i++)
        for (size_t j = 0; j < 8; j++) acc[j] += a[i * 8 + j] * b[i * 8 + j];
    float s = 0.0f;
    for (size_t j = 0; j < 8; j++) s += acc[j];
    for (size_t i = chunks * 8; i < n; i++) s += a[i] * b[i];
    return s;
}

// src/kernels.rs:2333-2344 (softmax_inplace)
void softmax_inplace(float* x, size_t n) {
    float mx = -INFINITY;
    for (size_t i = 0; i < n; i++) mx = std::max(mx, x[i]);
    float sum = 0.0f;
    for (size_t i = 0; i < n; i++) {
        x[i] = fast_exp(x[i] - mx);
        sum += x[i];
    }
    float inv = 1.0f / sum;
    for (size_t i = 0; i < n; i++) x[i] *= inv;
}

}  // namespace

ORC_API void orc_softmax_inplace(float* x, size_t n) { softmax_inplace(x, n); }

// src/model.rs:2214-2309 (attention_ext, one token, causal): for each head, scores of the (already
// scaled) query against keys lo .. len - 1 of its KV head by `dot`, softmax_inplace, then the values
// accumulated by axpy in key order. kc / vc are [len][nkv][hd].
ORC_API void orc_attention(const float* q, const float* kc, const float* vc, size_t len, size_t lo, size_t nh, size_t nkv, size_t hd,
                           float* out, int threads) {
    size_t rep = nh / nkv, n = len - lo;
    parallel_for(nh, threads, [&](size_t h) {
        size_t kvh = h / rep;
        std::vector<float> sc(n);
        for (size_t j = 0; j < n; j++) sc[j] = dot8(q + h * hd, kc + ((lo + j) * nkv + kvh) * hd, hd);
        softmax_inplace(sc.data(), n);
        float* o = out + h * hd;
        for (size_t d = 0; d < hd; d++) o[d] = 0.0f;
        for (size_t j = 0; j < n; j++) {
            const float* v = vc + ((lo + j) * nkv + kvh) * hd;
            float a = sc[j];
            for (size_t d = 0; d < hd; d++) o[d] += a * v[d];
        }
    });
}

struct orc_llama_cfg {
    uint32_t n_layers, h, nh, nkv, hd, inter, vocab, interleaved;
    float eps, scale;
};

namespace {

// y = W x for one token: the CPU decode path (int8 activations), or the f64 product of the dequantized
// weights rounded to f32 (`exact`), which is what a GPU result is bounded against.
void matvec(const Matrix& m, const float* x, float* y, int exact, int threads) {
    if (!exact) {
        matmul_quant(m, x, 1, y, threads);
        return;
    }
    std::vector<double> yd(m.n_out);
    orc_matmul_f64((void*)&m, x, 1, yd.data(), threads);
    for (size_t i = 0; i < m.n_out; i++) y[i] = (float)yd[i];
}

}  // namespace

// One token at position `pos`. mats: per layer q, k, v, o, gate, up, down (7 * n_layers), then the head.
// norms: per layer ln_pre, ln_post (2 * n_layers), then the final norm. kcache / vcache:
// [n_layers][max_len][nkv][hd], rows 0 .. pos - 1 filled; row pos is written. x: the token's embedding
// (h values). Outputs: hidden (h, after the final norm) and logits (vocab), either may be null.
ORC_API void orc_llama_step(const orc_llama_cfg* c, void* const* mats, const float* const* norms, float* kcache, float* vcache,
                            size_t max_len, size_t pos, const float* x_in, const float* rope_cs, float* hidden, float* logits, int exact,
                            int threads) {
    size_t h = c->h, nh = c->nh, nkv = c->nkv, hd = c->hd, inter = c->inter, half = hd / 2;
    std::vector<float> x(x_in, x_in + h), hn(h), q(nh * hd), k(nkv * hd), v(nkv * hd), att(nh * hd), y(h), g(inter), u(inter);
    for (size_t l = 0; l < c->n_layers; l++) {
        void* const* m = mats + 7 * l;
        orc_rmsnorm_f32w(x.data(), norms[2 * l], h, c->eps, hn.data());
        matvec(*(Matrix*)m[0], hn.data(), q.data(), exact, threads);
        matvec(*(Matrix*)m[1], hn.data(), k.data(), exact, threads);
        matvec(*(Matrix*)m[2], hn.data(), v.data(), exact, threads);
        for (size_t hh = 0; hh < nh; hh++) {
            orc_apply_rope(q.data() + hh * hd, rope_cs, half, (int)c->interleaved);
            for (size_t d = 0; d < hd; d++) q[hh * hd + d] *= c->scale;
        }
        for (size_t hh = 0; hh < nkv; hh++) orc_apply_rope(k.data() + hh * hd, rope_cs, half, (int)c->interleaved);
        float* kc = kcache + l * max_len * nkv * hd;
        float* vc = vcache + l * max_len * nkv * hd;
        std::memcpy(kc + pos * nkv * hd, k.data(), nkv * hd * sizeof(float));
        std::memcpy(vc + pos * nkv * hd, v.data(), nkv * hd * sizeof(float));
        orc_attention(q.data(), kc, vc, pos + 1, 0, nh, nkv, hd, att.data(), threads);
        matvec(*(Matrix*)m[3], att.data(), y.data(), exact, threads);
        for (size_t i = 0; i < h; i++) x[i] += y[i];
        orc_rmsnorm_f32w(x.data(), norms[2 * l + 1], h, c->eps, hn.data());
        matvec(*(Matrix*)m[4], hn.data(), g.data(), exact, threads);
        matvec(*(Matrix*)m[5], hn.data(), u.data(), exact, threads);
        // src/kernels.rs:2188-2198 (silu_mul)
        for (size_t i = 0; i < inter; i++) g[i] = g[i] / (1.0f + fast_exp(-g[i])) * u[i];
        matvec(*(Matrix*)m[6], g.data(), y.data(), exact, threads);
        for (size_t i = 0; i < h; i++) x[i] += y[i];
    }
    orc_rmsnorm_f32w(x.data(), norms[2 * c->n_layers], h, c->eps, hn.data());
    if (hidden) std::memcpy(hidden, hn.data(), h * sizeof(float));
    if (logits) matvec(*(Matrix*)mats[7 * c->n_layers], hn.data(), logits, exact, threads);
}
