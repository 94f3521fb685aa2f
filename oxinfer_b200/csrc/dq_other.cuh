// The other GGUF block formats (the legacy 32-blocks Q4_0 / Q4_1 / Q5_0 / Q5_1, the K-quants Q2_K / Q3_K / Q5_K, the
// non-linear IQ4_NL / IQ4_XS and the microscaling MXFP4): bit-exact decode of 32 consecutive weights, the arithmetic of the
// matching arms of the reference's dequantize_row (src/ggml.rs:665-706, 713-773, 915-960) with explicit round-to-nearest
// multiplies and adds. These formats stay in their raw GGUF layout on the device (blocks of 17 .. 176 bytes, only
// byte-aligned in general), are read with byte loads, and run through one generic dequantize-and-multiply matrix-vector
// kernel (gemv_other.cu): every format has a device path, none of them is tuned.
#pragma once
#include "formats.cuh"

namespace b2 {

// The format ids (B2_FMT_Q4_0 ...) are GgmlType's (src/ggml.rs:42-93), defined in the public header.
__host__ __device__ inline bool fmt_is_other(int fmt) {
    switch (fmt) {
        case B2_FMT_Q4_0: case B2_FMT_Q4_1: case B2_FMT_Q5_0: case B2_FMT_Q5_1: case B2_FMT_Q2_K: case B2_FMT_Q3_K: case B2_FMT_Q5_K:
        case B2_FMT_IQ4_NL: case B2_FMT_IQ4_XS: case B2_FMT_MXFP4: case B2_FMT_NVFP4: return true;
        default: return false;
    }
}
__host__ __device__ inline int other_block_size(int fmt) {  // src/ggml.rs:173-185
    return (fmt == B2_FMT_Q2_K || fmt == B2_FMT_Q3_K || fmt == B2_FMT_Q5_K || fmt == B2_FMT_IQ4_XS) ? 256 : fmt == B2_FMT_NVFP4 ? 64 : 32;
}
__host__ __device__ inline int other_type_size(int fmt) {  // src/ggml.rs:187-215
    switch (fmt) {
        case B2_FMT_Q4_0: return 18;
        case B2_FMT_Q4_1: return 20;
        case B2_FMT_Q5_0: return 22;
        case B2_FMT_Q5_1: return 24;
        case B2_FMT_Q2_K: return 84;
        case B2_FMT_Q3_K: return 110;
        case B2_FMT_Q5_K: return 176;
        case B2_FMT_IQ4_NL: return 18;
        case B2_FMT_IQ4_XS: return 136;
        case B2_FMT_MXFP4: return 17;
        case B2_FMT_NVFP4: return 36;
        default: return 0;
    }
}
__host__ __device__ inline size_t other_row_bytes(int fmt, size_t n_in) { return n_in / other_block_size(fmt) * other_type_size(fmt); }

// ggml's non-linear 4-bit code book (kvalues_iq4nl) and the doubled E2M1 values of MXFP4 (kvalues_mxfp4).
static __constant__ int8_t K_IQ4NL[16] = {-127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113};
static __constant__ int8_t K_MXFP4[16] = {0, 1, 2, 3, 4, 6, 8, 12, 0, -1, -2, -3, -4, -6, -8, -12};
// The kernels copy the code book of their format into 16 floats of shared memory (lanes index it differently, which a
// constant-memory table would serialize; 16 words sit in 16 banks): lut_fill by the first 16 threads, then a barrier.
template <int FMT>
__device__ __forceinline__ void lut_fill(float* lut, int tid) {
    if (tid < 16) lut[tid] = (FMT == B2_FMT_MXFP4 || FMT == B2_FMT_NVFP4) ? (float)K_MXFP4[tid] : (float)K_IQ4NL[tid];
}
// A small non-negative integer as a float through the mantissa of 2^23 (exact; keeps the conversion unit out of the loop).
__device__ __forceinline__ float uint_to_f32(uint32_t n) { return __uint_as_float(0x4B000000u | n) - 8388608.0f; }
__device__ __forceinline__ float f16_at(const uint8_t* b, int i) { return f16_bits_to_f32((uint16_t)(b[i] | (b[i + 1] << 8))); }
__device__ __forceinline__ uint32_t u32_at(const uint8_t* b, int i) { return b[i] | (b[i + 1] << 8) | (b[i + 2] << 16) | ((uint32_t)b[i + 3] << 24); }
// Half the value of an E8M0 scale byte, 2^(e - 128) (src/ggml.rs:466-474).
__device__ __forceinline__ float e8m0_half(uint32_t e) { return __uint_as_float(e < 2 ? (0x00200000u << e) : ((e - 1) << 23)); }

// Half the value of an unsigned E4M3 scale byte (src/ggml.rs:477-491): 0 and 0x7f give 0; every product below is exact.
__device__ __forceinline__ float ue4m3_half(uint32_t x) {
    if (x == 0 || x == 0x7F) return 0.0f;
    const uint32_t e = (x >> 3) & 0xF;
    const float m = (float)(x & 7);
    const float raw = e == 0 ? m * 0.001953125f : (1.0f + m * 0.125f) * __uint_as_float((e + 120u) << 23);  // 2^-9; 2^(e - 7)
    return raw * 0.5f;
}

// v[0..32) = weights 32 sub .. 32 sub + 31 of the block at `b`.
template <int FMT>
__device__ __forceinline__ void dequant32_other(const uint8_t* b, int sub, float (&v)[32], const float* lut) {
    if constexpr (FMT == B2_FMT_Q4_0) {
        const float d = f16_at(b, 0);
#pragma unroll
        for (int j = 0; j < 16; j++) {
            v[j] = __fmul_rn((uint_to_f32(b[2 + j] & 0xF) - 8.0f), d);
            v[j + 16] = __fmul_rn((uint_to_f32(b[2 + j] >> 4) - 8.0f), d);
        }
    } else if constexpr (FMT == B2_FMT_Q4_1) {
        const float d = f16_at(b, 0), m = f16_at(b, 2);
#pragma unroll
        for (int j = 0; j < 16; j++) {
            v[j] = __fadd_rn(__fmul_rn(uint_to_f32(b[4 + j] & 0xF), d), m);
            v[j + 16] = __fadd_rn(__fmul_rn(uint_to_f32(b[4 + j] >> 4), d), m);
        }
    } else if constexpr (FMT == B2_FMT_Q5_0 || FMT == B2_FMT_Q5_1) {
        constexpr bool ONE = FMT == B2_FMT_Q5_1;
        const float d = f16_at(b, 0), m = ONE ? f16_at(b, 2) : 0.0f;
        const uint32_t qh = u32_at(b, ONE ? 4 : 2);
        const uint8_t* q = b + (ONE ? 8 : 6);
#pragma unroll
        for (int j = 0; j < 16; j++) {
            const uint32_t h0 = ((qh >> j) << 4) & 0x10, h1 = (qh >> (j + 12)) & 0x10;
            const uint32_t lo = (q[j] & 0xF) | h0, hi = (q[j] >> 4) | h1;
            if (ONE) {
                v[j] = __fadd_rn(__fmul_rn(uint_to_f32(lo), d), m);
                v[j + 16] = __fadd_rn(__fmul_rn(uint_to_f32(hi), d), m);
            } else {
                v[j] = __fmul_rn((uint_to_f32(lo) - 16.0f), d);
                v[j + 16] = __fmul_rn((uint_to_f32(hi) - 16.0f), d);
            }
        }
    } else if constexpr (FMT == B2_FMT_IQ4_NL) {
        const float d = f16_at(b, 0);
#pragma unroll
        for (int j = 0; j < 16; j++) {
            v[j] = __fmul_rn(d, lut[b[2 + j] & 0xF]);
            v[j + 16] = __fmul_rn(d, lut[b[2 + j] >> 4]);
        }
    } else if constexpr (FMT == B2_FMT_MXFP4) {
        const float d = e8m0_half(b[0]);
#pragma unroll
        for (int j = 0; j < 16; j++) {
            v[j] = __fmul_rn(d, lut[b[1 + j] & 0xF]);
            v[j + 16] = __fmul_rn(d, lut[b[1 + j] >> 4]);
        }
    } else if constexpr (FMT == B2_FMT_NVFP4) {
        // four scale bytes, then per 16-value sub-block 8 bytes holding elements j (low nibble) and j + 8 (high); chunk `sub`
        // covers sub-blocks 2 sub and 2 sub + 1 (src/ggml.rs:936-947)
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const int s = 2 * sub + h;
            const float d = ue4m3_half(b[s]);
            const uint8_t* q = b + 4 + 8 * s;
#pragma unroll
            for (int j = 0; j < 8; j++) {
                v[16 * h + j] = __fmul_rn(d, lut[q[j] & 0xF]);
                v[16 * h + j + 8] = __fmul_rn(d, lut[q[j] >> 4]);
            }
        }
    } else if constexpr (FMT == B2_FMT_Q2_K) {
        // scales b[0..16), quants b[16..80), d @80, min @82; chunk sub = 4 n + j covers h = 0, 1 (src/ggml.rs:713-730)
        const float d = f16_at(b, 80), mn = f16_at(b, 82);
        const int n = sub >> 2, j = sub & 3;
        const uint8_t* q = b + 16 + 32 * n;
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const uint32_t s = b[8 * n + 2 * j + h];
            const float dl = __fmul_rn(d, (float)(s & 0xF)), ml = __fmul_rn(mn, (float)(s >> 4));
#pragma unroll
            for (int l = 0; l < 16; l++) v[16 * h + l] = __fsub_rn(__fmul_rn(dl, uint_to_f32((q[16 * h + l] >> (2 * j)) & 3)), ml);
        }
    } else if constexpr (FMT == B2_FMT_Q3_K) {
        // high-bit mask b[0..32), quants b[32..96), 12 scale bytes @96, d @108 (src/ggml.rs:731-749, q3k_scales :513-531)
        const float d = f16_at(b, 108);
        const int n = sub >> 2, j = sub & 3;
        const uint8_t* q = b + 32 + 32 * n;
        const uint32_t a0 = u32_at(b, 96), a1 = u32_at(b, 100), tmp = u32_at(b, 104);
        const uint32_t aux[4] = {(a0 & 0x0f0f0f0fu) | ((tmp & 0x03030303u) << 4), (a1 & 0x0f0f0f0fu) | (((tmp >> 2) & 0x03030303u) << 4),
                                 ((a0 >> 4) & 0x0f0f0f0fu) | (((tmp >> 4) & 0x03030303u) << 4), ((a1 >> 4) & 0x0f0f0f0fu) | (((tmp >> 6) & 0x03030303u) << 4)};
        const uint32_t m = 1u << (4 * n + j);
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const int si = 8 * n + 2 * j + h;
            const int sc = (int)(int8_t)((aux[si >> 2] >> (8 * (si & 3))) & 0xff);
            const float dl = __fmul_rn(d, (float)(sc - 32));
#pragma unroll
            for (int l = 0; l < 16; l++) {
                const int i = 16 * h + l;
                const float val = uint_to_f32((q[i] >> (2 * j)) & 3) - ((b[i] & m) ? 0.0f : 4.0f);
                v[16 * h + l] = __fmul_rn(dl, val);
            }
        }
    } else if constexpr (FMT == B2_FMT_Q5_K) {
        // d @0, min @2, 12 scale bytes @4, high bits b[16..48), quants b[48..176); chunk sub = 2 j + h (src/ggml.rs:750-773)
        const float d = f16_at(b, 0), mn = f16_at(b, 2);
        const int j = sub >> 1, h = sub & 1;
        uint32_t sc, mm;
        q4k_scale_min(sub, u32_at(b, 4), u32_at(b, 8), u32_at(b, 12), sc, mm);
        const float d1 = __fmul_rn(d, (float)sc), m1 = __fmul_rn(mn, (float)mm);
        const uint8_t* q = b + 48 + 32 * j;
        const uint8_t* qh = b + 16;
#pragma unroll
        for (int l = 0; l < 32; l++) {
            uint32_t val = (q[l] >> (4 * h)) & 0xF;
            if (qh[l] & (1u << sub)) val += 16;
            v[l] = __fsub_rn(__fmul_rn(d1, uint_to_f32(val)), m1);
        }
    } else {  // IQ4_XS: d @0, high scale bits u16 @2, low scale nibbles b[4..8), quants @8 + 16 ib (src/ggml.rs:948-958, :544-547)
        const float d = f16_at(b, 0);
        const uint32_t sh = b[2] | (b[3] << 8);
        const int ls = (int)(((b[4 + sub / 2] >> (4 * (sub % 2))) & 0xF) | (((sh >> (2 * sub)) & 3) << 4)) - 32;
        const float dl = __fmul_rn(d, (float)ls);
        const uint8_t* q = b + 8 + 16 * sub;
#pragma unroll
        for (int j = 0; j < 16; j++) {
            v[j] = __fmul_rn(dl, lut[q[j] & 0xF]);
            v[j + 16] = __fmul_rn(dl, lut[q[j] >> 4]);
        }
    }
}

// The dispatch over the formats: evaluates `expr`, in which FMT is the compile-time format, for the run-time format `fmt`.
#define B2_OTHER_CASE(F, expr) \
    case F: {                  \
        constexpr int FMT = F; \
        return (expr);         \
    }
#define B2_OTHER_SWITCH(fmt, expr)            \
    switch (fmt) {                            \
        B2_OTHER_CASE(B2_FMT_Q4_0, expr)      \
        B2_OTHER_CASE(B2_FMT_Q4_1, expr)      \
        B2_OTHER_CASE(B2_FMT_Q5_0, expr)      \
        B2_OTHER_CASE(B2_FMT_Q5_1, expr)      \
        B2_OTHER_CASE(B2_FMT_Q2_K, expr)      \
        B2_OTHER_CASE(B2_FMT_Q3_K, expr)      \
        B2_OTHER_CASE(B2_FMT_Q5_K, expr)      \
        B2_OTHER_CASE(B2_FMT_IQ4_NL, expr)    \
        B2_OTHER_CASE(B2_FMT_IQ4_XS, expr)    \
        B2_OTHER_CASE(B2_FMT_MXFP4, expr)     \
        B2_OTHER_CASE(B2_FMT_NVFP4, expr)     \
        default: return cudaErrorInvalidValue; \
    }

}  // namespace b2
