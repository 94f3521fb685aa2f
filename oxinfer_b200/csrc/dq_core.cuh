// Bit-exact decode of eight consecutive weights of a row, per device format: the arithmetic of the reference's
// dequantize functions with explicit round-to-nearest multiplies and adds (see dq.cu). Shared by the
// dequantization kernels and the decode plan's embedding lookup.
#pragma once
#include "kernels.h"

namespace b2 {

// v[0..8) = weights e0 .. e0 + 7 (e0 a multiple of 8) of row r.
template <int FMT>
__device__ __forceinline__ void dequant8(const WeightDev& w, size_t r, size_t e0, float (&v)[8]) {
    const size_t K = w.n_in;
    if constexpr (FMT == B2_FMT_MLX4) {
        // dequantize_rows_q4 over from_mlx_q4's repack (src/quant.rs:518-563, 586-606):
        // d = f16(scale), offset = bf16(bias + 8 scale), value = (nib - 8) * d + offset.
        // Device blocks (repack_mlx4_kernel / repack_q4a_kernel): the four f16 d and the four bf16 offsets of the block's
        // 64-groups (the fields of the reference's Q4Matrix), then 128 nibble bytes in Q4_K order.
        const uint8_t* blk = w.p0 + (r * (K / 256) + e0 / 256) * 144;
        int e = (int)(e0 % 256), j = e / 64, h = (e % 64) / 32, l = e % 32;
        float d = f16_bits_to_f32(((const uint16_t*)blk)[j]);
        float off = bf16_bits_to_f32(((const uint16_t*)blk)[4 + j]);
        const uint8_t* q = blk + 16 + 32 * j + l;
#pragma unroll
        for (int k = 0; k < 8; k++) v[k] = __fadd_rn(__fmul_rn((float)((int)((q[k] >> (4 * h)) & 0xF) - 8), d), off);
    } else if constexpr (FMT == B2_FMT_Q4_K) {
        const uint8_t* blk = w.p0 + (r * (K / 256) + e0 / 256) * 144;
        uint32_t hdr = *(const uint32_t*)blk;
        float d = f16_bits_to_f32((uint16_t)(hdr & 0xffff)), dmin = f16_bits_to_f32((uint16_t)(hdr >> 16));
        const uint32_t* sw = (const uint32_t*)(blk + 4);
        int e = (int)(e0 % 256), j = e / 64, h = (e % 64) / 32, l = e % 32;
        uint32_t sc, mn;
        q4k_scale_min(2 * j + h, sw[0], sw[1], sw[2], sc, mn);
        float d1 = __fmul_rn(d, (float)sc), m1 = __fmul_rn(dmin, (float)mn);
        const uint8_t* q = blk + 16 + 32 * j + l;
#pragma unroll
        for (int k = 0; k < 8; k++) v[k] = __fsub_rn(__fmul_rn(d1, (float)((q[k] >> (4 * h)) & 0xF)), m1);
    } else if constexpr (FMT == B2_FMT_Q6_K) {
        size_t blk = e0 / 256;
        int e = (int)(e0 % 256), n = e / 128, k4 = (e % 128) / 32, l = e % 32;
        const uint8_t* ql = w.p0 + r * (K / 2) + blk * 128 + 64 * n + (k4 & 1) * 32 + l;
        const uint8_t* qh = w.p1 + r * (K / 4) + blk * 64 + 32 * n + l;
        const int8_t* sc = (const int8_t*)w.p2 + r * (K / 16) + blk * 16 + 8 * n + 2 * k4;
        float d = f16_bits_to_f32(((const uint16_t*)w.p3)[r * (K / 256) + blk]);
#pragma unroll
        for (int k = 0; k < 8; k++) {
            int nib = (k4 & 2) ? (ql[k] >> 4) : (ql[k] & 0xF);
            int hb = (qh[k] >> (2 * k4)) & 3;
            int q = (nib | (hb << 4)) - 32;
            float a = __fmul_rn(d, (float)sc[(l + k) / 16]);
            v[k] = __fmul_rn(a, (float)q);
        }
    } else if constexpr (FMT == B2_FMT_Q8_0) {
        const int8_t* q = (const int8_t*)w.p0 + r * K + e0;
        float d = f16_bits_to_f32(((const uint16_t*)w.p1)[r * (K / 32) + e0 / 32]);
#pragma unroll
        for (int k = 0; k < 8; k++) v[k] = __fmul_rn((float)q[k], d);
    } else {  // F8E4M3: e4m3 * block scale (src/ggml.rs:273-293, 433-443)
        const uint8_t* q = w.p0 + r * K + e0;
        float s = 1.0f;
        if (w.p1) s = ((const float*)w.p1)[((w.bs_row0 + r) / w.bs_rows) * w.bs_ncb + e0 / w.bs_cols];
#pragma unroll
        for (int k = 0; k < 8; k++) {
            // the scale may change inside the run only if bs_cols is not a multiple of 8
            float sk = (w.p1 && (w.bs_cols & 7)) ? ((const float*)w.p1)[((w.bs_row0 + r) / w.bs_rows) * w.bs_ncb + (e0 + k) / w.bs_cols] : s;
            v[k] = __fmul_rn(e4m3_to_f32(q[k]), sk);
        }
    }
}

}  // namespace b2
