// Bit-exact dequantization kernels: the f32 values the reference's CPU decode produces, computed
// with explicit round-to-nearest multiplies and adds (no FMA contraction), because the reference
// never fuses `d1 * v - m1` (src/ggml.rs:769), `(q - 8) * d + m` (src/quant.rs:601) or
// `d * sc * q` (src/ggml.rs:787).
#include "kernels.h"
#include "xplanes.cuh"

namespace b2 {

namespace {

// One thread per 8 consecutive output elements of a row.
template <int FMT>
__global__ void __launch_bounds__(256) dq_kernel(WeightDev w, size_t r0, size_t nrows, float* __restrict__ out,
                                                 const int* __restrict__ row_dev) {
    pdl_launch_dependents();
    pdl_wait();
    size_t K = w.n_in;
    if (row_dev) {  // the row is named on the device (a token's embedding); out-of-range ids read row 0
        int t = *row_dev;
        r0 = (t >= 0 && (size_t)t < w.n_out) ? (size_t)t : 0;
    }
    size_t per_row = K / 8;
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= nrows * per_row) return;
    size_t r = r0 + i / per_row;
    size_t e0 = (i % per_row) * 8;
    float v[8];
    if constexpr (FMT == B2_FMT_MLX4) {
        // dequantize_rows_q4 over from_mlx_q4's repack (src/quant.rs:518-563, 586-606):
        // d = f16(scale), offset = bf16(bias + 8 scale), value = (nib - 8) * d + offset.
        // Device blocks (repack_mlx4_kernel): 4 bf16 scales, 4 bf16 biases, 128 nibble bytes in Q4_K order.
        const uint8_t* blk = w.p0 + (r * (K / 256) + e0 / 256) * 144;
        int e = (int)(e0 % 256), j = e / 64, h = (e % 64) / 32, l = e % 32;
        float s = bf16_bits_to_f32(((const uint16_t*)blk)[j]);
        float b = bf16_bits_to_f32(((const uint16_t*)blk)[4 + j]);
        float d = __half2float(__float2half_rn(s));
        float off = bf16_bits_to_f32(f32_to_bf16_bits(__fadd_rn(b, __fmul_rn(8.0f, s))));
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
    float4* o = (float4*)(out + (i / per_row) * K + e0);
    o[0] = make_float4(v[0], v[1], v[2], v[3]);
    o[1] = make_float4(v[4], v[5], v[6], v[7]);
}

__global__ void repack_q6k_kernel(const uint8_t* __restrict__ raw, size_t nblocks, size_t /*bpr*/, uint8_t* ql, uint8_t* qh, int8_t* sc,
                                  uint16_t* d) {
    size_t b = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= nblocks) return;
    // Blocks are consecutive in both layouts (rows are whole numbers of blocks), so block b of the
    // raw stream is block b of every plane.
    const uint8_t* s = raw + b * 210;
    for (int i = 0; i < 128; i++) ql[b * 128 + i] = s[i];
    for (int i = 0; i < 64; i++) qh[b * 64 + i] = s[128 + i];
    for (int i = 0; i < 16; i++) sc[b * 16 + i] = (int8_t)s[192 + i];
    d[b] = (uint16_t)(s[208] | (s[209] << 8));
}

// MLX triple (u32 words of eight nibbles, bf16 scale and bias per 64) -> Q4_K-shaped blocks of 256 weights.
__global__ void repack_mlx4_kernel(const uint32_t* __restrict__ w, const uint16_t* __restrict__ scales, const uint16_t* __restrict__ biases,
                                   size_t nblocks, uint8_t* __restrict__ out) {
    size_t b = (size_t)blockIdx.x * blockDim.x + threadIdx.x;  // block b = 256 consecutive weights of the row-major matrix
    if (b >= nblocks) return;
    uint8_t* o = out + b * 144;
    for (int g = 0; g < 4; g++) {
        ((uint16_t*)o)[g] = scales[b * 4 + g];
        ((uint16_t*)o)[4 + g] = biases[b * 4 + g];
    }
    const uint32_t* words = w + b * 32;
    for (int j = 0; j < 4; j++)
        for (int l = 0; l < 32; l++) {
            int e0 = 64 * j + l, e1 = e0 + 32;
            uint32_t n0 = (words[e0 / 8] >> (4 * (e0 % 8))) & 15, n1 = (words[e1 / 8] >> (4 * (e1 % 8))) & 15;
            o[16 + 32 * j + l] = (uint8_t)(n0 | (n1 << 4));
        }
}

__global__ void repack_q8_0_kernel(const uint8_t* __restrict__ raw, size_t nblocks, int8_t* qs, uint16_t* d) {
    size_t b = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= nblocks) return;
    const uint8_t* s = raw + b * 34;
    d[b] = (uint16_t)(s[0] | (s[1] << 8));
    for (int i = 0; i < 32; i++) qs[b * 32 + i] = (int8_t)s[2 + i];
}

}  // namespace

cudaError_t launch_dequantize(const WeightDev& w, size_t r0, size_t nrows, float* out, cudaStream_t st, const int* row_dev, bool pdl) {
    if (nrows == 0) return cudaSuccess;
    size_t n = nrows * (w.n_in / 8);
    unsigned grid = (unsigned)((n + 255) / 256);
    switch (w.fmt) {
        case B2_FMT_MLX4: return launch_k(dq_kernel<B2_FMT_MLX4>, dim3(grid), dim3(256), 0, st, pdl, w, r0, nrows, out, row_dev);
        case B2_FMT_Q4_K: return launch_k(dq_kernel<B2_FMT_Q4_K>, dim3(grid), dim3(256), 0, st, pdl, w, r0, nrows, out, row_dev);
        case B2_FMT_Q6_K: return launch_k(dq_kernel<B2_FMT_Q6_K>, dim3(grid), dim3(256), 0, st, pdl, w, r0, nrows, out, row_dev);
        case B2_FMT_Q8_0: return launch_k(dq_kernel<B2_FMT_Q8_0>, dim3(grid), dim3(256), 0, st, pdl, w, r0, nrows, out, row_dev);
        case B2_FMT_F8E4M3: return launch_k(dq_kernel<B2_FMT_F8E4M3>, dim3(grid), dim3(256), 0, st, pdl, w, r0, nrows, out, row_dev);
        default: return cudaErrorInvalidValue;
    }
    return cudaGetLastError();
}

cudaError_t launch_repack_q6k(const uint8_t* raw, size_t n_out, size_t n_in, uint8_t* ql, uint8_t* qh, int8_t* sc, uint16_t* d,
                              cudaStream_t st) {
    size_t nb = n_out * (n_in / 256);
    repack_q6k_kernel<<<(unsigned)((nb + 127) / 128), 128, 0, st>>>(raw, nb, n_in / 256, ql, qh, sc, d);
    return cudaGetLastError();
}

cudaError_t launch_repack_mlx4(const uint32_t* w, const uint16_t* scales, const uint16_t* biases, size_t n_out, size_t n_in, uint8_t* out,
                               cudaStream_t st) {
    size_t nb = n_out * (n_in / 256);
    repack_mlx4_kernel<<<(unsigned)((nb + 127) / 128), 128, 0, st>>>(w, scales, biases, nb, out);
    return cudaGetLastError();
}

cudaError_t launch_repack_q8_0(const uint8_t* raw, size_t n_out, size_t n_in, int8_t* qs, uint16_t* d, cudaStream_t st) {
    size_t nb = n_out * (n_in / 32);
    repack_q8_0_kernel<<<(unsigned)((nb + 127) / 128), 128, 0, st>>>(raw, nb, qs, d);
    return cudaGetLastError();
}

}  // namespace b2
