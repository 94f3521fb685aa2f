// Bit-exact dequantization kernels: the f32 values the reference's CPU decode produces, computed
// with explicit round-to-nearest multiplies and adds (no FMA contraction), because the reference
// never fuses `d1 * v - m1` (src/ggml.rs:769), `(q - 8) * d + m` (src/quant.rs:601) or
// `d * sc * q` (src/ggml.rs:787).
#include "dq_core.cuh"
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
    dequant8<FMT>(w, r, e0, v);
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
    for (int g = 0; g < 4; g++) {  // from_mlx_q4 (src/quant.rs:518-563): d = f16(scale), offset = bf16(bias + 8 scale)
        const float s = bf16_bits_to_f32(scales[b * 4 + g]), bias = bf16_bits_to_f32(biases[b * 4 + g]);
        ((uint16_t*)o)[g] = __half_as_ushort(__float2half_rn(s));
        ((uint16_t*)o)[4 + g] = (uint16_t)f32_to_bf16_bits(__fadd_rn(bias, __fmul_rn(8.0f, s)));
    }
    const uint32_t* words = w + b * 32;
    for (int j = 0; j < 4; j++)
        for (int l = 0; l < 32; l++) {
            int e0 = 64 * j + l, e1 = e0 + 32;
            uint32_t n0 = (words[e0 / 8] >> (4 * (e0 % 8))) & 15, n1 = (words[e1 / 8] >> (4 * (e1 % 8))) & 15;
            o[16 + 32 * j + l] = (uint8_t)(n0 | (n1 << 4));
        }
}

// The reference's Q4Matrix with offsets (src/quant.rs:427-440: q in Q4_0 order, byte j of a 32-block = element j low,
// element j + 16 high; one f16 scale per 32-block; one bf16 offset per group) -> the same blocks. The device block has one
// scale per 64-group: *mismatch is set when the two 32-blocks of a group differ in scale (a matrix from_mlx_q4 did not make).
__global__ void repack_q4a_kernel(const uint8_t* __restrict__ q, const uint16_t* __restrict__ scales, const uint16_t* __restrict__ offsets,
                                  size_t nblocks, size_t blocks_per_row, size_t group, uint8_t* __restrict__ out, int* __restrict__ mismatch) {
    size_t b = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= nblocks) return;
    uint8_t* o = out + b * 144;
    const size_t row = b / blocks_per_row, k0 = (b % blocks_per_row) * 256, gpr = blocks_per_row * 256 / group;
    for (int g = 0; g < 4; g++) {
        const uint16_t d0 = scales[b * 8 + 2 * g], d1 = scales[b * 8 + 2 * g + 1];
        if (d0 != d1) *mismatch = 1;
        ((uint16_t*)o)[g] = d0;
        ((uint16_t*)o)[4 + g] = offsets[row * gpr + (k0 + 64 * g) / group];
    }
    const uint8_t* src = q + b * 128;  // eight 32-blocks of 16 bytes
    for (int j = 0; j < 4; j++)
        for (int l = 0; l < 32; l++) {
            const uint8_t* b0 = src + (2 * j) * 16;      // elements 64 j .. 64 j + 31
            const uint8_t* b1 = src + (2 * j + 1) * 16;  // elements 64 j + 32 .. 64 j + 63
            const uint32_t n0 = l < 16 ? (b0[l] & 15u) : (b0[l - 16] >> 4), n1 = l < 16 ? (b1[l] & 15u) : (b1[l - 16] >> 4);
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

cudaError_t launch_repack_q4a(const uint8_t* q, const uint16_t* scales, const uint16_t* offsets, size_t n_out, size_t n_in, size_t group,
                              uint8_t* out, int* mismatch, cudaStream_t st) {
    size_t nb = n_out * (n_in / 256);
    repack_q4a_kernel<<<(unsigned)((nb + 127) / 128), 128, 0, st>>>(q, scales, offsets, nb, n_in / 256, group, out, mismatch);
    return cudaGetLastError();
}

cudaError_t launch_repack_q8_0(const uint8_t* raw, size_t n_out, size_t n_in, int8_t* qs, uint16_t* d, cudaStream_t st) {
    size_t nb = n_out * (n_in / 32);
    repack_q8_0_kernel<<<(unsigned)((nb + 127) / 128), 128, 0, st>>>(raw, nb, qs, d);
    return cudaGetLastError();
}

}  // namespace b2
