// The other GGUF block formats on the device (dq_other.cuh): bit-exact dequantization, and one generic matrix-vector
// kernel that decodes 32 weights at a time in registers and multiplies them with the f32 activations (no integer planes,
// no repack: the rows stay as they are in the GGUF file). It takes the five output modes of dmv_out
// (src/cuda_decode.cu:131-137), the SiLU / GELU pair, and up to four tokens per launch with the weights read once (each
// token's row equals its one-token row bit for bit). The reference declines every GGUF type on its CUDA backend
// (src/cuda.rs:642); these formats get a correct device path here, not a tuned one: a lane decodes whole 32-weight chunks
// with byte loads, which costs four to six instructions per weight.
#include "dq_other.cuh"
#include "gemv_core.cuh"

namespace b2 {

using namespace gemv_core;

namespace {

// One thread per 32 consecutive output elements of a row.
template <int FMT>
__global__ void __launch_bounds__(128) dq_other_kernel(WeightDev w, size_t r0, size_t nrows, float* __restrict__ out, const int* __restrict__ row_dev) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t K = w.n_in, per_row = K / 32;
    if (row_dev) {
        const int t = *row_dev;
        r0 = (t >= 0 && (size_t)t < w.n_out) ? (size_t)t : 0;
    }
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= nrows * per_row) return;
    const size_t r = r0 + i / per_row, c = i % per_row;
    constexpr int BS = (FMT == B2_FMT_Q2_K || FMT == B2_FMT_Q3_K || FMT == B2_FMT_Q5_K || FMT == B2_FMT_IQ4_XS) ? 256 : 32;
    const uint8_t* blk = w.p0 + r * other_row_bytes(FMT, K) + (c * 32 / BS) * other_type_size(FMT);
    float v[32];
    dequant32_other<FMT>(blk, (int)(c % (BS / 32)), v);
    float4* o = (float4*)(out + (i / per_row) * K + c * 32);
#pragma unroll
    for (int k = 0; k < 8; k++) o[k] = make_float4(v[4 * k], v[4 * k + 1], v[4 * k + 2], v[4 * k + 3]);
}

constexpr int OW = 8;  // warps per CTA, one weight row per warp at a time

template <int FMT, bool PAIR, int NT>
__global__ void __launch_bounds__(OW * 32) gemv_other_kernel(WeightDev w, WeightDev w2, const float* __restrict__ x, size_t x_stride, float* __restrict__ y,
                                                            size_t y_stride, int mode, const float* __restrict__ gate) {
    pdl_launch_dependents();
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const size_t K = w.n_in, chunks = K / 32, rb = other_row_bytes(FMT, K);
    constexpr int BS = (FMT == B2_FMT_Q2_K || FMT == B2_FMT_Q3_K || FMT == B2_FMT_Q5_K || FMT == B2_FMT_IQ4_XS) ? 256 : 32;
    constexpr int TS = FMT == B2_FMT_Q4_0 ? 18 : FMT == B2_FMT_Q4_1 ? 20 : FMT == B2_FMT_Q5_0 ? 22 : FMT == B2_FMT_Q5_1 ? 24 : FMT == B2_FMT_Q2_K ? 84
                       : FMT == B2_FMT_Q3_K ? 110 : FMT == B2_FMT_Q5_K ? 176 : FMT == B2_FMT_IQ4_NL ? 18 : FMT == B2_FMT_IQ4_XS ? 136 : 17;
    for (size_t r = (size_t)blockIdx.x * OW + warp; r < w.n_out; r += (size_t)gridDim.x * OW) {
        float acc[PAIR ? 2 : 1][NT];
#pragma unroll
        for (int m = 0; m < (PAIR ? 2 : 1); m++)
#pragma unroll
            for (int tk = 0; tk < NT; tk++) acc[m][tk] = 0.0f;
        for (size_t c = lane; c < chunks; c += 32) {
#pragma unroll
            for (int m = 0; m < (PAIR ? 2 : 1); m++) {
                const uint8_t* blk = (m ? w2.p0 : w.p0) + r * rb + (c * 32 / BS) * TS;
                float v[32];
                dequant32_other<FMT>(blk, (int)(c % (BS / 32)), v);
#pragma unroll
                for (int tk = 0; tk < NT; tk++) {
                    const float4* xv = (const float4*)(x + (size_t)tk * x_stride + c * 32);
                    float a = acc[m][tk];
#pragma unroll
                    for (int k = 0; k < 8; k++) {
                        const float4 q = __ldg(xv + k);
                        a = fmaf(v[4 * k], q.x, a);
                        a = fmaf(v[4 * k + 1], q.y, a);
                        a = fmaf(v[4 * k + 2], q.z, a);
                        a = fmaf(v[4 * k + 3], q.w, a);
                    }
                    acc[m][tk] = a;
                }
            }
        }
#pragma unroll
        for (int tk = 0; tk < NT; tk++) {
            const float a = warp_sum(acc[0][tk]), b = PAIR ? warp_sum(acc[PAIR ? 1 : 0][tk]) : 0.0f;
            if (lane == 0) {
                float* o = y + (size_t)tk * y_stride + r;
                if (PAIR)
                    *o = (mode == B2_MODE_SILU_PAIR ? silu(a) : gelu_tanh(a)) * b;
                else if (mode == B2_MODE_STORE)
                    *o = a;
                else if (mode == B2_MODE_ADD)
                    *o += a;
                else
                    *o += a * (1.0f / (1.0f + __expf(-gate[0])));
            }
        }
    }
}

template <int FMT, int NT>
cudaError_t launch_other_nt(const WeightDev& w, const WeightDev* up, const float* x, size_t x_stride, float* y, size_t y_stride, int mode,
                            const float* gate, int sm_count, cudaStream_t st, bool pdl) {
    const bool pair = mode == B2_MODE_SILU_PAIR || mode == B2_MODE_GELU_PAIR;
    auto kern = pair ? gemv_other_kernel<FMT, true, NT> : gemv_other_kernel<FMT, false, NT>;
    const size_t groups = (w.n_out + OW - 1) / OW, cap = (size_t)sm_count * 6;
    return launch_k(kern, dim3((unsigned)(groups < cap ? groups : cap)), dim3(OW * 32), 0, st, pdl, w, pair ? *up : w, x, x_stride, y, y_stride, mode, gate);
}

}  // namespace

bool gemv_other_supports(const WeightDev& w) { return fmt_is_other(w.fmt) && w.n_in > 0 && w.n_in % other_block_size(w.fmt) == 0 && w.n_in % 32 == 0; }

cudaError_t launch_dequantize_other(const WeightDev& w, size_t r0, size_t nrows, float* out, cudaStream_t st, const int* row_dev, bool pdl) {
    if (nrows == 0) return cudaSuccess;
    const size_t n = nrows * (w.n_in / 32);
    const unsigned grid = (unsigned)((n + 127) / 128);
    B2_OTHER_SWITCH(w.fmt, launch_k(dq_other_kernel<FMT>, dim3(grid), dim3(128), 0, st, pdl, w, r0, nrows, out, row_dev))
}

cudaError_t launch_gemv_other(const WeightDev& w, const WeightDev* up, const float* x, size_t x_stride, float* y, size_t y_stride, int nt, int mode,
                              const float* gate, int sm_count, cudaStream_t st, bool pdl) {
    if (!gemv_other_supports(w) || nt < 1 || nt > 4) return cudaErrorInvalidValue;
    B2_OTHER_SWITCH(w.fmt, (nt == 1   ? launch_other_nt<FMT, 1>(w, up, x, x_stride, y, y_stride, mode, gate, sm_count, st, pdl)
                            : nt == 2 ? launch_other_nt<FMT, 2>(w, up, x, x_stride, y, y_stride, mode, gate, sm_count, st, pdl)
                            : nt == 3 ? launch_other_nt<FMT, 3>(w, up, x, x_stride, y, y_stride, mode, gate, sm_count, st, pdl)
                                      : launch_other_nt<FMT, 4>(w, up, x, x_stride, y, y_stride, mode, gate, sm_count, st, pdl)))
}

}  // namespace b2
