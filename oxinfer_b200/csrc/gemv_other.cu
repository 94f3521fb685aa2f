// The other GGUF block formats on the device (dq_other.cuh): bit-exact dequantization, and one generic matrix-vector
// kernel that decodes 32 weights at a time in registers and multiplies them with the f32 activations (no integer planes,
// no repack: the rows stay as they are in the GGUF file). It takes the five output modes of dmv_out
// (src/cuda_decode.cu:131-137), the SiLU / GELU pair, and up to four tokens per launch with the weights read once (each
// token's row equals its one-token row bit for bit). The reference declines every GGUF type on its CUDA backend
// (src/cuda.rs:642); these formats get a correct device path here, not a tuned one: a warp brings 1024 weights' worth of
// its row's bytes into shared memory with aligned 16-byte loads (the next run is in flight while this one is decoded), and a
// lane decodes one 32-weight chunk of it with byte reads, five to seven instructions per weight.
#include "dq_other.cuh"
#include "gemv_core.cuh"

namespace b2 {

using namespace gemv_core;

namespace {

// One thread per 32 consecutive output elements of a row.
template <int FMT>
__global__ void __launch_bounds__(128) dq_other_kernel(WeightDev w, size_t r0, size_t nrows, float* __restrict__ out, const int* __restrict__ row_dev) {
    __shared__ float lut[16];
    lut_fill<FMT>(lut, threadIdx.x);
    __syncthreads();
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
    constexpr int BS = (FMT == B2_FMT_Q2_K || FMT == B2_FMT_Q3_K || FMT == B2_FMT_Q5_K || FMT == B2_FMT_IQ4_XS) ? 256 : FMT == B2_FMT_NVFP4 ? 64 : 32;
    const uint8_t* blk = w.p0 + r * other_row_bytes(FMT, K) + (c * 32 / BS) * other_type_size(FMT);
    float v[32];
    dequant32_other<FMT>(blk, (int)(c % (BS / 32)), v, lut);
    if constexpr (FMT == B2_FMT_NVFP4) {  // the tensor's global scale on top of what the blocks decode (src/ggml.rs:420-432)
        if (w.p1) {
            const float gs = __ldg((const float*)w.p1);
#pragma unroll
            for (int k = 0; k < 32; k++) v[k] = __fmul_rn(v[k], gs);
        }
    }
    float4* o = (float4*)(out + (i / per_row) * K + c * 32);
#pragma unroll
    for (int k = 0; k < 8; k++) o[k] = make_float4(v[4 * k], v[4 * k + 1], v[4 * k + 2], v[4 * k + 3]);
}

constexpr int OW = 8;       // warps per CTA, one weight row per warp at a time
constexpr int STAGE = 800;  // bytes of a warp's staging run: the largest run (32 x 24 bytes) + 15 of misalignment, in 16-byte words

template <int FMT>
struct OtherShape {
    static constexpr int BS = (FMT == B2_FMT_Q2_K || FMT == B2_FMT_Q3_K || FMT == B2_FMT_Q5_K || FMT == B2_FMT_IQ4_XS) ? 256 : FMT == B2_FMT_NVFP4 ? 64 : 32;
    static constexpr int TS = FMT == B2_FMT_NVFP4 ? 36 : FMT == B2_FMT_Q4_0 ? 18 : FMT == B2_FMT_Q4_1 ? 20 : FMT == B2_FMT_Q5_0 ? 22 : FMT == B2_FMT_Q5_1 ? 24 : FMT == B2_FMT_Q2_K ? 84
                              : FMT == B2_FMT_Q3_K ? 110 : FMT == B2_FMT_Q5_K ? 176 : FMT == B2_FMT_IQ4_NL ? 18 : FMT == B2_FMT_IQ4_XS ? 136 : 17;
    static constexpr int RUN = 1024 / BS * TS;  // bytes of 1024 weights
    static_assert(RUN + 15 <= STAGE, "staging run");
};

// The 16-byte words that cover the n bytes at `p` (n <= RUN), two per lane at most, into registers / from registers into
// the warp's staging buffer. The words start at the address rounded down to 16 (never below the allocation, which is
// 256-byte aligned; a row shard starts at any byte) and may reach up to 15 bytes past p + n (the uploads leave that much
// room after the last row).
__device__ __forceinline__ void run_load(const uint8_t* p, int n, int lane, uint4 (&r)[2]) {
    const uintptr_t a = (uintptr_t)p;
    const uint4* src = (const uint4*)(a & ~(uintptr_t)15);
    const int words = (int)((a & 15) + n + 15) >> 4;
#pragma unroll
    for (int i = 0; i < 2; i++)
        if (lane + 32 * i < words) r[i] = ldg_stream(src + lane + 32 * i);
}
__device__ __forceinline__ void run_store(uint8_t* stage, int lane, const uint4 (&r)[2]) {
#pragma unroll
    for (int i = 0; i < 2; i++)
        if (lane + 32 * i < STAGE / 16) ((uint4*)stage)[lane + 32 * i] = r[i];
}

template <int FMT, bool PAIR, int NT>
__global__ void __launch_bounds__(OW * 32, 3) gemv_other_kernel(WeightDev w, WeightDev w2, const float* __restrict__ x, size_t x_stride, float* __restrict__ y,
                                                            size_t y_stride, int mode, const float* __restrict__ gate) {
    using S = OtherShape<FMT>;
    constexpr int M = PAIR ? 2 : 1;
    extern __shared__ __align__(16) uint8_t xsm[];  // the NT activation vectors, 16-byte slots permuted (xslot)
    __shared__ __align__(16) uint8_t stage_all[OW][M][STAGE];
    __shared__ float lut[16];
    lut_fill<FMT>(lut, threadIdx.x);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const size_t K = w.n_in, chunks = K / 32, rb = other_row_bytes(FMT, K);
    const int iters = (int)((chunks + 31) / 32);
    // bytes of iteration `it` of a row: whole blocks, the last run may be shorter
    auto run_bytes = [&](int it) { return (int)min((size_t)S::RUN, rb - (size_t)it * S::RUN); };
    size_t r = (size_t)blockIdx.x * OW + warp;
    uint4 pre[M][2] = {};
    if (r < w.n_out) {  // the weights do not depend on the kernel ahead: fetch the first run before waiting for it
#pragma unroll
        for (int m = 0; m < M; m++) run_load((m ? w2.p0 : w.p0) + r * rb, run_bytes(0), lane, pre[m]);
    }
    pdl_launch_dependents();
    pdl_wait();
    // A lane multiplies 32 consecutive weights by 32 consecutive activations: read from global memory that is 32 different
    // cache lines per load instruction, so the vectors go to shared memory once per CTA, with the eight 16-byte slots of
    // each lane's 128 bytes rotated by the lane number (slot g -> g ^ ((g >> 3) & 7)): conflict-free reads.
    for (int tk = 0; tk < NT; tk++) {
        const float4* src = (const float4*)(x + (size_t)tk * x_stride);
        float4* dst = (float4*)xsm + (size_t)tk * (K / 4);
        for (int g = threadIdx.x; g < (int)(K / 4); g += OW * 32) dst[g ^ ((g >> 3) & 7)] = __ldg(src + g);
    }
    __syncthreads();
    for (; r < w.n_out; r += (size_t)gridDim.x * OW) {
        float acc[M][NT];
#pragma unroll
        for (int m = 0; m < M; m++)
#pragma unroll
            for (int tk = 0; tk < NT; tk++) acc[m][tk] = 0.0f;
        for (int it = 0; it < iters; it++) {
            __syncwarp();  // the previous run has been decoded by every lane
#pragma unroll
            for (int m = 0; m < M; m++) run_store(stage_all[warp][m], lane, pre[m]);
            __syncwarp();
            // the next run of this row, or the first of the warp's next row, while this one is decoded
            {
                const bool more = it + 1 < iters;
                const size_t rn = more ? r : r + (size_t)gridDim.x * OW;
                if (rn < w.n_out) {
                    const int itn = more ? it + 1 : 0;
#pragma unroll
                    for (int m = 0; m < M; m++) run_load((m ? w2.p0 : w.p0) + rn * rb + (size_t)itn * S::RUN, run_bytes(itn), lane, pre[m]);
                }
            }
            const size_t c = (size_t)it * 32 + lane;
            if (c < chunks) {
#pragma unroll
                for (int m = 0; m < M; m++) {
                    const uint8_t* gm = (m ? w2.p0 : w.p0) + r * rb + (size_t)it * S::RUN;  // where this run starts in global memory
                    const uint8_t* blk = stage_all[warp][m] + ((uintptr_t)gm & 15) + (lane * 32 / S::BS) * S::TS;
                    float v[32];
                    dequant32_other<FMT>(blk, (int)(c % (S::BS / 32)), v, lut);
                    if constexpr (FMT == B2_FMT_NVFP4) {  // the global scale multiplies the decoded values, as in the bit-exact rows
                        const WeightDev& wm = m ? w2 : w;
                        if (wm.p1) {
                            const float gs = __ldg((const float*)wm.p1);
#pragma unroll
                            for (int k = 0; k < 32; k++) v[k] = __fmul_rn(v[k], gs);
                        }
                    }
#pragma unroll
                    for (int tk = 0; tk < NT; tk++) {
                        const float4* xv = (const float4*)xsm + (size_t)tk * (K / 4) + c * 8;
                        float a = acc[m][tk];
#pragma unroll
                        for (int k = 0; k < 8; k++) {
                            const float4 q = xv[k ^ (lane & 7)];
                            a = fmaf(v[4 * k], q.x, a);
                            a = fmaf(v[4 * k + 1], q.y, a);
                            a = fmaf(v[4 * k + 2], q.z, a);
                            a = fmaf(v[4 * k + 3], q.w, a);
                        }
                        acc[m][tk] = a;
                    }
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
    const size_t smem = w.n_in * 4 * NT;
    if (cudaError_t e = ensure_dynamic_smem((const void*)kern, smem, 32 * 1024); e != cudaSuccess) return e;
    size_t per_sm = (size_t)(220 * 1024) / (smem + 16 * 1024);
    per_sm = per_sm < 1 ? 1 : (per_sm > 6 ? 6 : per_sm);
    const size_t groups = (w.n_out + OW - 1) / OW, cap = (size_t)sm_count * per_sm;
    return launch_k(kern, dim3((unsigned)(groups < cap ? groups : cap)), dim3(OW * 32), smem, st, pdl, w, pair ? *up : w, x, x_stride, y, y_stride, mode, gate);
}

}  // namespace

// One token's vector must fit in shared memory (launch_gemv_other lowers the tokens per launch until they all do).
bool gemv_other_supports(const WeightDev& w) {
    return fmt_is_other(w.fmt) && w.n_in > 0 && w.n_in % other_block_size(w.fmt) == 0 && w.n_in % 32 == 0 && w.n_in * 4 <= 160 * 1024;
}

cudaError_t launch_dequantize_other(const WeightDev& w, size_t r0, size_t nrows, float* out, cudaStream_t st, const int* row_dev, bool pdl) {
    if (nrows == 0) return cudaSuccess;
    const size_t n = nrows * (w.n_in / 32);
    const unsigned grid = (unsigned)((n + 127) / 128);
    B2_OTHER_SWITCH(w.fmt, launch_k(dq_other_kernel<FMT>, dim3(grid), dim3(128), 0, st, pdl, w, r0, nrows, out, row_dev))
}

cudaError_t launch_gemv_other(const WeightDev& w, const WeightDev* up, const float* x, size_t x_stride, float* y, size_t y_stride, int nt, int mode,
                              const float* gate, int sm_count, cudaStream_t st, bool pdl) {
    if (!gemv_other_supports(w) || nt < 1 || nt > 4) return cudaErrorInvalidValue;
    if (nt > 1 && w.n_in * 4 * (size_t)nt > 160 * 1024) {  // the vectors of nt tokens do not fit together: fewer per launch
        const int half = nt / 2;
        if (cudaError_t e = launch_gemv_other(w, up, x, x_stride, y, y_stride, half, mode, gate, sm_count, st, pdl); e != cudaSuccess) return e;
        return launch_gemv_other(w, up, x + (size_t)half * x_stride, x_stride, y + (size_t)half * y_stride, y_stride, nt - half, mode, gate, sm_count, st, pdl);
    }
    B2_OTHER_SWITCH(w.fmt, (nt == 1   ? launch_other_nt<FMT, 1>(w, up, x, x_stride, y, y_stride, mode, gate, sm_count, st, pdl)
                            : nt == 2 ? launch_other_nt<FMT, 2>(w, up, x, x_stride, y, y_stride, mode, gate, sm_count, st, pdl)
                            : nt == 3 ? launch_other_nt<FMT, 3>(w, up, x, x_stride, y, y_stride, mode, gate, sm_count, st, pdl)
                                      : launch_other_nt<FMT, 4>(w, up, x, x_stride, y, y_stride, mode, gate, sm_count, st, pdl)))
}

}  // namespace b2
