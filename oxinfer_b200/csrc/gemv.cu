// One-token dequant matrix-vector products (batch-1 decode): the role of dmv_* in the reference
// (src/cuda_decode.cu:139-174), written for B200 as HBM-bound streaming kernels.
//
// Design. A 4-bit weight costs 0.5 to 0.56 bytes; at B200's HBM rate one SM has only about three
// issue slots per weight, and a float dequant (extract, convert, multiply-add) needs more than
// that. So the activation vector is first split, per block of 32, into three signed 7-bit planes
// (x ~= xs * (q0 + 128 q1 + 16384 q2), 21 significant bits per block: xplanes_kernel), and the
// dot products run on dp4a over the packed nibbles / bytes with exact int32 sums; a sub-block's
// sum is converted once and scaled by `weight scale * xs` in f32. The result differs from the
// exact product by the 2^-21 rounding of x only. FP8 weights take the float path (hardware
// e4m3x2 -> f16x2 conversion), with f32 x.
//
// Every lane issues all of its 16-byte weight loads for a row group before using any of them;
// a warp owns ROWS rows at a time and the vector lives in shared memory, staged once per CTA.
#include <cuda_fp8.h>

#include <cstdio>

#include "kernels.h"

namespace b2 {

namespace {

constexpr int GEMV_THREADS = 256;
constexpr int GEMV_WARPS = GEMV_THREADS / 32;
constexpr float XQ_MAX = 1040000.0f;  // |q0 + 128 q1 + 16384 q2| <= 63 + 128*63 + 16384*63 = 1040319

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// ---- activation planes ----------------------------------------------------------------------
__global__ void __launch_bounds__(256) xplanes_kernel(const float* __restrict__ x, int K, int perm8, XPlanes out) {
    int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (warp >= K / 32) return;
    float v = x[warp * 32 + lane];
    float a = fabsf(v);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, o));
    float s = a / XQ_MAX;
    int q = a > 0.0f ? __float2int_rn(v * (XQ_MAX / a)) : 0;
    q = max(-(int)XQ_MAX, min((int)XQ_MAX, q));
    int q0 = ((q + 64) & 127) - 64;
    int r1 = (q - q0) >> 7;
    int q1 = ((r1 + 64) & 127) - 64;
    int q2 = (r1 - q1) >> 7;
    int pos = lane;
    if (perm8) {
        int i = lane & 7;
        pos = (lane & ~7) | ((i & 1) ? 4 + (i >> 1) : (i >> 1));
    }
    size_t at = (size_t)warp * 32 + pos;
    out.planes[at] = (int8_t)q0;
    out.planes[(size_t)K + at] = (int8_t)q1;
    out.planes[2 * (size_t)K + at] = (int8_t)q2;
    int sum16 = q;
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) sum16 += __shfl_xor_sync(0xffffffffu, sum16, o);
    int sum32 = sum16 + __shfl_xor_sync(0xffffffffu, sum16, 16);
    if ((lane & 15) == 0) out.v16[warp * 2 + (lane >> 4)] = sum16;
    if (lane == 0) {
        out.xs[warp] = s;
        out.xsum[warp] = s * (float)sum32;
    }
}

// The vector as the kernels see it in shared memory.
struct XS {
    const int8_t* p0;  // plane 0, K bytes; planes 1 and 2 follow at +K, +2K
    const float* xs;
    const float* xsum;
    const int32_t* v16;
    const float* xf;  // FP8: the f32 vector
    int K;
};

__device__ __forceinline__ int dp(uint32_t a, uint32_t b, int c) { return __dp4a((int)a, (int)b, c); }
__device__ __forceinline__ int planes3(int a0, int a1, int a2) { return a0 + (a1 << 7) + (a2 << 14); }

__device__ __forceinline__ float silu(float a) { return a / (1.0f + __expf(-a)); }
__device__ __forceinline__ float gelu_tanh(float a) {
    float t = 0.7978845608f * (a + 0.044715f * a * a * a);
    return 0.5f * a * (1.0f + tanhf(t));
}

// ---- per-format row pieces: `load` issues the global loads of one warp-iteration of one row,
// `dot` consumes them against the vector. An iteration covers ITER_K consecutive k.

struct FmtQ4K {
    static constexpr int ITER_K = 2048;  // 8 super-blocks, 4 lanes each (one 64-group per lane)
    struct Regs {
        uint4 hdr, q0, q1;
    };
    __device__ static __forceinline__ bool active(int K, int it, int lane) { return it * 8 + (lane >> 2) < K / 256; }
    __device__ static __forceinline__ void load(const WeightDev& w, size_t row, int it, int lane, Regs& r) {
        const uint8_t* blk = w.p0 + (row * (w.n_in / 256) + it * 8 + (lane >> 2)) * 144;
        r.hdr = __ldg((const uint4*)blk);
        r.q0 = __ldg((const uint4*)(blk + 16 + 32 * (lane & 3)));
        r.q1 = __ldg((const uint4*)(blk + 32 + 32 * (lane & 3)));
    }
    __device__ static __forceinline__ float dot(const Regs& r, const XS& x, int it, int lane) {
        int j = lane & 3;
        int k0 = (it * 8 + (lane >> 2)) * 256 + 64 * j;
        float d = __half2float(__ushort_as_half((unsigned short)(r.hdr.x & 0xffff)));
        float dmin = __half2float(__ushort_as_half((unsigned short)(r.hdr.x >> 16)));
        uint32_t sc0, mn0, sc1, mn1;
        q4k_scale_min(2 * j, r.hdr.y, r.hdr.z, r.hdr.w, sc0, mn0);
        q4k_scale_min(2 * j + 1, r.hdr.y, r.hdr.z, r.hdr.w, sc1, mn1);
        const uint32_t qw[8] = {r.q0.x, r.q0.y, r.q0.z, r.q0.w, r.q1.x, r.q1.y, r.q1.z, r.q1.w};
        int lo[3], hi[3];
#pragma unroll
        for (int p = 0; p < 3; p++) {
            const uint4* xp = (const uint4*)(x.p0 + (size_t)p * x.K + k0);
            uint4 a = xp[0], b = xp[1], c = xp[2], e = xp[3];
            const uint32_t xl[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
            const uint32_t xh[8] = {c.x, c.y, c.z, c.w, e.x, e.y, e.z, e.w};
            int sl = 0, sh = 0;
#pragma unroll
            for (int i = 0; i < 8; i++) {
                sl = dp(qw[i] & 0x0F0F0F0Fu, xl[i], sl);
                sh = dp((qw[i] >> 4) & 0x0F0F0F0Fu, xh[i], sh);
            }
            lo[p] = sl;
            hi[p] = sh;
        }
        int b0 = k0 >> 5;
        float acc = (d * (float)sc0) * x.xs[b0] * (float)planes3(lo[0], lo[1], lo[2]);
        acc = fmaf((d * (float)sc1) * x.xs[b0 + 1], (float)planes3(hi[0], hi[1], hi[2]), acc);
        acc = fmaf(-(dmin * (float)mn0), x.xsum[b0], acc);
        acc = fmaf(-(dmin * (float)mn1), x.xsum[b0 + 1], acc);
        return acc;
    }
};

struct FmtMLX4 {
    static constexpr int ITER_K = 2048;  // 32 groups of 64, one per lane
    struct Regs {
        uint4 q0, q1;
        uint32_t sb;  // scale | bias << 16 (bf16 bits)
    };
    __device__ static __forceinline__ bool active(int K, int it, int lane) { return it * 32 + lane < K / 64; }
    __device__ static __forceinline__ void load(const WeightDev& w, size_t row, int it, int lane, Regs& r) {
        size_t g = row * (w.n_in / 64) + it * 32 + lane;
        const uint4* q = (const uint4*)(w.p0 + g * 32);
        r.q0 = __ldg(q);
        r.q1 = __ldg(q + 1);
        r.sb = (uint32_t)__ldg((const uint16_t*)w.p1 + g) | ((uint32_t)__ldg((const uint16_t*)w.p2 + g) << 16);
    }
    __device__ static __forceinline__ float dot(const Regs& r, const XS& x, int it, int lane) {
        int k0 = (it * 32 + lane) * 64;
        // The CPU path's values (src/quant.rs:518-563,586-606): d = f16(scale), offset = bf16(bias + 8 scale),
        // w = (nib - 8) d + offset = nib d + (offset - 8 d).
        float s = bf16_bits_to_f32(r.sb & 0xffff), b = bf16_bits_to_f32(r.sb >> 16);
        float d = __half2float(__float2half_rn(s));
        float off = bf16_bits_to_f32(f32_to_bf16_bits(__fadd_rn(b, __fmul_rn(8.0f, s))));
        const uint32_t qw[8] = {r.q0.x, r.q0.y, r.q0.z, r.q0.w, r.q1.x, r.q1.y, r.q1.z, r.q1.w};
        int sa[3], sb[3];
#pragma unroll
        for (int p = 0; p < 3; p++) {
            // perm8 layout: word pair (2i, 2i+1) of the plane holds the even / odd elements of weight word i
            const uint4* xp = (const uint4*)(x.p0 + (size_t)p * x.K + k0);
            uint4 a = xp[0], bq = xp[1], c = xp[2], e = xp[3];
            const uint32_t xw[16] = {a.x, a.y, a.z, a.w, bq.x, bq.y, bq.z, bq.w, c.x, c.y, c.z, c.w, e.x, e.y, e.z, e.w};
            int s0 = 0, s1 = 0;
#pragma unroll
            for (int i = 0; i < 4; i++) {
                s0 = dp(qw[i] & 0x0F0F0F0Fu, xw[2 * i], s0);
                s0 = dp((qw[i] >> 4) & 0x0F0F0F0Fu, xw[2 * i + 1], s0);
                s1 = dp(qw[4 + i] & 0x0F0F0F0Fu, xw[8 + 2 * i], s1);
                s1 = dp((qw[4 + i] >> 4) & 0x0F0F0F0Fu, xw[8 + 2 * i + 1], s1);
            }
            sa[p] = s0;
            sb[p] = s1;
        }
        int b0 = k0 >> 5;
        float dots = x.xs[b0] * (float)planes3(sa[0], sa[1], sa[2]);
        dots = fmaf(x.xs[b0 + 1], (float)planes3(sb[0], sb[1], sb[2]), dots);
        float acc = d * dots;
        acc = fmaf(off - 8.0f * d, x.xsum[b0] + x.xsum[b0 + 1], acc);
        return acc;
    }
};

struct FmtQ6K {
    static constexpr int ITER_K = 2048;  // 8 blocks of 256, 4 lanes each (64 elements per lane)
    struct Regs {
        uint4 qh, qa, qb;
        uint2 sc;
        uint32_t d;
    };
    __device__ static __forceinline__ bool active(int K, int it, int lane) { return it * 8 + (lane >> 2) < K / 256; }
    __device__ static __forceinline__ void load(const WeightDev& w, size_t row, int it, int lane, Regs& r) {
        size_t K = w.n_in;
        size_t blk = it * 8 + (lane >> 2);
        int n = (lane >> 1) & 1, u = lane & 1;
        r.qh = __ldg((const uint4*)(w.p1 + row * (K / 4) + blk * 64 + 32 * n + 16 * u));
        r.qa = __ldg((const uint4*)(w.p0 + row * (K / 2) + blk * 128 + 64 * n + 16 * u));
        r.qb = __ldg((const uint4*)(w.p0 + row * (K / 2) + blk * 128 + 64 * n + 32 + 16 * u));
        r.sc = __ldg((const uint2*)(w.p2 + row * (K / 16) + blk * 16 + 8 * n));
        r.d = __ldg((const uint16_t*)w.p3 + row * (K / 256) + blk);
    }
    __device__ static __forceinline__ float dot(const Regs& r, const XS& x, int it, int lane) {
        int n = (lane >> 1) & 1, u = lane & 1;
        int kb = (it * 8 + (lane >> 2)) * 256 + 128 * n + 16 * u;  // quarter k4 adds 32 k4
        float d = __half2float(__ushort_as_half((unsigned short)r.d));
        const uint32_t H[4] = {r.qh.x, r.qh.y, r.qh.z, r.qh.w};
        const uint32_t A[4] = {r.qa.x, r.qa.y, r.qa.z, r.qa.w};
        const uint32_t B[4] = {r.qb.x, r.qb.y, r.qb.z, r.qb.w};
        uint64_t scw = (uint64_t)r.sc.x | ((uint64_t)r.sc.y << 32);
        float acc = 0.0f;
#pragma unroll
        for (int k4 = 0; k4 < 4; k4++) {
            uint32_t q[4];
#pragma unroll
            for (int i = 0; i < 4; i++) {
                uint32_t lo = (k4 & 1) ? B[i] : A[i];
                lo = (k4 & 2) ? (lo >> 4) : lo;
                uint32_t hb = (k4 == 0) ? (H[i] << 4) : (k4 == 1) ? (H[i] << 2) : (k4 == 2) ? H[i] : (H[i] >> 2);
                q[i] = (lo & 0x0F0F0F0Fu) | (hb & 0x30303030u);
            }
            int k0 = kb + 32 * k4;
            int s[3];
#pragma unroll
            for (int p = 0; p < 3; p++) {
                uint4 xv = *(const uint4*)(x.p0 + (size_t)p * x.K + k0);
                int a = dp(q[0], xv.x, 0);
                a = dp(q[1], xv.y, a);
                a = dp(q[2], xv.z, a);
                a = dp(q[3], xv.w, a);
                s[p] = a;
            }
            int total = planes3(s[0], s[1], s[2]) - 32 * x.v16[k0 >> 4];
            float scale = (float)(int8_t)((scw >> (8 * (u + 2 * k4))) & 0xff);
            acc = fmaf((d * scale) * x.xs[k0 >> 5], (float)total, acc);
        }
        return acc;
    }
};

struct FmtQ8_0 {
    static constexpr int ITER_K = 512;  // 16 bytes = 16 weights per lane
    struct Regs {
        uint4 q;
        uint32_t d;
    };
    __device__ static __forceinline__ bool active(int K, int it, int lane) { return it * 512 + lane * 16 < K; }
    __device__ static __forceinline__ void load(const WeightDev& w, size_t row, int it, int lane, Regs& r) {
        size_t k0 = (size_t)it * 512 + lane * 16;
        r.q = __ldg((const uint4*)(w.p0 + row * w.n_in + k0));
        r.d = __ldg((const uint16_t*)w.p1 + row * (w.n_in / 32) + k0 / 32);
    }
    __device__ static __forceinline__ float dot(const Regs& r, const XS& x, int it, int lane) {
        int k0 = it * 512 + lane * 16;
        int s[3];
#pragma unroll
        for (int p = 0; p < 3; p++) {
            uint4 xv = *(const uint4*)(x.p0 + (size_t)p * x.K + k0);
            int a = dp(r.q.x, xv.x, 0);
            a = dp(r.q.y, xv.y, a);
            a = dp(r.q.z, xv.z, a);
            a = dp(r.q.w, xv.w, a);
            s[p] = a;
        }
        float d = __half2float(__ushort_as_half((unsigned short)r.d));
        return (d * x.xs[k0 >> 5]) * (float)planes3(s[0], s[1], s[2]);
    }
};

struct FmtF8 {
    static constexpr int ITER_K = 512;  // 16 e4m3 bytes per lane
    struct Regs {
        uint4 q;
        float s;
    };
    __device__ static __forceinline__ bool active(int K, int it, int lane) { return it * 512 + lane * 16 < K; }
    __device__ static __forceinline__ void load(const WeightDev& w, size_t row, int it, int lane, Regs& r) {
        size_t k0 = (size_t)it * 512 + lane * 16;
        r.q = __ldg((const uint4*)(w.p0 + row * w.n_in + k0));
        r.s = w.p1 ? __ldg((const float*)w.p1 + ((w.bs_row0 + row) / w.bs_rows) * w.bs_ncb + k0 / w.bs_cols) : 1.0f;
    }
    __device__ static __forceinline__ float dot(const Regs& r, const XS& x, int it, int lane) {
        int k0 = it * 512 + lane * 16;
        const uint32_t qw[4] = {r.q.x, r.q.y, r.q.z, r.q.w};
        const float4* xv = (const float4*)(x.xf + k0);
        float part = 0.0f;
#pragma unroll
        for (int i = 0; i < 4; i++) {
            float4 xx = xv[i];
            __half2_raw h01 = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(qw[i] & 0xffff), __NV_E4M3);
            __half2_raw h23 = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(qw[i] >> 16), __NV_E4M3);
            float2 f01 = __half22float2(*(const __half2*)&h01), f23 = __half22float2(*(const __half2*)&h23);
            part = fmaf(f01.x, xx.x, part);
            part = fmaf(f01.y, xx.y, part);
            part = fmaf(f23.x, xx.z, part);
            part = fmaf(f23.y, xx.w, part);
        }
        return part * r.s;
    }
};

template <class F, int ROWS, bool PAIR, bool XF32>
__global__ void __launch_bounds__(GEMV_THREADS)
gemv_kernel(WeightDev w, WeightDev w2, const float* __restrict__ x, XPlanes xp, float* __restrict__ y, int mode,
            const float* __restrict__ gate) {
    extern __shared__ __align__(16) uint8_t smem[];
    const int K = (int)w.n_in;
    XS xs;
    xs.K = K;
    if constexpr (XF32) {
        float* xf = (float*)smem;
        for (int i = threadIdx.x; i < K / 4; i += GEMV_THREADS) ((float4*)xf)[i] = ((const float4*)x)[i];
        xs.xf = xf;
        xs.p0 = nullptr;
        xs.xs = xs.xsum = nullptr;
        xs.v16 = nullptr;
    } else {
        // planes | xs | xsum | v16 are contiguous in global memory in this order: one 16-byte copy loop
        size_t bytes = xplanes_bytes((size_t)K);
        const uint4* src = (const uint4*)xp.planes;
        for (int i = threadIdx.x; i < (int)(bytes / 16); i += GEMV_THREADS) ((uint4*)smem)[i] = src[i];
        xs.p0 = (const int8_t*)smem;
        xs.xs = (const float*)(smem + 3 * (size_t)K);
        xs.xsum = xs.xs + K / 32;
        xs.v16 = (const int32_t*)(xs.xsum + K / 32);
        xs.xf = nullptr;
    }
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const size_t n_out = w.n_out;
    const int iters = (K + F::ITER_K - 1) / F::ITER_K;
    for (size_t r0 = ((size_t)blockIdx.x * GEMV_WARPS + warp) * ROWS; r0 < n_out; r0 += (size_t)gridDim.x * GEMV_WARPS * ROWS) {
        float acc[ROWS], acc2[ROWS];
#pragma unroll
        for (int r = 0; r < ROWS; r++) acc[r] = acc2[r] = 0.0f;
        for (int it = 0; it < iters; it++) {
            if (!F::active(K, it, lane)) continue;
            typename F::Regs regs[ROWS], regs2[PAIR ? ROWS : 1];
#pragma unroll
            for (int r = 0; r < ROWS; r++) {
                size_t row = min(r0 + r, n_out - 1);
                F::load(w, row, it, lane, regs[r]);
                if constexpr (PAIR) F::load(w2, row, it, lane, regs2[r]);
            }
#pragma unroll
            for (int r = 0; r < ROWS; r++) {
                acc[r] += F::dot(regs[r], xs, it, lane);
                if constexpr (PAIR) acc2[r] += F::dot(regs2[r], xs, it, lane);
            }
        }
#pragma unroll
        for (int r = 0; r < ROWS; r++) {
            float a = warp_sum(acc[r]);
            float b = PAIR ? warp_sum(acc2[r]) : 0.0f;
            if (lane == 0 && r0 + r < n_out) {
                float* o = y + r0 + r;
                if (mode == B2_MODE_STORE)
                    *o = a;
                else if (mode == B2_MODE_ADD)
                    *o += a;
                else if (mode == B2_MODE_SILU_PAIR)
                    *o = silu(a) * b;
                else if (mode == B2_MODE_GELU_PAIR)
                    *o = gelu_tanh(a) * b;
                else
                    *o += a * (1.0f / (1.0f + __expf(-gate[0])));
            }
        }
    }
}

template <class F, bool XF32>
cudaError_t launch_fmt(const WeightDev& w, const WeightDev* up, const float* x, XPlanes xp, float* y, int mode, const float* gate,
                       int sm_count, cudaStream_t st) {
    constexpr int ROWS = 2;
    size_t smem = XF32 ? w.n_in * 4 : xplanes_bytes(w.n_in);
    bool pair = mode == B2_MODE_SILU_PAIR || mode == B2_MODE_GELU_PAIR;
    auto kern = pair ? gemv_kernel<F, ROWS, true, XF32> : gemv_kernel<F, ROWS, false, XF32>;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
    }
    size_t groups = (w.n_out + (size_t)GEMV_WARPS * ROWS - 1) / ((size_t)GEMV_WARPS * ROWS);
    size_t per_sm = smem ? (size_t)(220 * 1024) / (smem + 1024) : 8;
    per_sm = per_sm < 1 ? 1 : (per_sm > 4 ? 4 : per_sm);
    size_t grid = groups < (size_t)sm_count * per_sm ? groups : (size_t)sm_count * per_sm;
    kern<<<(unsigned)grid, GEMV_THREADS, smem, st>>>(w, pair ? *up : w, x, xp, y, mode, gate);
    return cudaGetLastError();
}

}  // namespace

bool gemv_supports(const WeightDev& w) {
    switch (w.fmt) {
        case B2_FMT_MLX4: return w.group == 64 && w.n_in % 64 == 0 && w.n_in * 3 + w.n_in / 2 <= 200 * 1024;
        case B2_FMT_Q4_K:
        case B2_FMT_Q6_K: return w.n_in % 256 == 0 && xplanes_bytes(w.n_in) <= 200 * 1024;
        case B2_FMT_Q8_0: return w.n_in % 32 == 0 && xplanes_bytes(w.n_in) <= 200 * 1024;
        case B2_FMT_F8E4M3: return w.n_in % 16 == 0 && w.n_in * 4 <= 200 * 1024 && (w.p1 == nullptr || w.bs_cols % 16 == 0);
        default: return false;
    }
}

cudaError_t launch_xplanes(const float* x, size_t K, int perm8, XPlanes out, cudaStream_t st) {
    unsigned warps = (unsigned)(K / 32);
    xplanes_kernel<<<(warps + 7) / 8, 256, 0, st>>>(x, (int)K, perm8, out);
    return cudaGetLastError();
}

cudaError_t launch_gemv(const WeightDev& w, const WeightDev* up, const float* x, XPlanes xp, float* y, int mode, const float* gate,
                        int sm_count, cudaStream_t st) {
    switch (w.fmt) {
        case B2_FMT_MLX4: return launch_fmt<FmtMLX4, false>(w, up, x, xp, y, mode, gate, sm_count, st);
        case B2_FMT_Q4_K: return launch_fmt<FmtQ4K, false>(w, up, x, xp, y, mode, gate, sm_count, st);
        case B2_FMT_Q6_K: return launch_fmt<FmtQ6K, false>(w, up, x, xp, y, mode, gate, sm_count, st);
        case B2_FMT_Q8_0: return launch_fmt<FmtQ8_0, false>(w, up, x, xp, y, mode, gate, sm_count, st);
        case B2_FMT_F8E4M3: return launch_fmt<FmtF8, true>(w, up, x, xp, y, mode, gate, sm_count, st);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace b2

// =============================================================================================
// b2_matvec_q4k_noalloc: the Q4_K matrix-vector product for callers that must not allocate.
//
// Some hosts of this library cannot call cudaMalloc at the moment they need a product: a serving
// process that handed the whole device to its own arena at start-up (oxinfer's decode plans carve
// every buffer out of one arena they own, src/cuda_decode.rs:372-383) has nothing left for the
// runtime to give, and a latency-critical decode loop must not enter the allocator at all. The
// regular entry points keep their scratch (the activation planes the GEMV kernels read) in buffers
// that grow on demand; this one keeps it in a fixed array that is part of the loaded library.
//
// The array below is device memory reserved once per GPU for as long as the library stays loaded:
// 57,344 bytes, enough for an activation vector of B2_NOALLOC_MAX_K = 16384 elements.
// In host code the name of a __device__ array is only a stand-in: the device address comes from
// cudaGetSymbolAddress, asked for once per device with that device current (the first call on a
// device does this set-up, so make that first call outside any stream capture).
// Every call writes the whole part of the array it uses before reading it, so nothing has to be
// cleared between calls; but all calls share the one array, so two calls whose kernels can overlap
// on the GPU (different streams, no dependency between them) race on it. Serialize them.
// =============================================================================================
namespace b2 {
namespace {
constexpr size_t NOALLOC_MAX_K = 16384;
constexpr size_t NOALLOC_BYTES = 3 * NOALLOC_MAX_K + 8 * (NOALLOC_MAX_K / 32) + 4 * (NOALLOC_MAX_K / 16);
static __device__ __align__(256) uint8_t g_noalloc_scratch[NOALLOC_BYTES];

constexpr int NOALLOC_MAX_DEVICES = 64;
void* g_noalloc_ptr[NOALLOC_MAX_DEVICES];   // device address of g_noalloc_scratch, per device
int g_noalloc_sms[NOALLOC_MAX_DEVICES];

int noalloc_fail(char* err, size_t err_len, int code, const char* text, cudaError_t e = cudaSuccess) {
    if (err && err_len) {
        if (e != cudaSuccess)
            snprintf(err, err_len, "[b200qmm: matvec_q4k_noalloc: %s: %s]", text, cudaGetErrorString(e));
        else
            snprintf(err, err_len, "[b200qmm: matvec_q4k_noalloc: %s]", text);
    }
    return code;
}
}  // namespace
}  // namespace b2

extern "C" __attribute__((visibility("default"))) int b2_matvec_q4k_noalloc(const void* w_blocks_dev, size_t n_out, size_t n_in,
                                                                             const float* x_dev, float* y_dev, void* cuda_stream,
                                                                             char* err, size_t err_len) {
    using namespace b2;
    if (!w_blocks_dev || !x_dev || !y_dev || n_out == 0) return noalloc_fail(err, err_len, B2_ERR_ARG, "null pointer or empty matrix");
    if (n_in == 0 || n_in % 256 != 0) return noalloc_fail(err, err_len, B2_ERR_ARG, "n_in must be a positive multiple of 256 (Q4_K super-blocks)");
    if (n_in > NOALLOC_MAX_K) {
        if (err && err_len)
            snprintf(err, err_len, "[b200qmm: matvec_q4k_noalloc: n_in = %zu exceeds the built-in scratch (at most %zu); use b2_matvec_dev]", n_in,
                     NOALLOC_MAX_K);
        return B2_ERR_ARG;
    }
    if (((uintptr_t)w_blocks_dev & 15) || ((uintptr_t)x_dev & 3) || ((uintptr_t)y_dev & 3))
        return noalloc_fail(err, err_len, B2_ERR_ARG, "weights must be 16-byte aligned, x and y 4-byte aligned");
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return noalloc_fail(err, err_len, B2_ERR_CUDA, "cudaGetDevice", e);
    if (dev < 0 || dev >= NOALLOC_MAX_DEVICES) return noalloc_fail(err, err_len, B2_ERR_ARG, "device ordinal out of range");
    if (!g_noalloc_ptr[dev]) {
        // once per device, with that device current: the device-side address of the scratch array
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
        if (e != cudaSuccess || !p) return noalloc_fail(err, err_len, B2_ERR_CUDA, "cudaGetSymbolAddress(scratch)", e);
        int sms = 0;
        e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        if (e != cudaSuccess || sms <= 0) return noalloc_fail(err, err_len, B2_ERR_CUDA, "cudaDeviceGetAttribute", e);
        g_noalloc_sms[dev] = sms;
        g_noalloc_ptr[dev] = p;
    }
    WeightDev w{};
    w.fmt = B2_FMT_Q4_K;
    w.n_out = n_out;
    w.n_in = n_in;
    w.p0 = (const uint8_t*)w_blocks_dev;
    XPlanes xp = xplanes_at(g_noalloc_ptr[dev], n_in);
    cudaStream_t st = (cudaStream_t)cuda_stream;
    e = launch_xplanes(x_dev, n_in, 0, xp, st);
    if (e != cudaSuccess) return noalloc_fail(err, err_len, B2_ERR_CUDA, "activation planes kernel", e);
    e = launch_gemv(w, nullptr, x_dev, xp, y_dev, B2_MODE_STORE, nullptr, g_noalloc_sms[dev], st);
    if (e != cudaSuccess) return noalloc_fail(err, err_len, B2_ERR_CUDA, "gemv kernel", e);
    return B2_OK;
}
