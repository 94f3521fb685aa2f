// Element-wise pieces of the routed-expert layer around the grouped tensor-core GEMM:
//   route_topk   : top-k of the router logits with the reference's order and weights
//                  (route_top_k, src/moe.rs:180-193; dtopk, src/cuda_decode.cu:285-312)
//   moe_gather   : token rows -> per-expert segments, f32 -> f16, pad rows zero
//                  (moe_gather, src/cuda.rs:293-297)
//   moe_act      : act(gate) * up over the fused gate_up output, to f16 for the down projection
//                  (moe_act, src/cuda.rs:300-316; SiLU with expf as on the reference's GPU path)
//   moe_combine  : y[t] += sum_j w_j * o[slot(t, j)] in route order, multiply and add unfused
//                  (moe_combine, src/cuda.rs:319-330)
#include <algorithm>

#include "kernels.h"
#include "xplanes.cuh"

namespace b2 {

namespace {

// One warp per token: k rounds of "largest remaining logit, ties to the lower index".
__global__ void route_topk_kernel(const float* __restrict__ logits, int t, int n, int k, int* __restrict__ ids, float* __restrict__ w) {
    const int tok = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (tok >= t) return;
    const float* l = logits + (size_t)tok * n;
    // each lane keeps the candidates i = lane, lane + 32, ...; a chosen index is masked out
    unsigned long long taken = 0;  // bit j: candidate lane + 32 j already chosen (n <= 2048)
    float first = 0.0f, sum = 0.0f, mine = 0.0f;
    for (int r = 0; r < k; r++) {
        float best = -INFINITY;
        int bi = 0x7fffffff;
        for (int i = lane, j = 0; i < n; i += 32, j++) {
            if ((taken >> j) & 1ull) continue;
            float v = l[i];
            if (v > best || (v == best && i < bi)) {
                best = v;
                bi = i;
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            float ob = __shfl_xor_sync(0xffffffffu, best, o);
            int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ob > best || (ob == best && oi < bi)) {
                best = ob;
                bi = oi;
            }
        }
        if ((bi & 31) == lane) taken |= 1ull << (bi >> 5);
        if (r == 0) first = best;
        float e = expf(best - first);
        sum += e;
        if (lane == r) mine = e;
        if (lane == 0) ids[(size_t)tok * k + r] = bi;
    }
    if (lane < k) w[(size_t)tok * k + lane] = mine / sum;
}

// A power of two that brings a row's largest magnitude mx into [2^14, 2^15) (1 for an all-zero or non-finite row), and
// its inverse: f16 operands then neither overflow nor sink into subnormals, whatever the row's magnitude.
__device__ __forceinline__ void row_factor(float mx, float& s, float& inv) {
    s = inv = 1.0f;
    if (mx > 0.0f && mx < INFINITY) {
        int e;
        frexpf(mx, &e);
        const int up = min(100, max(-100, 15 - e));
        s = ldexpf(1.0f, up);
        inv = ldexpf(1.0f, -up);
    }
}
__device__ __forceinline__ float cta_max_256(float mx, float* red) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = mx;
    __syncthreads();
    mx = red[0];
#pragma unroll
    for (int i = 1; i < 8; i++) mx = fmaxf(mx, red[i]);
    return mx;
}
// Four values times a power of two -> four f16 (hi) and, with lo, the f16 of what that rounding left over.
__device__ __forceinline__ void store_terms(float4 v, float f, __half* hi, __half* lo) {
    v.x *= f; v.y *= f; v.z *= f; v.w *= f;
    const __half2 a = __floats2half2_rn(v.x, v.y), b = __floats2half2_rn(v.z, v.w);
    *(uint2*)hi = make_uint2(*(const uint32_t*)&a, *(const uint32_t*)&b);
    if (lo) {
        const float2 fa = __half22float2(a), fb = __half22float2(b);
        const __half2 c = __floats2half2_rn(v.x - fa.x, v.y - fa.y), d = __floats2half2_rn(v.z - fb.x, v.w - fb.y);
        *(uint2*)lo = make_uint2(*(const uint32_t*)&c, *(const uint32_t*)&d);
    }
}

// xg[row][h] (f16) = x[src[row]][h] (f32) * factor[row], zeros where src[row] < 0; unscale[row] = 1 / factor, which the
// GEMM's epilogue multiplies the row's results by. lo_off > 0: two-term rows (see launch_to_f16), the second term
// lo_off elements behind the first. One CTA of 256 threads per row; h is a multiple of 256 and at most 8192.
constexpr int GATHER_KEEP = 8;
__global__ void __launch_bounds__(256) moe_gather_kernel(const float* __restrict__ x, const int* __restrict__ src, int h, __half* __restrict__ xg,
                                                         float* __restrict__ unscale, size_t lo_off) {
    __shared__ float red[8];
    pdl_launch_dependents();  // a dependent launch: the kernel behind may set itself up; nothing is read or written before the wait
    pdl_wait();
    const int row = blockIdx.x;
    const int s = src[row];
    __half* o = xg + (size_t)row * h;
    if (s < 0) {
        for (int c = threadIdx.x * 4; c < h; c += 1024) {
            *(uint2*)(o + c) = make_uint2(0u, 0u);
            if (lo_off) *(uint2*)(o + lo_off + c) = make_uint2(0u, 0u);
        }
        if (threadIdx.x == 0) unscale[row] = 1.0f;
        return;
    }
    const float4* in = (const float4*)(x + (size_t)s * h);
    float4 v[GATHER_KEEP];
    float mx = 0.0f;
#pragma unroll
    for (int j = 0; j < GATHER_KEEP; j++) {
        const int i = j * 256 + threadIdx.x;
        v[j] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (i < h / 4) {
            v[j] = in[i];
            mx = fmaxf(fmaxf(mx, fmaxf(fabsf(v[j].x), fabsf(v[j].y))), fmaxf(fabsf(v[j].z), fabsf(v[j].w)));
        }
    }
    mx = cta_max_256(mx, red);
    float f, inv;
    row_factor(mx, f, inv);
#pragma unroll
    for (int j = 0; j < GATHER_KEEP; j++) {
        const int i = j * 256 + threadIdx.x;
        if (i < h / 4) store_terms(v[j], f, o + 4 * i, lo_off ? o + lo_off + 4 * i : nullptr);
    }
    if (threadIdx.x == 0) unscale[row] = inv;
}

// The same with a warp per row (eight rows per CTA, no CTA barrier): h = 128 * VPL, a lane keeps VPL float4. A CTA per row
// costs more in CTA launches than in bytes once there are tens of thousands of rows.
__device__ __forceinline__ float warp_max(float mx) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    return mx;
}
template <int VPL>
__global__ void __launch_bounds__(256) moe_gather_warp_kernel(const float* __restrict__ x, const int* __restrict__ src, int rows, __half* __restrict__ xg,
                                                              float* __restrict__ unscale, size_t lo_off) {
    constexpr int H = 128 * VPL;
    pdl_launch_dependents();  // a dependent launch: the kernel behind may set itself up; nothing is read or written before the wait
    pdl_wait();
    const int row = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (row >= rows) return;
    const int s = src[row];
    __half* o = xg + (size_t)row * H;
    if (s < 0) {
#pragma unroll
        for (int j = 0; j < VPL; j++) {
            const int c = (j * 32 + lane) * 4;
            *(uint2*)(o + c) = make_uint2(0u, 0u);
            if (lo_off) *(uint2*)(o + lo_off + c) = make_uint2(0u, 0u);
        }
        if (lane == 0) unscale[row] = 1.0f;
        return;
    }
    const float4* in = (const float4*)(x + (size_t)s * H);
    float4 v[VPL];
    float mx = 0.0f;
#pragma unroll
    for (int j = 0; j < VPL; j++) {
        v[j] = in[j * 32 + lane];
        mx = fmaxf(fmaxf(mx, fmaxf(fabsf(v[j].x), fabsf(v[j].y))), fmaxf(fabsf(v[j].z), fabsf(v[j].w)));
    }
    mx = warp_max(mx);
    float f, inv;
    row_factor(mx, f, inv);
#pragma unroll
    for (int j = 0; j < VPL; j++) {
        const int c = (j * 32 + lane) * 4;
        store_terms(v[j], f, o + c, lo_off ? o + lo_off + c : nullptr);
    }
    if (lane == 0) unscale[row] = inv;
}

// a[row][inter] (f16) = silu(g[row][c]) * g[row][inter + c] * factor[row] over the fused gate_up output g [rows][2 inter]
// (f32); factor[row] is the power of two of row_factor and unscale[row] = 1 / factor is what the down projection's epilogue
// multiplies the row's results by. lo_off as for the gather. src[row] < 0 marks a padding row (src may be null: no
// padding). One CTA per row; the row is read once (a thread keeps its products in registers between the maximum and the
// store) when inter <= 256 * 4 * ACT_KEEP.
constexpr int ACT_KEEP = 2;
// kind (MoeAct, src/gpu.rs:36-54; the arithmetic of the reference's moe_act, src/cuda.rs:300-316): 0 SiLU, 1 tanh GELU
// written as g * sigmoid(1.5957692 (g + 0.044715 g^3)), 2 SiLU with the clamp silu(min(g, l)) * clamp(u, -l, l).
__device__ __forceinline__ float gated_act(float g, float u, int kind, float limit) {
    if (kind == 1) {
        const float k = 1.5957692f * (g + 0.044715f * g * g * g);
        return g / (1.0f + expf(-k)) * u;
    }
    if (kind == 2) {
        g = fminf(g, limit);
        u = fminf(fmaxf(u, -limit), limit);
    }
    return g / (1.0f + expf(-g)) * u;
}

__global__ void __launch_bounds__(256) moe_act_kernel(const float* __restrict__ g, const int* __restrict__ src, int inter, __half* __restrict__ a,
                                                      float* __restrict__ unscale, size_t lo_off, int kind, float limit) {
    __shared__ float red[8];
    pdl_launch_dependents();  // a dependent launch: the kernel behind may set itself up; nothing is read or written before the wait
    pdl_wait();
    const size_t row = blockIdx.x;
    __half* ar = a + row * inter;
    if (src && src[row] < 0) {  // a padding row of an expert's last tile: its products are zero, nothing to read
        for (int c = threadIdx.x * 4; c < inter; c += 256 * 4) {
            *(uint2*)(ar + c) = make_uint2(0u, 0u);
            if (lo_off) *(uint2*)(ar + lo_off + c) = make_uint2(0u, 0u);
        }
        if (threadIdx.x == 0) unscale[row] = 1.0f;
        return;
    }
    const float* gr = g + row * 2 * (size_t)inter;
    const bool keep = inter <= 256 * 4 * ACT_KEEP;  // inter is a multiple of 256: whole float4 per thread
    auto act4 = [&](int c) {
        const float4 gate = *(const float4*)(gr + c), up = *(const float4*)(gr + inter + c);
        float4 r;
        r.x = gated_act(gate.x, up.x, kind, limit);
        r.y = gated_act(gate.y, up.y, kind, limit);
        r.z = gated_act(gate.z, up.z, kind, limit);
        r.w = gated_act(gate.w, up.w, kind, limit);
        return r;
    };
    float4 v[ACT_KEEP];
    float mx = 0.0f;
    if (keep) {
#pragma unroll
        for (int j = 0; j < ACT_KEEP; j++) {
            const int c = (j * 256 + threadIdx.x) * 4;
            v[j] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (c < inter) {
                v[j] = act4(c);
                mx = fmaxf(fmaxf(mx, fmaxf(fabsf(v[j].x), fabsf(v[j].y))), fmaxf(fabsf(v[j].z), fabsf(v[j].w)));
            }
        }
    } else {
        for (int c = threadIdx.x * 4; c < inter; c += 256 * 4) {
            const float4 r = act4(c);
            mx = fmaxf(fmaxf(mx, fmaxf(fabsf(r.x), fabsf(r.y))), fmaxf(fabsf(r.z), fabsf(r.w)));
        }
    }
    mx = cta_max_256(mx, red);
    float f, inv;
    row_factor(mx, f, inv);
    if (keep) {
#pragma unroll
        for (int j = 0; j < ACT_KEEP; j++) {
            const int c = (j * 256 + threadIdx.x) * 4;
            if (c < inter) store_terms(v[j], f, ar + c, lo_off ? ar + lo_off + c : nullptr);
        }
    } else {
        for (int c = threadIdx.x * 4; c < inter; c += 256 * 4) store_terms(act4(c), f, ar + c, lo_off ? ar + lo_off + c : nullptr);
    }
    if (threadIdx.x == 0) unscale[row] = inv;
}

// The same with a warp per row (eight rows per CTA): inter = 128 * VPL, a lane keeps its VPL float4 of products.
template <int VPL>
__global__ void __launch_bounds__(256) moe_act_warp_kernel(const float* __restrict__ g, const int* __restrict__ src, int rows, __half* __restrict__ a,
                                                           float* __restrict__ unscale, size_t lo_off, int kind, float limit) {
    constexpr int INTER = 128 * VPL;
    pdl_launch_dependents();  // a dependent launch: the kernel behind may set itself up; nothing is read or written before the wait
    pdl_wait();
    const int row = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (row >= rows) return;
    __half* ar = a + (size_t)row * INTER;
    if (src && src[row] < 0) {
#pragma unroll
        for (int j = 0; j < VPL; j++) {
            const int c = (j * 32 + lane) * 4;
            *(uint2*)(ar + c) = make_uint2(0u, 0u);
            if (lo_off) *(uint2*)(ar + lo_off + c) = make_uint2(0u, 0u);
        }
        if (lane == 0) unscale[row] = 1.0f;
        return;
    }
    const float* gr = g + (size_t)row * 2 * INTER;
    float4 v[VPL];
    float mx = 0.0f;
#pragma unroll
    for (int j = 0; j < VPL; j++) {
        const int c = (j * 32 + lane) * 4;
        const float4 gate = *(const float4*)(gr + c), up = *(const float4*)(gr + INTER + c);
        v[j].x = gated_act(gate.x, up.x, kind, limit);
        v[j].y = gated_act(gate.y, up.y, kind, limit);
        v[j].z = gated_act(gate.z, up.z, kind, limit);
        v[j].w = gated_act(gate.w, up.w, kind, limit);
        mx = fmaxf(fmaxf(mx, fmaxf(fabsf(v[j].x), fabsf(v[j].y))), fmaxf(fabsf(v[j].z), fabsf(v[j].w)));
    }
    mx = warp_max(mx);
    float f, inv;
    row_factor(mx, f, inv);
#pragma unroll
    for (int j = 0; j < VPL; j++) {
        const int c = (j * 32 + lane) * 4;
        store_terms(v[j], f, ar + c, lo_off ? ar + lo_off + c : nullptr);
    }
    if (lane == 0) unscale[row] = inv;
}

// y[tok][c] += sum over the token's k routes, in order, of w * o[slot][c].
__global__ void moe_combine_kernel(const float* __restrict__ o, const int* __restrict__ slots, const float* __restrict__ w, int k, int h,
                                   float* __restrict__ y) {
    pdl_launch_dependents();  // a dependent launch: the kernel behind may set itself up; nothing is read or written before the wait
    pdl_wait();
    const int tok = blockIdx.y;
    const int c = (blockIdx.x * blockDim.x + threadIdx.x) * 4;  // four columns per thread (h is a multiple of 256)
    if (c >= h) return;
    float4 acc = *(const float4*)(y + (size_t)tok * h + c);
    for (int j = 0; j < k; j++) {
        const int slot = slots[(size_t)tok * k + j];
        const float wj = w[(size_t)tok * k + j];
        const float4 v = *(const float4*)(o + (size_t)slot * h + c);
        acc.x = __fadd_rn(acc.x, __fmul_rn(wj, v.x));
        acc.y = __fadd_rn(acc.y, __fmul_rn(wj, v.y));
        acc.z = __fadd_rn(acc.z, __fmul_rn(wj, v.z));
        acc.w = __fadd_rn(acc.w, __fmul_rn(wj, v.w));
    }
    *(float4*)(y + (size_t)tok * h + c) = acc;
}

// y[tok][c] += sum over the token's k routes, in order, of w * o[tok k + j][c]; the weights are kernel arguments.
__global__ void moe_combine_small_kernel(const float* __restrict__ o, SmallRoutes r, int k, int h, float* __restrict__ y) {
    pdl_launch_dependents();
    pdl_wait();
    const int tok = blockIdx.y;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= h) return;
    float acc = y[(size_t)tok * h + c];
    for (int j = 0; j < k; j++) {
        const int slot = tok * k + j;
        acc = __fadd_rn(acc, __fmul_rn(r.w[slot], o[(size_t)slot * h + c]));
    }
    y[(size_t)tok * h + c] = acc;
}

// out[r][h] = x[idx[r]][h] (f32 rows gathered by index), and the all-gather's rank-major blocks into column blocks.
__global__ void gather_rows_kernel(const float* __restrict__ x, const int* __restrict__ idx, int h, float* __restrict__ out) {
    const size_t r = blockIdx.x;
    const float4* in = (const float4*)(x + (size_t)idx[r] * h);
    float4* o = (float4*)(out + r * h);
    for (int i = threadIdx.x; i < h / 4; i += blockDim.x) o[i] = in[i];
}
__global__ void scatter_blocks_kernel(const float* __restrict__ g, int t, size_t nl, size_t world, float* __restrict__ y) {
    // g [world][t][nl] -> y [t][world * nl]
    const size_t n = (size_t)world * t * nl;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const size_t r = i / ((size_t)t * nl), rem = i - r * (size_t)t * nl, tok = rem / nl, c = rem - tok * nl;
        y[tok * world * nl + r * nl + c] = g[i];
    }
}

}  // namespace

cudaError_t launch_gather_rows(const float* x, const int* idx, size_t rows, size_t h, float* out, cudaStream_t st) {
    if (rows == 0) return cudaSuccess;
    if (h % 4) return cudaErrorInvalidValue;
    gather_rows_kernel<<<(unsigned)rows, 256, 0, st>>>(x, idx, (int)h, out);
    return cudaGetLastError();
}

cudaError_t launch_scatter_blocks(const float* gathered, size_t world, size_t t, size_t n_local, float* y, cudaStream_t st) {
    const size_t n = world * t * n_local;
    if (n == 0) return cudaSuccess;
    const unsigned grid = (unsigned)std::min<size_t>((n + 255) / 256, 148 * 16);
    scatter_blocks_kernel<<<grid, 256, 0, st>>>(gathered, (int)t, n_local, world, y);
    return cudaGetLastError();
}

cudaError_t launch_moe_combine_small(const float* o, const SmallRoutes& r, size_t t, size_t k, size_t h, float* y, cudaStream_t st, bool pdl) {
    if (t * k > GEMV_BATCH_MAX) return cudaErrorInvalidValue;
    dim3 grid((unsigned)((h + 255) / 256), (unsigned)t);
    return launch_k(moe_combine_small_kernel, grid, dim3(256), 0, st, pdl, o, r, (int)k, (int)h, y);
}

cudaError_t launch_route_topk(const float* logits, size_t t, size_t n, size_t k, int* ids, float* w, cudaStream_t st) {
    if (n > 2048 || k > 32 || k > n) return cudaErrorInvalidValue;
    route_topk_kernel<<<(unsigned)((t + 3) / 4), 128, 0, st>>>(logits, (int)t, (int)n, (int)k, ids, w);
    return cudaGetLastError();
}

cudaError_t launch_moe_gather(const float* x, const int* src, size_t rows, size_t h, void* xg, float* unscale, size_t lo_row0, cudaStream_t st) {
    if (h % 256 || h > (size_t)GATHER_KEEP * 1024) return cudaErrorInvalidValue;
    if (rows == 0) return cudaSuccess;
    const unsigned wgrid = (unsigned)((rows + 7) / 8);
    switch (rows >= 1024 ? h / 128 : 0) {  // many rows of a common width: a warp per row
        case 8: return launch_k(moe_gather_warp_kernel<8>, dim3(wgrid), dim3(256), 0, st, true, x, src, (int)rows, (__half*)xg, unscale, lo_row0 * h);
        case 16: return launch_k(moe_gather_warp_kernel<16>, dim3(wgrid), dim3(256), 0, st, true, x, src, (int)rows, (__half*)xg, unscale, lo_row0 * h);
        default: return launch_k(moe_gather_kernel, dim3((unsigned)rows), dim3(256), 0, st, true, x, src, (int)h, (__half*)xg, unscale, lo_row0 * h);
    }
}

cudaError_t launch_moe_act(const float* g, const int* src, size_t rows, size_t inter, void* a, float* unscale, size_t lo_row0, cudaStream_t st,
                           int kind, float limit) {
    if (inter % 256) return cudaErrorInvalidValue;
    if (rows == 0) return cudaSuccess;
    const unsigned wgrid = (unsigned)((rows + 7) / 8);
    switch (rows >= 1024 ? inter / 128 : 0) {  // many rows of a common width: a warp per row
        case 4: return launch_k(moe_act_warp_kernel<4>, dim3(wgrid), dim3(256), 0, st, true, g, src, (int)rows, (__half*)a, unscale, lo_row0 * inter, kind, limit);
        case 6: return launch_k(moe_act_warp_kernel<6>, dim3(wgrid), dim3(256), 0, st, true, g, src, (int)rows, (__half*)a, unscale, lo_row0 * inter, kind, limit);
        case 8: return launch_k(moe_act_warp_kernel<8>, dim3(wgrid), dim3(256), 0, st, true, g, src, (int)rows, (__half*)a, unscale, lo_row0 * inter, kind, limit);
        default: return launch_k(moe_act_kernel, dim3((unsigned)rows), dim3(256), 0, st, true, g, src, (int)inter, (__half*)a, unscale, lo_row0 * inter, kind, limit);
    }
}

cudaError_t launch_moe_combine(const float* o, const int* slots, const float* w, size_t t, size_t k, size_t h, float* y, cudaStream_t st) {
    dim3 grid((unsigned)((h / 4 + 255) / 256), (unsigned)t);
    return launch_k(moe_combine_kernel, grid, dim3(256), 0, st, true, o, slots, w, (int)k, (int)h, y);
}

}  // namespace b2
