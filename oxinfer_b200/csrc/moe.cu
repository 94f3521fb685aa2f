// Element-wise pieces of the routed-expert layer around the grouped tensor-core GEMM:
//   route_topk   : top-k of the router logits with the reference's order and weights
//                  (route_top_k, src/moe.rs:180-193; dtopk, src/cuda_decode.cu:285-312)
//   moe_gather   : token rows -> per-expert segments, f32 -> f16, pad rows zero
//                  (moe_gather, src/cuda.rs:293-297)
//   moe_act      : act(gate) * up over the fused gate_up output, to f16 for the down projection
//                  (moe_act, src/cuda.rs:300-316; SiLU with expf as on the reference's GPU path)
//   moe_combine  : y[t] += sum_j w_j * o[slot(t, j)] in route order, multiply and add unfused
//                  (moe_combine, src/cuda.rs:319-330)
#include "kernels.h"

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

// xg[row][h] (f16) = x[src[row]][h] (f32), zeros where src[row] < 0. One CTA per row.
__global__ void moe_gather_kernel(const float* __restrict__ x, const int* __restrict__ src, int h, __half* __restrict__ xg) {
    const int row = blockIdx.x;
    const int s = src[row];
    uint2* o = (uint2*)(xg + (size_t)row * h);  // four halves at a time (h is a multiple of 256)
    if (s < 0) {
        for (int i = threadIdx.x; i < h / 4; i += blockDim.x) o[i] = make_uint2(0u, 0u);
        return;
    }
    const float4* in = (const float4*)(x + (size_t)s * h);
    for (int i = threadIdx.x; i < h / 4; i += blockDim.x) {
        const float4 v = in[i];
        const __half2 lo = __floats2half2_rn(v.x, v.y), hi = __floats2half2_rn(v.z, v.w);
        o[i] = make_uint2(*(const uint32_t*)&lo, *(const uint32_t*)&hi);
    }
}

// a[row][inter] (f16) = silu(g[row][c]) * g[row][inter + c] / scale[row] over the fused gate_up output
// g [rows][2 inter] (f32). scale[row] is a power of two (1 unless the row would leave f16's range) that the
// combine step multiplies back, so the down projection sees operands it can represent. src[row] < 0 marks a padding row
// (src may be null: no padding). One CTA per row; the row is read
// once (a thread keeps its products in registers between the maximum and the store) when inter <= 256 * 4 * ACT_KEEP.
constexpr int ACT_KEEP = 2;
__global__ void __launch_bounds__(256) moe_act_kernel(const float* __restrict__ g, const int* __restrict__ src, int inter, __half* __restrict__ a,
                                                      float* __restrict__ scale) {
    __shared__ float red[8];
    const size_t row = blockIdx.x;
    if (src && src[row] < 0) {  // a padding row of an expert's last tile: its products are zero, nothing to read
        for (int c = threadIdx.x * 4; c < inter; c += 256 * 4) *(uint2*)(a + row * inter + c) = make_uint2(0u, 0u);
        if (threadIdx.x == 0) scale[row] = 1.0f;
        return;
    }
    const float* gr = g + row * 2 * (size_t)inter;
    const bool keep = inter <= 256 * 4 * ACT_KEEP;  // inter is a multiple of 256: whole float4 per thread
    float4 v[ACT_KEEP];
    float mx = 0.0f;
    if (keep) {
#pragma unroll
        for (int j = 0; j < ACT_KEEP; j++) {
            const int c = (j * 256 + threadIdx.x) * 4;
            v[j] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (c < inter) {
                const float4 gate = *(const float4*)(gr + c), up = *(const float4*)(gr + inter + c);
                v[j].x = gate.x / (1.0f + expf(-gate.x)) * up.x;
                v[j].y = gate.y / (1.0f + expf(-gate.y)) * up.y;
                v[j].z = gate.z / (1.0f + expf(-gate.z)) * up.z;
                v[j].w = gate.w / (1.0f + expf(-gate.w)) * up.w;
                mx = fmaxf(fmaxf(mx, fmaxf(fabsf(v[j].x), fabsf(v[j].y))), fmaxf(fabsf(v[j].z), fabsf(v[j].w)));
            }
        }
    } else {
        for (int c = threadIdx.x; c < inter; c += 256) {
            float gate = gr[c], up = gr[inter + c];
            mx = fmaxf(mx, fabsf(gate / (1.0f + expf(-gate)) * up));
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = mx;
    __syncthreads();
    mx = red[0];
#pragma unroll
    for (int i = 1; i < 8; i++) mx = fmaxf(mx, red[i]);
    float sc = 1.0f;
    if (mx > 32768.0f && mx < INFINITY) sc = exp2f(ceilf(log2f(mx * (1.0f / 32768.0f))));
    const float inv = 1.0f / sc;  // exact: a power of two
    if (keep) {
#pragma unroll
        for (int j = 0; j < ACT_KEEP; j++) {
            const int c = (j * 256 + threadIdx.x) * 4;
            if (c < inter) {
                const __half2 lo = __floats2half2_rn(v[j].x * inv, v[j].y * inv), hi = __floats2half2_rn(v[j].z * inv, v[j].w * inv);
                *(uint2*)(a + row * inter + c) = make_uint2(*(const uint32_t*)&lo, *(const uint32_t*)&hi);
            }
        }
    } else {
        for (int c = threadIdx.x; c < inter; c += 256) {
            float gate = gr[c], up = gr[inter + c];
            a[row * inter + c] = __float2half_rn(gate / (1.0f + expf(-gate)) * up * inv);
        }
    }
    if (threadIdx.x == 0) scale[row] = sc;
}

// y[tok][c] += sum over the token's k routes, in order, of w * o[slot][c].
__global__ void moe_combine_kernel(const float* __restrict__ o, const float* __restrict__ scale, const int* __restrict__ slots,
                                   const float* __restrict__ w, int k, int h, float* __restrict__ y) {
    const int tok = blockIdx.y;
    const int c = (blockIdx.x * blockDim.x + threadIdx.x) * 4;  // four columns per thread (h is a multiple of 256)
    if (c >= h) return;
    float4 acc = *(const float4*)(y + (size_t)tok * h + c);
    for (int j = 0; j < k; j++) {
        const int slot = slots[(size_t)tok * k + j];
        const float wj = w[(size_t)tok * k + j], sc = scale[slot];
        const float4 v = *(const float4*)(o + (size_t)slot * h + c);
        acc.x = __fadd_rn(acc.x, __fmul_rn(wj, v.x * sc));
        acc.y = __fadd_rn(acc.y, __fmul_rn(wj, v.y * sc));
        acc.z = __fadd_rn(acc.z, __fmul_rn(wj, v.z * sc));
        acc.w = __fadd_rn(acc.w, __fmul_rn(wj, v.w * sc));
    }
    *(float4*)(y + (size_t)tok * h + c) = acc;
}

// y[tok][c] += sum over the token's k routes, in order, of w * o[tok k + j][c]; the weights are kernel arguments.
__global__ void moe_combine_small_kernel(const float* __restrict__ o, SmallRoutes r, int k, int h, float* __restrict__ y) {
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

}  // namespace

cudaError_t launch_moe_combine_small(const float* o, const SmallRoutes& r, size_t t, size_t k, size_t h, float* y, cudaStream_t st) {
    if (t * k > GEMV_BATCH_MAX) return cudaErrorInvalidValue;
    dim3 grid((unsigned)((h + 255) / 256), (unsigned)t);
    moe_combine_small_kernel<<<grid, 256, 0, st>>>(o, r, (int)k, (int)h, y);
    return cudaGetLastError();
}

cudaError_t launch_route_topk(const float* logits, size_t t, size_t n, size_t k, int* ids, float* w, cudaStream_t st) {
    if (n > 2048 || k > 32 || k > n) return cudaErrorInvalidValue;
    route_topk_kernel<<<(unsigned)((t + 3) / 4), 128, 0, st>>>(logits, (int)t, (int)n, (int)k, ids, w);
    return cudaGetLastError();
}

cudaError_t launch_moe_gather(const float* x, const int* src, size_t rows, size_t h, void* xg, cudaStream_t st) {
    moe_gather_kernel<<<(unsigned)rows, 256, 0, st>>>(x, src, (int)h, (__half*)xg);
    return cudaGetLastError();
}

cudaError_t launch_moe_act(const float* g, const int* src, size_t rows, size_t inter, void* a, float* scale, cudaStream_t st) {
    moe_act_kernel<<<(unsigned)rows, 256, 0, st>>>(g, src, (int)inter, (__half*)a, scale);
    return cudaGetLastError();
}

cudaError_t launch_moe_combine(const float* o, const float* scale, const int* slots, const float* w, size_t t, size_t k, size_t h, float* y,
                               cudaStream_t st) {
    dim3 grid((unsigned)((h / 4 + 255) / 256), (unsigned)t);
    moe_combine_kernel<<<grid, 256, 0, st>>>(o, scale, slots, w, (int)k, (int)h, y);
    return cudaGetLastError();
}

}  // namespace b2
