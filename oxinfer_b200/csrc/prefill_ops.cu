// The non-matmul kernels of a prefill step: the ops of decode_ops.cu over many token rows at once
// (Backend::decode_plan_prefill, src/gpu.rs:283-289: "steps of up to `tokens` tokens on batched kernels, the activations
// kept on the device for the whole step"). Token row r of every activation sits `stride` floats behind row r - 1.
//
//   qk_rope_rows : per-head q / k norm, RoPE and cache append of every token (rope_head, the one-token arithmetic)
//   attend_rows  : causal attention of a tile of 64 query tokens of one or two query heads (of one KV head) over the cache,
//                  keys in tiles of 64 brought in by cp.async two stages deep: S = Q K^T and O += P V on mma.sync m16n8k16
//                  (f16 operands, f32 accumulators), softmax running in f32 registers. An f32 cache is first copied to f16.
//                  The reference's prefill attention is its f32 CPU kernel (attention_ext, src/model.rs:2214-2309) or
//                  attention_cached on the device; this one rounds q, k, v and the probabilities to f16, which the parity
//                  bound of the prefill plan covers.
//   glu_rows, rows_op : the element-wise ops
#include <cuda_fp16.h>

#include <algorithm>

#include "attend_core.cuh"

namespace b2 {

using namespace attend_core;

namespace {

__device__ __forceinline__ uint32_t pack_h2f(float a, float b) {
    const __half2 h = __floats2half2_rn(a, b);
    return *(const uint32_t*)&h;
}

template <typename T>
__global__ void __launch_bounds__(256) qk_rope_rows_kernel(const float* __restrict__ qkv, float* __restrict__ qo, size_t stride, T* __restrict__ kc,
                                                           T* __restrict__ vc, const float* __restrict__ qn, const float* __restrict__ kn,
                                                           const float* __restrict__ cs_table, const uint32_t* __restrict__ sp, DecRope p) {
    __shared__ float buf[256];
    __shared__ float red[32];
    const size_t off = (size_t)blockIdx.y * stride;
    rope_head<T>(blockIdx.x, threadIdx.x, sp[0] + blockIdx.y, sp[1], qkv + off, qo + off, kc, vc, qn, kn, cs_table, p, buf, red);
}

// RoPE and cache append without per-head norms: a warp per head of a token, lane l owning dimensions 4 l .. 4 l + 3 (and
// 128 + 4 l .. for heads of 256). The rotation is rope_head's arithmetic (unfused multiplies and adds), so the rows that
// reach the caches equal the one-token kernel's bit for bit. hd and half_rot are multiples of 4.
template <typename T>
__device__ __forceinline__ void store4(T* p, float4 v);
template <>
__device__ __forceinline__ void store4<float>(float* p, float4 v) { *(float4*)p = v; }
template <>
__device__ __forceinline__ void store4<__half>(__half* p, float4 v) {
    const __half2 a = __floats2half2_rn(v.x, v.y), b = __floats2half2_rn(v.z, v.w);
    *(uint2*)p = make_uint2(*(const uint32_t*)&a, *(const uint32_t*)&b);
}

template <typename T>
__global__ void __launch_bounds__(256) qk_rope_fast_kernel(const float* __restrict__ qkv, float* __restrict__ qo, size_t stride, uint32_t rows,
                                                           T* __restrict__ kc, T* __restrict__ vc, const float* __restrict__ cs_table,
                                                           const uint32_t* __restrict__ sp, DecRope p) {
    const uint32_t heads = p.nh + 2 * p.nkv;
    const uint32_t unit = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (unit >= rows * heads) return;
    const uint32_t tok = unit / heads, h = unit - tok * heads;
    const uint32_t kind = h < p.nh ? 0 : (h < p.nh + p.nkv ? 1 : 2);
    const uint32_t hh = kind == 0 ? h : (kind == 1 ? h - p.nh : h - p.nh - p.nkv);
    const uint32_t pos = sp[0] + tok, hd = p.hd, hr = p.half_rot;
    if (pos >= p.max_len) return;
    const float* src = qkv + (size_t)tok * stride + (kind == 0 ? hh * p.q_stride : (kind == 1 || p.v_from_k) ? p.k_off + hh * hd : p.v_off + hh * hd);
    const float* cs = cs_table + (size_t)(pos - sp[1]) * p.cs_stride + p.cs_off;
    const size_t at = ((size_t)hh * p.max_len + pos) * hd;
    for (uint32_t d0 = 4 * lane; d0 < hd; d0 += 128) {
        float4 v = *(const float4*)(src + d0);
        if (kind != 2 && d0 < 2 * hr) {
            if (p.interleaved) {  // pairs (2 j, 2 j + 1): both in this lane
                const uint32_t j = d0 >> 1;
                const float c0 = cs[j], s0 = cs[hr + j], c1 = cs[j + 1], s1 = cs[hr + j + 1];
                v = make_float4(__fsub_rn(__fmul_rn(v.x, c0), __fmul_rn(v.y, s0)), __fadd_rn(__fmul_rn(v.y, c0), __fmul_rn(v.x, s0)),
                                __fsub_rn(__fmul_rn(v.z, c1), __fmul_rn(v.w, s1)), __fadd_rn(__fmul_rn(v.w, c1), __fmul_rn(v.z, s1)));
            } else {  // pairs (j, j + hr): the partner's four values come from global memory again (L1)
                const bool first = d0 < hr;
                const uint32_t j = first ? d0 : d0 - hr;
                const float4 o = *(const float4*)(src + (first ? d0 + hr : d0 - hr));
                const float4 c = *(const float4*)(cs + j), s = *(const float4*)(cs + hr + j);
                if (first)
                    v = make_float4(__fsub_rn(__fmul_rn(v.x, c.x), __fmul_rn(o.x, s.x)), __fsub_rn(__fmul_rn(v.y, c.y), __fmul_rn(o.y, s.y)),
                                    __fsub_rn(__fmul_rn(v.z, c.z), __fmul_rn(o.z, s.z)), __fsub_rn(__fmul_rn(v.w, c.w), __fmul_rn(o.w, s.w)));
                else
                    v = make_float4(__fadd_rn(__fmul_rn(v.x, c.x), __fmul_rn(o.x, s.x)), __fadd_rn(__fmul_rn(v.y, c.y), __fmul_rn(o.y, s.y)),
                                    __fadd_rn(__fmul_rn(v.z, c.z), __fmul_rn(o.z, s.z)), __fadd_rn(__fmul_rn(v.w, c.w), __fmul_rn(o.w, s.w)));
            }
        }
        if (kind == 0) *(float4*)(qo + (size_t)tok * stride + hh * hd + d0) = v;
        else store4<T>((kind == 1 ? kc : vc) + at + d0, v);
    }
}

// RMS norm of many rows, one CTA of 256 threads per row, the row in registers between the passes (n <= 8192). With x16 the
// row also leaves as f16 operands of the GEMM behind it: multiplied by the power of two that brings its largest magnitude
// into [2^14, 2^15), the inverse factor in unscale[row] (what to_f16_rows_kernel makes of the f32 row).
constexpr int NORM_ROWS_V = 8;
__global__ void __launch_bounds__(256) norm_rows_kernel(const float* __restrict__ x, size_t x_stride, float* __restrict__ out, size_t out_stride,
                                                        const float* __restrict__ w, uint32_t n, float pre, float eps, int add,
                                                        __half* __restrict__ x16, float* __restrict__ unscale) {
    __shared__ float red[32];
    const size_t row = blockIdx.x;
    const float4* xr = (const float4*)(x + row * x_stride);
    float4* o = (float4*)(out + row * out_stride);
    const uint32_t n4 = n / 4;
    float4 v[NORM_ROWS_V];
    float s = 0.0f;
#pragma unroll
    for (int j = 0; j < NORM_ROWS_V; j++) {
        const uint32_t i = threadIdx.x + 256 * j;
        v[j] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        if (i < n4) {
            const float4 t = xr[i];
            v[j] = make_float4(t.x * pre, t.y * pre, t.z * pre, t.w * pre);
            s += v[j].x * v[j].x + v[j].y * v[j].y + v[j].z * v[j].z + v[j].w * v[j].w;
        }
    }
    const float k = 1.0f / sqrtf(block_sum(s, red) / (float)n + eps);
    float mx = 0.0f;
#pragma unroll
    for (int j = 0; j < NORM_ROWS_V; j++) {
        const uint32_t i = threadIdx.x + 256 * j;
        if (i < n4) {
            float4 t = make_float4(v[j].x * k, v[j].y * k, v[j].z * k, v[j].w * k);
            if (w) {
                const float4 ww = ((const float4*)w)[i];
                t = make_float4(t.x * ww.x, t.y * ww.y, t.z * ww.z, t.w * ww.w);
            }
            if (add) {
                const float4 a = o[i];
                t = make_float4(t.x + a.x, t.y + a.y, t.z + a.z, t.w + a.w);
            }
            o[i] = t;
            v[j] = t;
            mx = fmaxf(fmaxf(mx, fmaxf(fabsf(t.x), fabsf(t.y))), fmaxf(fabsf(t.z), fabsf(t.w)));
        }
    }
    if (!x16) return;
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, d));
    __syncthreads();  // red is read by every thread in block_sum above
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = mx;
    __syncthreads();
    mx = red[0];
#pragma unroll
    for (int i = 1; i < 8; i++) mx = fmaxf(mx, red[i]);
    float sc = 1.0f, inv = 1.0f;
    if (mx > 0.0f && mx < INFINITY) {
        int e;
        frexpf(mx, &e);
        const int up = min(100, max(-100, 15 - e));
        sc = ldexpf(1.0f, up);
        inv = ldexpf(1.0f, -up);
    }
    __half* h = x16 + row * n;
#pragma unroll
    for (int j = 0; j < NORM_ROWS_V; j++) {
        const uint32_t i = threadIdx.x + 256 * j;
        if (i < n4) *(uint2*)(h + 4 * (size_t)i) = make_uint2(pack_h2f(v[j].x * sc, v[j].y * sc), pack_h2f(v[j].z * sc, v[j].w * sc));
    }
    if (threadIdx.x == 0) unscale[row] = inv;
}

__global__ void __launch_bounds__(256) glu_rows_kernel(const float* __restrict__ g, size_t g_stride, const float* __restrict__ u, size_t u_stride,
                                                       float* __restrict__ out, size_t out_stride, uint32_t n, int gelu) {
    const uint32_t i = (blockIdx.x * blockDim.x + threadIdx.x) * 4;
    if (i >= n) return;
    const size_t r = blockIdx.y;
    const float4 a4 = *(const float4*)(g + r * g_stride + i), u4 = *(const float4*)(u + r * u_stride + i);
    const float a[4] = {a4.x, a4.y, a4.z, a4.w}, uu[4] = {u4.x, u4.y, u4.z, u4.w};
    float o[4];
#pragma unroll
    for (int j = 0; j < 4; j++) {  // the arithmetic of glu_kernel (decode_ops.cu)
        float v;
        if (gelu) {
            const float K2 = 2.0f * 0.7978846f;
            const float t = K2 * (a[j] + 0.044715f * a[j] * a[j] * a[j]);
            v = a[j] / (1.0f + expf(-t));
        } else {
            v = a[j] / (1.0f + expf(-a[j]));
        }
        o[j] = v * uu[j];
    }
    *(float4*)(out + r * out_stride + i) = make_float4(o[0], o[1], o[2], o[3]);
}

// act(g) * u of a whole row by one CTA, the row in registers (n <= 16384): the f32 result and, with x16, the f16 operand
// rows of the product behind it with their power-of-two row factor (what to_f16_rows_kernel makes of the f32 row), so that
// product needs no conversion launch and the row is not read again.
constexpr int GLU_ROW_V = 16;
__global__ void __launch_bounds__(256) glu_rows_f16_kernel(const float* __restrict__ g, size_t g_stride, const float* __restrict__ u, size_t u_stride,
                                                           float* __restrict__ out, size_t out_stride, uint32_t n, int gelu,
                                                           __half* __restrict__ x16, float* __restrict__ unscale) {
    __shared__ float red[8];
    const size_t r = blockIdx.x;
    const uint32_t n4 = n / 4;
    float4 v[GLU_ROW_V];
    float mx = 0.0f;
#pragma unroll
    for (int j = 0; j < GLU_ROW_V; j++) {
        const uint32_t i = threadIdx.x + 256 * j;
        v[j] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        if (i < n4) {
            const float4 a4 = ((const float4*)(g + r * g_stride))[i], u4 = ((const float4*)(u + r * u_stride))[i];
            const float a[4] = {a4.x, a4.y, a4.z, a4.w}, uu[4] = {u4.x, u4.y, u4.z, u4.w};
            float o[4];
#pragma unroll
            for (int e = 0; e < 4; e++) {  // the arithmetic of glu_rows_kernel
                float t;
                if (gelu) {
                    const float K2 = 2.0f * 0.7978846f;
                    const float z = K2 * (a[e] + 0.044715f * a[e] * a[e] * a[e]);
                    t = a[e] / (1.0f + expf(-z));
                } else {
                    t = a[e] / (1.0f + expf(-a[e]));
                }
                o[e] = t * uu[e];
                mx = fmaxf(mx, fabsf(o[e]));
            }
            v[j] = make_float4(o[0], o[1], o[2], o[3]);
            ((float4*)(out + r * out_stride))[i] = v[j];
        }
    }
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, d));
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = mx;
    __syncthreads();
    mx = red[0];
#pragma unroll
    for (int i = 1; i < 8; i++) mx = fmaxf(mx, red[i]);
    float sc = 1.0f, inv = 1.0f;
    if (mx > 0.0f && mx < INFINITY) {
        int e;
        frexpf(mx, &e);
        const int up = min(100, max(-100, 15 - e));
        sc = ldexpf(1.0f, up);
        inv = ldexpf(1.0f, -up);
    }
    __half* h = x16 + r * n;
#pragma unroll
    for (int j = 0; j < GLU_ROW_V; j++) {
        const uint32_t i = threadIdx.x + 256 * j;
        if (i < n4) *(uint2*)(h + 4 * (size_t)i) = make_uint2(pack_h2f(v[j].x * sc, v[j].y * sc), pack_h2f(v[j].z * sc, v[j].w * sc));
    }
    if (threadIdx.x == 0) unscale[r] = inv;
}

template <bool ADD>
__global__ void __launch_bounds__(256) rows_op_kernel(float* __restrict__ dst, size_t dst_stride, const float* __restrict__ src, size_t src_stride,
                                                      uint32_t n) {
    const uint32_t i = (blockIdx.x * blockDim.x + threadIdx.x) * 4;
    if (i >= n) return;
    const size_t r = blockIdx.y;
    float4 s = *(const float4*)(src + r * src_stride + i);
    float4* d = (float4*)(dst + r * dst_stride + i);
    if (ADD) {
        const float4 o = *d;
        s = make_float4(o.x + s.x, o.y + s.y, o.z + s.z, o.w + s.w);
    }
    *d = s;
}

// ---- attention over many query tokens ------------------------------------------------------------------------------
constexpr int PF_TILE = 64;      // query tokens per CTA, and keys per shared-memory tile

__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], const void* p) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t (&r)[4], const void* p) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void mma_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_h2(float a, float b) {
    const __half2 h = __floats2half2_rn(a, b);
    return *(const uint32_t*)&h;
}
// 16 bytes global -> shared without passing through registers; `bytes` 0 writes zeros instead.
__device__ __forceinline__ void cp_async_16(void* smem_dst, const void* src, uint32_t bytes) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(smem_dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// f32 cache rows [0, len) of every KV head -> an f16 copy with the same layout ([nkv][max_len][hd]).
__global__ void __launch_bounds__(256) kv_rows_to_f16_kernel(const float* __restrict__ src, __half* __restrict__ dst, uint32_t max_len, uint32_t len,
                                                             uint32_t hd4) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;  // a group of 4 values of the head's first `len` rows
    if (i >= len * hd4) return;
    const size_t at = ((size_t)blockIdx.y * max_len * hd4 + i) * 4;
    const float4 v = *(const float4*)(src + at);
    *(uint2*)(dst + at) = make_uint2(pack_h2(v.x, v.y), pack_h2(v.z, v.w));
}

template <int HD, int HEADS>
__host__ __device__ constexpr size_t attend_rows_smem() {
    return (size_t)(HEADS + 4) * PF_TILE * (HD + 8) * 2;  // the queries of HEADS heads, two stages of a key and a value tile
}

// Grid (query tiles, heads / HEADS). A CTA takes 64 query tokens of HEADS query heads that share a KV head (warp w: head
// w / 4, rows 16 (w % 4) ..); token row r (position sp[0] + r) attends to the keys 0 .. sp[0] + r of the cache (the keys of
// this step's tokens were appended by the RoPE kernel ahead), or to the last `window` of them. kc / vc: f16 rows. The key
// and value tiles arrive by cp.async, the next tile's copies in flight while the current one is multiplied.
template <int HD, int HEADS>
__global__ void __launch_bounds__(HEADS * 128) attend_rows_kernel(const float* __restrict__ q, float* __restrict__ out, size_t stride,
                                                                  const __half* __restrict__ kc, const __half* __restrict__ vc,
                                                                  const uint32_t* __restrict__ sp, DecAttn p, uint32_t rows) {
    extern __shared__ __align__(16) uint8_t smem[];
    constexpr int P = HD + 8;  // halves per shared-memory row: rows 16 bytes apart modulo 128, so ldmatrix reads without conflicts
    constexpr int THREADS = HEADS * 128;
    __half* Qs = (__half*)smem;                 // [HEADS][64][P]
    __half* KV = Qs + HEADS * PF_TILE * P;      // [stage][K | V][64][P]
    const uint32_t pos0 = sp[0];
    const uint32_t qt = gridDim.x - 1 - blockIdx.x;  // the tiles with the most keys first
    const uint32_t head0 = blockIdx.y * HEADS, kvh = head0 / (p.nh / p.nkv);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, c = lane & 3;
    const int wh = warp >> 2, wr = warp & 3;  // the warp's head within the CTA, and its block of 16 query rows
    const uint32_t r0 = qt * PF_TILE;
    const uint32_t last_row = min(r0 + PF_TILE, rows) - 1;
    const uint32_t qp_first = pos0 + r0, qp_last = pos0 + last_row;
    const uint32_t lo = (p.window != 0 && qp_first + 1 > p.window) ? qp_first + 1 - p.window : 0;
    const uint32_t tile_first = lo / PF_TILE, tile_last = qp_last / PF_TILE;
    auto issue = [&](uint32_t tk, int stage) {  // every thread: its share of the 2 x 64 rows of HD halves
        const uint32_t j0 = tk * PF_TILE;
        __half* Ks = KV + (size_t)stage * 2 * PF_TILE * P;
        __half* Vs = Ks + PF_TILE * P;
        for (int i = tid; i < PF_TILE * (HD / 8); i += THREADS) {
            const int r = i / (HD / 8), d8 = i % (HD / 8);
            const bool in = j0 + r <= qp_last;  // rows behind the last query's position: zeros (never a stale NaN under a zero weight)
            const size_t at = ((size_t)kvh * p.max_len + (in ? j0 + r : 0)) * HD + d8 * 8;
            cp_async_16(Ks + r * P + d8 * 8, kc + at, in ? 16u : 0u);
            cp_async_16(Vs + r * P + d8 * 8, vc + at, in ? 16u : 0u);
        }
        cp_async_commit();
    };
    issue(tile_first, 0);
    for (int i = tid; i < HEADS * PF_TILE * (HD / 4); i += THREADS) {
        const int hh = i / (PF_TILE * (HD / 4)), r = (i / (HD / 4)) % PF_TILE, d4 = i % (HD / 4);
        uint2 h = make_uint2(0u, 0u);
        if (r0 + r < rows) {
            const float4 v = *(const float4*)(q + (size_t)(r0 + r) * stride + (head0 + hh) * HD + d4 * 4);
            h = make_uint2(pack_h2(v.x, v.y), pack_h2(v.z, v.w));
        }
        *(uint2*)(Qs + (hh * PF_TILE + r) * P + d4 * 4) = h;
    }
    float o[HD / 8][4];
#pragma unroll
    for (int nb = 0; nb < HD / 8; nb++) o[nb][0] = o[nb][1] = o[nb][2] = o[nb][3] = 0.0f;
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.0f, 0.0f};
    const uint32_t my_qp[2] = {pos0 + r0 + wr * 16 + g, pos0 + r0 + wr * 16 + g + 8};
    const __half* Qw = Qs + (wh * PF_TILE + wr * 16 + (lane & 15)) * P + (lane >> 4) * 8;
    for (uint32_t tk = tile_first; tk <= tile_last; tk++) {
        const int stage = (int)((tk - tile_first) & 1);
        if (tk < tile_last) {
            issue(tk + 1, stage ^ 1);  // (the barrier at the end of the previous round freed that stage)
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        const __half* Ks = KV + (size_t)stage * 2 * PF_TILE * P;
        const __half* Vs = Ks + PF_TILE * P;
        const uint32_t j0 = tk * PF_TILE;
        float s[PF_TILE / 8][4];
#pragma unroll
        for (int nb = 0; nb < PF_TILE / 8; nb++) s[nb][0] = s[nb][1] = s[nb][2] = s[nb][3] = 0.0f;
#pragma unroll
        for (int ks = 0; ks < HD / 16; ks++) {
            uint32_t qa[4];
            ldsm_x4(qa, Qw + ks * 16);
#pragma unroll
            for (int nb2 = 0; nb2 < PF_TILE / 16; nb2++) {
                uint32_t b[4];
                ldsm_x4(b, Ks + (nb2 * 16 + (lane & 7) + 8 * (lane >> 4)) * P + ks * 16 + 8 * ((lane >> 3) & 1));
                mma_16816(s[2 * nb2], qa, b[0], b[1]);
                mma_16816(s[2 * nb2 + 1], qa, b[2], b[3]);
            }
        }
        float mx[2] = {-INFINITY, -INFINITY};
        // only tiles that reach past the first query's position or start inside the window's edge need the mask
        const bool masked = j0 + PF_TILE - 1 > qp_first || (p.window != 0 && j0 + p.window <= qp_last);
#pragma unroll
        for (int nb = 0; nb < PF_TILE / 8; nb++) {
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const int row = e >> 1;
                float v = s[nb][e] * p.scale;
                if (masked) {
                    const uint32_t j = j0 + nb * 8 + 2 * c + (e & 1), qp = my_qp[row];
                    const bool ok = j <= qp && (p.window == 0 || j + p.window > qp);
                    v = ok ? v : -INFINITY;
                }
                s[nb][e] = v;
                mx[row] = fmaxf(mx[row], v);
            }
        }
        float m_use[2];
#pragma unroll
        for (int row = 0; row < 2; row++) {
            mx[row] = fmaxf(mx[row], __shfl_xor_sync(0xffffffffu, mx[row], 1));
            mx[row] = fmaxf(mx[row], __shfl_xor_sync(0xffffffffu, mx[row], 2));
            const float m_new = fmaxf(m[row], mx[row]);
            m_use[row] = m_new == -INFINITY ? 0.0f : m_new;  // nothing but masked keys so far
            const float alpha = __expf(m[row] - m_use[row]);
            m[row] = m_new;
            l[row] *= alpha;
#pragma unroll
            for (int nb = 0; nb < HD / 8; nb++) {
                o[nb][2 * row] *= alpha;
                o[nb][2 * row + 1] *= alpha;
            }
        }
#pragma unroll
        for (int nb = 0; nb < PF_TILE / 8; nb++) {
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const float pe = __expf(s[nb][e] - m_use[e >> 1]);
                s[nb][e] = pe;
                l[e >> 1] += pe;
            }
        }
#pragma unroll
        for (int kk = 0; kk < PF_TILE / 16; kk++) {
            const uint32_t pa[4] = {pack_h2(s[2 * kk][0], s[2 * kk][1]), pack_h2(s[2 * kk][2], s[2 * kk][3]), pack_h2(s[2 * kk + 1][0], s[2 * kk + 1][1]),
                                    pack_h2(s[2 * kk + 1][2], s[2 * kk + 1][3])};
#pragma unroll
            for (int nb2 = 0; nb2 < HD / 16; nb2++) {
                uint32_t b[4];
                ldsm_x4_trans(b, Vs + (kk * 16 + (lane & 7) + 8 * ((lane >> 3) & 1)) * P + nb2 * 16 + 8 * (lane >> 4));
                mma_16816(o[2 * nb2], pa, b[0], b[1]);
                mma_16816(o[2 * nb2 + 1], pa, b[2], b[3]);
            }
        }
        __syncthreads();  // every warp is done with this stage before the next round's copies land in it
    }
#pragma unroll
    for (int row = 0; row < 2; row++) {
        l[row] += __shfl_xor_sync(0xffffffffu, l[row], 1);
        l[row] += __shfl_xor_sync(0xffffffffu, l[row], 2);
        const uint32_t r = r0 + wr * 16 + g + 8 * row;
        if (r >= rows) continue;
        const float inv = l[row] > 0.0f ? 1.0f / l[row] : 0.0f;
        float* dst = out + (size_t)r * stride + (head0 + wh) * HD + 2 * c;
#pragma unroll
        for (int nb = 0; nb < HD / 8; nb++) *(float2*)(dst + nb * 8) = make_float2(o[nb][2 * row] * inv, o[nb][2 * row + 1] * inv);
    }
}

template <int HD, int HEADS>
cudaError_t attend_rows_t(const float* q, float* out, size_t stride, const __half* kc, const __half* vc, const uint32_t* sp, const DecAttn& p,
                          uint32_t rows, cudaStream_t st) {
    constexpr size_t smem = attend_rows_smem<HD, HEADS>();
    if (cudaError_t e = ensure_dynamic_smem((const void*)attend_rows_kernel<HD, HEADS>, smem); e != cudaSuccess) return e;
    attend_rows_kernel<HD, HEADS><<<dim3((rows + PF_TILE - 1) / PF_TILE, p.nh / HEADS), HEADS * 128, smem, st>>>(q, out, stride, kc, vc, sp, p, rows);
    return cudaGetLastError();
}

}  // namespace

cudaError_t launch_qk_rope_rows(const float* qkv, float* qo, size_t stride, uint32_t rows, void* kc, void* vc, int kv_f16, const float* qn,
                                const float* kn, const float* cs, const uint32_t* sp, const DecRope& p, cudaStream_t st) {
    if (p.hd > 256 || p.hd % 32 || 2 * p.half_rot > p.hd || rows == 0 || rows > 65535) return cudaErrorInvalidValue;
    // (the fast kernel reads a rotation partner's values from the input again: input and output must not overlap)
    const size_t in_extent = std::max<size_t>((size_t)(p.nh - 1) * p.q_stride + p.hd, std::max<size_t>(p.k_off, p.v_off) + (size_t)p.nkv * p.hd);
    const bool apart = qo + (size_t)p.nh * p.hd <= qkv || qkv + in_extent <= qo;
    if (apart && !qn && !kn && !p.v_norm && p.half_rot % 4 == 0 && stride % 4 == 0 && p.q_stride % 4 == 0 && p.k_off % 4 == 0 && p.v_off % 4 == 0 &&
        p.cs_off % 4 == 0 && p.cs_stride % 4 == 0 && (((uintptr_t)qkv | (uintptr_t)qo | (uintptr_t)cs) & 15) == 0) {
        const size_t units = (size_t)rows * (p.nh + 2 * p.nkv);
        const unsigned grid = (unsigned)((units + 7) / 8);
        if (kv_f16)
            qk_rope_fast_kernel<__half><<<grid, 256, 0, st>>>(qkv, qo, stride, rows, (__half*)kc, (__half*)vc, cs, sp, p);
        else
            qk_rope_fast_kernel<float><<<grid, 256, 0, st>>>(qkv, qo, stride, rows, (float*)kc, (float*)vc, cs, sp, p);
        return cudaGetLastError();
    }
    const dim3 grid(p.nh + 2 * p.nkv, rows);
    if (kv_f16)
        qk_rope_rows_kernel<__half><<<grid, p.hd, 0, st>>>(qkv, qo, stride, (__half*)kc, (__half*)vc, qn, kn, cs, sp, p);
    else
        qk_rope_rows_kernel<float><<<grid, p.hd, 0, st>>>(qkv, qo, stride, (float*)kc, (float*)vc, qn, kn, cs, sp, p);
    return cudaGetLastError();
}

bool attend_rows_supports(uint32_t nh, uint32_t nkv, uint32_t hd) { return nkv != 0 && nh % nkv == 0 && (hd == 64 || hd == 128); }

size_t attend_rows_scratch_bytes(uint32_t nkv, uint32_t max_len, uint32_t hd, int kv_f16) {
    return kv_f16 ? 0 : (size_t)2 * nkv * max_len * hd * 2;
}

cudaError_t launch_attend_rows(const float* q, float* out, size_t stride, uint32_t rows, const void* kc, const void* vc, int kv_f16, void* scratch,
                               uint32_t len, const uint32_t* sp, const DecAttn& p, cudaStream_t st) {
    if (!attend_rows_supports(p.nh, p.nkv, p.hd) || rows == 0 || stride % 4 || ((uintptr_t)q & 15) || ((uintptr_t)out & 15) || len > p.max_len)
        return cudaErrorInvalidValue;
    const __half *kh = (const __half*)kc, *vh = (const __half*)vc;
    if (!kv_f16) {  // an f16 copy of the rows the step reads (the kernel's operands are f16 either way)
        if (!scratch) return cudaErrorInvalidValue;
        __half* k16 = (__half*)scratch;
        __half* v16 = k16 + (size_t)p.nkv * p.max_len * p.hd;
        const dim3 grid((len * (p.hd / 4) + 255) / 256, p.nkv);
        kv_rows_to_f16_kernel<<<grid, 256, 0, st>>>((const float*)kc, k16, p.max_len, len, p.hd / 4);
        kv_rows_to_f16_kernel<<<grid, 256, 0, st>>>((const float*)vc, v16, p.max_len, len, p.hd / 4);
        if (cudaError_t e = cudaGetLastError(); e != cudaSuccess) return e;
        kh = k16;
        vh = v16;
    }
    const bool two = (p.nh / p.nkv) % 2 == 0;  // two query heads of a KV head share a CTA's key and value tiles
    if (p.hd == 64) return two ? attend_rows_t<64, 2>(q, out, stride, kh, vh, sp, p, rows, st) : attend_rows_t<64, 1>(q, out, stride, kh, vh, sp, p, rows, st);
    return two ? attend_rows_t<128, 2>(q, out, stride, kh, vh, sp, p, rows, st) : attend_rows_t<128, 1>(q, out, stride, kh, vh, sp, p, rows, st);
}

bool norm_rows_supports(uint32_t n, const float* x, const float* out, const float* w, size_t x_stride, size_t out_stride) {
    return n % 4 == 0 && n <= 1024 * NORM_ROWS_V && x_stride % 4 == 0 && out_stride % 4 == 0 && (((uintptr_t)x | (uintptr_t)out | (uintptr_t)w) & 15) == 0;
}

cudaError_t launch_norm_rows(const float* x, size_t x_stride, float* out, size_t out_stride, const float* w, const DecNorm& p, uint32_t rows,
                             void* x16, float* unscale, cudaStream_t st) {
    if (!norm_rows_supports(p.n, x, out, w, x_stride, out_stride) || rows == 0 || (x16 && (p.n % 8 || ((uintptr_t)x16 & 15)))) return cudaErrorInvalidValue;
    norm_rows_kernel<<<rows, 256, 0, st>>>(x, x_stride, out, out_stride, w, p.n, p.pre, p.eps, (int)p.add, (__half*)x16, unscale);
    return cudaGetLastError();
}

bool glu_rows_f16_supports(uint32_t n) { return n % 8 == 0 && n <= 1024 * GLU_ROW_V; }

cudaError_t launch_glu_rows(const float* g, size_t g_stride, const float* u, size_t u_stride, float* out, size_t out_stride, uint32_t n,
                            uint32_t rows, int gelu, cudaStream_t st, void* x16, float* unscale) {
    if (n % 4 || g_stride % 4 || u_stride % 4 || out_stride % 4 || rows == 0 || rows > 65535 || (((uintptr_t)g | (uintptr_t)u | (uintptr_t)out) & 15))
        return cudaErrorInvalidValue;
    if (x16) {
        if (!glu_rows_f16_supports(n) || ((uintptr_t)x16 & 15)) return cudaErrorInvalidValue;
        glu_rows_f16_kernel<<<rows, 256, 0, st>>>(g, g_stride, u, u_stride, out, out_stride, n, gelu, (__half*)x16, unscale);
        return cudaGetLastError();
    }
    glu_rows_kernel<<<dim3((n / 4 + 255) / 256, rows), 256, 0, st>>>(g, g_stride, u, u_stride, out, out_stride, n, gelu);
    return cudaGetLastError();
}

cudaError_t launch_rows_op(float* dst, size_t dst_stride, const float* src, size_t src_stride, uint32_t n, uint32_t rows, bool add,
                           cudaStream_t st) {
    if (n % 4 || dst_stride % 4 || src_stride % 4 || rows == 0 || rows > 65535 || (((uintptr_t)dst | (uintptr_t)src) & 15)) return cudaErrorInvalidValue;
    const dim3 grid((n / 4 + 255) / 256, rows);
    if (add)
        rows_op_kernel<true><<<grid, 256, 0, st>>>(dst, dst_stride, src, src_stride, n);
    else
        rows_op_kernel<false><<<grid, 256, 0, st>>>(dst, dst_stride, src, src_stride, n);
    return cudaGetLastError();
}

}  // namespace b2
