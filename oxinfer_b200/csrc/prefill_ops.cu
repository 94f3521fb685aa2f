// The non-matmul kernels of a prefill step: the ops of decode_ops.cu over many token rows at once
// (Backend::decode_plan_prefill, src/gpu.rs:283-289: "steps of up to `tokens` tokens on batched kernels, the activations
// kept on the device for the whole step"). Token row r of every activation sits `stride` floats behind row r - 1.
//
//   qk_rope_rows : per-head q / k norm, RoPE and cache append of every token (rope_head, the one-token arithmetic)
//   attend_rows  : causal attention of a tile of 64 query tokens of one head over the cache, keys in tiles of 64:
//                  S = Q K^T and O += P V on mma.sync m16n8k16 (f16 operands, f32 accumulators), softmax running in f32
//                  registers. The reference's prefill attention is its f32 CPU kernel (attention_ext,
//                  src/model.rs:2214-2309) or attention_cached on the device; this one rounds q, k, v and the
//                  probabilities to f16, which the parity bound of the prefill plan covers.
//   glu_rows, rows_add / rows_copy : the element-wise ops
#include <cuda_fp16.h>

#include "attend_core.cuh"

namespace b2 {

using namespace attend_core;

namespace {

template <typename T>
__global__ void __launch_bounds__(256) qk_rope_rows_kernel(const float* __restrict__ qkv, float* __restrict__ qo, size_t stride, T* __restrict__ kc,
                                                           T* __restrict__ vc, const float* __restrict__ qn, const float* __restrict__ kn,
                                                           const float* __restrict__ cs_table, const uint32_t* __restrict__ sp, DecRope p) {
    __shared__ float buf[256];
    __shared__ float red[32];
    const size_t off = (size_t)blockIdx.y * stride;
    rope_head<T>(blockIdx.x, threadIdx.x, sp[0] + blockIdx.y, sp[1], qkv + off, qo + off, kc, vc, qn, kn, cs_table, p, buf, red);
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
constexpr int PF_THREADS = 128;  // four warps of 16 query rows

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
__device__ __forceinline__ uint2 to_h4(float4 v) { return make_uint2(pack_h2(v.x, v.y), pack_h2(v.z, v.w)); }
__device__ __forceinline__ uint2 row4_as_half(const float* p) { return to_h4(*(const float4*)p); }
__device__ __forceinline__ uint2 row4_as_half(const __half* p) { return *(const uint2*)p; }

template <int HD>
__host__ __device__ constexpr size_t attend_rows_smem() {
    return (size_t)3 * PF_TILE * (HD + 8) * 2;
}

// Grid (query tiles, heads). Token row r (position sp[0] + r) attends to the keys 0 .. sp[0] + r of its KV head's cache
// (the keys of this step's tokens were appended by the RoPE kernel ahead), or to the last `window` of them.
template <int HD, typename T>
__global__ void __launch_bounds__(PF_THREADS) attend_rows_kernel(const float* __restrict__ q, float* __restrict__ out, size_t stride,
                                                                 const T* __restrict__ kc, const T* __restrict__ vc,
                                                                 const uint32_t* __restrict__ sp, DecAttn p, uint32_t rows) {
    extern __shared__ __align__(16) uint8_t smem[];
    constexpr int P = HD + 8;  // halves per shared-memory row: rows 16 bytes apart modulo 128, so ldmatrix reads without conflicts
    __half* Qs = (__half*)smem;
    __half* Ks = Qs + PF_TILE * P;
    __half* Vs = Ks + PF_TILE * P;
    const uint32_t pos0 = sp[0];
    const uint32_t qt = gridDim.x - 1 - blockIdx.x;  // the tiles with the most keys first
    const uint32_t head = blockIdx.y, kvh = head / (p.nh / p.nkv);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, c = lane & 3;
    const uint32_t r0 = qt * PF_TILE;
    for (int i = tid; i < PF_TILE * (HD / 4); i += PF_THREADS) {
        const int r = i / (HD / 4), d4 = i % (HD / 4);
        uint2 h = make_uint2(0u, 0u);
        if (r0 + r < rows) h = row4_as_half(q + (size_t)(r0 + r) * stride + head * HD + d4 * 4);
        *(uint2*)(Qs + r * P + d4 * 4) = h;
    }
    __syncthreads();
    uint32_t qa[HD / 16][4];
#pragma unroll
    for (int ks = 0; ks < HD / 16; ks++) ldsm_x4(qa[ks], Qs + (warp * 16 + (lane & 15)) * P + ks * 16 + (lane >> 4) * 8);
    float o[HD / 8][4];
#pragma unroll
    for (int nb = 0; nb < HD / 8; nb++) o[nb][0] = o[nb][1] = o[nb][2] = o[nb][3] = 0.0f;
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.0f, 0.0f};
    const uint32_t last_row = min(r0 + PF_TILE, rows) - 1;
    const uint32_t qp_first = pos0 + r0, qp_last = pos0 + last_row;
    const uint32_t lo = (p.window != 0 && qp_first + 1 > p.window) ? qp_first + 1 - p.window : 0;
    const uint32_t my_qp[2] = {pos0 + r0 + warp * 16 + g, pos0 + r0 + warp * 16 + g + 8};
    for (uint32_t tk = lo / PF_TILE; tk <= qp_last / PF_TILE; tk++) {
        const uint32_t j0 = tk * PF_TILE;
        __syncthreads();  // every warp is done with the previous tile
        for (int i = tid; i < PF_TILE * (HD / 4); i += PF_THREADS) {
            const int r = i / (HD / 4), d4 = i % (HD / 4);
            uint2 kh = make_uint2(0u, 0u), vh = make_uint2(0u, 0u);
            if (j0 + r <= qp_last) {
                const size_t at = ((size_t)kvh * p.max_len + j0 + r) * HD + d4 * 4;
                kh = row4_as_half(kc + at);
                vh = row4_as_half(vc + at);
            }
            *(uint2*)(Ks + r * P + d4 * 4) = kh;
            *(uint2*)(Vs + r * P + d4 * 4) = vh;
        }
        __syncthreads();
        float s[PF_TILE / 8][4];
#pragma unroll
        for (int nb = 0; nb < PF_TILE / 8; nb++) s[nb][0] = s[nb][1] = s[nb][2] = s[nb][3] = 0.0f;
#pragma unroll
        for (int ks = 0; ks < HD / 16; ks++) {
#pragma unroll
            for (int nb2 = 0; nb2 < PF_TILE / 16; nb2++) {
                uint32_t b[4];
                ldsm_x4(b, Ks + (nb2 * 16 + (lane & 7) + 8 * (lane >> 4)) * P + ks * 16 + 8 * ((lane >> 3) & 1));
                mma_16816(s[2 * nb2], qa[ks], b[0], b[1]);
                mma_16816(s[2 * nb2 + 1], qa[ks], b[2], b[3]);
            }
        }
        float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int nb = 0; nb < PF_TILE / 8; nb++) {
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const int row = e >> 1;
                const uint32_t j = j0 + nb * 8 + 2 * c + (e & 1), qp = my_qp[row];
                const bool ok = j <= qp && (p.window == 0 || j + p.window > qp);
                const float v = ok ? s[nb][e] * p.scale : -INFINITY;
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
    }
#pragma unroll
    for (int row = 0; row < 2; row++) {
        l[row] += __shfl_xor_sync(0xffffffffu, l[row], 1);
        l[row] += __shfl_xor_sync(0xffffffffu, l[row], 2);
        const uint32_t r = r0 + warp * 16 + g + 8 * row;
        if (r >= rows) continue;
        const float inv = l[row] > 0.0f ? 1.0f / l[row] : 0.0f;
        float* dst = out + (size_t)r * stride + head * HD + 2 * c;
#pragma unroll
        for (int nb = 0; nb < HD / 8; nb++) *(float2*)(dst + nb * 8) = make_float2(o[nb][2 * row] * inv, o[nb][2 * row + 1] * inv);
    }
}

template <int HD, typename T>
cudaError_t attend_rows_t(const float* q, float* out, size_t stride, const void* kc, const void* vc, const uint32_t* sp, const DecAttn& p,
                          uint32_t rows, cudaStream_t st) {
    constexpr size_t smem = attend_rows_smem<HD>();
    if (cudaError_t e = ensure_dynamic_smem((const void*)attend_rows_kernel<HD, T>, smem); e != cudaSuccess) return e;
    attend_rows_kernel<HD, T><<<dim3((rows + PF_TILE - 1) / PF_TILE, p.nh), PF_THREADS, smem, st>>>(q, out, stride, (const T*)kc, (const T*)vc, sp, p, rows);
    return cudaGetLastError();
}

}  // namespace

cudaError_t launch_qk_rope_rows(const float* qkv, float* qo, size_t stride, uint32_t rows, void* kc, void* vc, int kv_f16, const float* qn,
                                const float* kn, const float* cs, const uint32_t* sp, const DecRope& p, cudaStream_t st) {
    if (p.hd > 256 || p.hd % 32 || 2 * p.half_rot > p.hd || rows == 0 || rows > 65535) return cudaErrorInvalidValue;
    const dim3 grid(p.nh + 2 * p.nkv, rows);
    if (kv_f16)
        qk_rope_rows_kernel<__half><<<grid, p.hd, 0, st>>>(qkv, qo, stride, (__half*)kc, (__half*)vc, qn, kn, cs, sp, p);
    else
        qk_rope_rows_kernel<float><<<grid, p.hd, 0, st>>>(qkv, qo, stride, (float*)kc, (float*)vc, qn, kn, cs, sp, p);
    return cudaGetLastError();
}

bool attend_rows_supports(uint32_t nh, uint32_t nkv, uint32_t hd) { return nkv != 0 && nh % nkv == 0 && (hd == 64 || hd == 128); }

cudaError_t launch_attend_rows(const float* q, float* out, size_t stride, uint32_t rows, const void* kc, const void* vc, int kv_f16,
                               const uint32_t* sp, const DecAttn& p, cudaStream_t st) {
    if (!attend_rows_supports(p.nh, p.nkv, p.hd) || rows == 0 || stride % 4 || ((uintptr_t)q & 15) || ((uintptr_t)out & 15)) return cudaErrorInvalidValue;
    if (p.hd == 64)
        return kv_f16 ? attend_rows_t<64, __half>(q, out, stride, kc, vc, sp, p, rows, st) : attend_rows_t<64, float>(q, out, stride, kc, vc, sp, p, rows, st);
    return kv_f16 ? attend_rows_t<128, __half>(q, out, stride, kc, vc, sp, p, rows, st) : attend_rows_t<128, float>(q, out, stride, kc, vc, sp, p, rows, st);
}

cudaError_t launch_glu_rows(const float* g, size_t g_stride, const float* u, size_t u_stride, float* out, size_t out_stride, uint32_t n,
                            uint32_t rows, int gelu, cudaStream_t st) {
    if (n % 4 || g_stride % 4 || u_stride % 4 || out_stride % 4 || rows == 0 || rows > 65535 || (((uintptr_t)g | (uintptr_t)u | (uintptr_t)out) & 15))
        return cudaErrorInvalidValue;
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
