// The non-matmul kernels of one decode token (the ops of the reference's decode graph that a dense
// Llama / Qwen3 layer uses, src/gpu_decode.rs:52-282), written so that a whole token is a fixed list of
// launches that does not depend on the position: every kernel reads the position from a device word.
//
//   norm      : RMSNorm rows (dnorm, src/cuda_decode.cu:314-328; CPU rmsnorm_f32w, src/kernels.rs:2157),
//               optionally writing the activation planes the next GEMV reads
//   qk_rope   : per-head q/k norm, RoPE, KV-cache append (dqk_rope, src/cuda_decode.cu:349-395)
//   attend    : one query per head over the cache (dattn / dattn_combine, src/cuda_decode.cu:396-536;
//               CPU attention_ext, src/model.rs:2214-2309), split over the keys, combined by the last CTA
//   glu       : act(g) * u (Op::Glu)
//   argmax    : greedy token from the logits, and the step to the next position
//
// KV cache layout here: [n_kv][max_len][hd] (f32 or f16), so that the 64 keys of a tile of one KV head are
// one contiguous run that a single bulk copy brings into shared memory.
#include <cuda_fp16.h>

#include "kernels.h"
#include "xplanes.cuh"

namespace b2 {

namespace {

__device__ __forceinline__ float block_sum(float v, float* red) {  // red: 32 floats of shared memory
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = (blockDim.x + 31) >> 5;
    __syncthreads();  // red may still be read from an earlier call
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float s = 0.0f;
    for (int i = 0; i < nw; i++) s += red[i];  // same order in every thread
    return s;
}

// ---- RMSNorm ---------------------------------------------------------------------------------
// One CTA per row. out (+)= (x * pre) * k * w with k = 1 / sqrt(mean((x pre)^2) + eps). Rows of up to
// 8 * blockDim values stay in registers between the two passes; longer rows are read twice.
constexpr int NORM_PER_THREAD = 8;
__global__ void __launch_bounds__(1024) norm_kernel(const float* __restrict__ x, float* __restrict__ out, const float* __restrict__ w, DecNorm p,
                                                    XPlanes xp) {
    __shared__ float red[32];
    pdl_launch_dependents();
    const float* xr = x + (size_t)blockIdx.x * p.x_stride;
    float* o = out + (size_t)blockIdx.x * p.out_stride;
    const bool in_regs = p.n <= NORM_PER_THREAD * blockDim.x;
    float wv[NORM_PER_THREAD], v[NORM_PER_THREAD];
    if (in_regs && w) {  // the weights do not depend on the kernel before this one
#pragma unroll
        for (int j = 0; j < NORM_PER_THREAD; j++) {
            const uint32_t i = threadIdx.x + j * blockDim.x;
            wv[j] = i < p.n ? w[i] : 0.0f;
        }
    }
    pdl_wait();
    float s = 0.0f;
    if (in_regs) {
#pragma unroll
        for (int j = 0; j < NORM_PER_THREAD; j++) {
            const uint32_t i = threadIdx.x + j * blockDim.x;
            v[j] = i < p.n ? xr[i] * p.pre : 0.0f;
            s += v[j] * v[j];
        }
    } else {
        for (uint32_t i = threadIdx.x; i < p.n; i += blockDim.x) {
            float t = xr[i] * p.pre;
            s += t * t;
        }
    }
    const float k = 1.0f / sqrtf(block_sum(s, red) / (float)p.n + p.eps);
    if (in_regs) {
#pragma unroll
        for (int j = 0; j < NORM_PER_THREAD; j++) {
            const uint32_t i = threadIdx.x + j * blockDim.x;
            if (i < p.n) {  // p.n % 32 == 0 when planes are asked for: whole warps stay together
                float t = v[j] * k;
                if (w) t *= wv[j];
                if (p.add) t += o[i];
                o[i] = t;
                if (p.planes) xplanes_block(t, (int)(i >> 5), threadIdx.x & 31, (int)p.n, xp);
            }
        }
    } else {
        for (uint32_t i = threadIdx.x; i < p.n; i += blockDim.x) {
            float t = xr[i] * p.pre * k;
            if (w) t *= w[i];
            if (p.add) t += o[i];
            o[i] = t;
            if (p.planes) xplanes_block(t, (int)(i >> 5), threadIdx.x & 31, (int)p.n, xp);
        }
    }
}

// ---- q / k norm, RoPE, cache append ------------------------------------------------------------
// Blocks: nh query heads, then nkv key heads, then nkv value heads; a thread per dimension.
template <typename T>
__global__ void __launch_bounds__(256) qk_rope_kernel(const float* __restrict__ qkv, float* __restrict__ qo, T* __restrict__ kc, T* __restrict__ vc,
                                                      const float* __restrict__ qn, const float* __restrict__ kn, const float* __restrict__ cs_table,
                                                      const uint32_t* __restrict__ sp, DecRope p) {
    __shared__ float buf[256];
    __shared__ float red[32];
    pdl_launch_dependents();
    pdl_wait();
    const uint32_t h = blockIdx.x, i = threadIdx.x, hd = p.hd, pos = sp[0];
    const uint32_t kind = h < p.nh ? 0 : (h < p.nh + p.nkv ? 1 : 2);
    const uint32_t hh = kind == 0 ? h : (kind == 1 ? h - p.nh : h - p.nh - p.nkv);
    float v = kind == 0 ? qkv[hh * p.q_stride + i] : (kind == 1 || p.v_from_k) ? qkv[p.k_off + hh * hd + i] : qkv[p.v_off + hh * hd + i];
    const bool norm = kind == 0 ? qn != nullptr : (kind == 1 ? kn != nullptr : p.v_norm != 0);
    if (norm) {
        float s = block_sum(v * v, red);
        v = v * (1.0f / sqrtf(s / (float)hd + p.eps));
        if (kind == 0) v *= qn[i];
        else if (kind == 1) v *= kn[i];
    }
    if (pos >= p.max_len) return;  // a full cache: nothing is written (the host refuses the step before this)
    const size_t at = ((size_t)hh * p.max_len + pos) * hd + i;
    if (kind == 2) {
        vc[at] = (T)v;
        return;
    }
    buf[i] = v;
    __syncthreads();
    const uint32_t hr = p.half_rot;
    const float* cs = cs_table + (size_t)(pos - sp[1]) * p.cs_stride + p.cs_off;  // cos[hr] then sin[hr] of this position
    if (i < 2 * hr) {
        if (p.interleaved) {
            uint32_t j = i >> 1;
            float c = cs[j], s = cs[hr + j];
            float x1 = buf[2 * j], x2 = buf[2 * j + 1];
            v = (i & 1) == 0 ? __fsub_rn(__fmul_rn(x1, c), __fmul_rn(x2, s)) : __fadd_rn(__fmul_rn(x2, c), __fmul_rn(x1, s));
        } else {
            uint32_t j = i < hr ? i : i - hr;
            float c = cs[j], s = cs[hr + j];
            float x1 = buf[j], x2 = buf[j + hr];
            v = i < hr ? __fsub_rn(__fmul_rn(x1, c), __fmul_rn(x2, s)) : __fadd_rn(__fmul_rn(x2, c), __fmul_rn(x1, s));
        }
    }
    if (kind == 0) qo[hh * hd + i] = v;
    else kc[at] = (T)v;
}

// ---- act(g) * u ---------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) glu_kernel(const float* __restrict__ g, const float* __restrict__ u, float* __restrict__ out, uint32_t n,
                                                  int gelu) {
    pdl_launch_dependents();
    pdl_wait();
    uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    float a = g[i];
    float r;
    if (gelu) {
        const float K2 = 2.0f * 0.7978846f;
        float t = K2 * (a + 0.044715f * a * a * a);
        r = a / (1.0f + expf(-t));
    } else {
        r = a / (1.0f + expf(-a));
    }
    out[i] = r * u[i];
}

// ---- attention -----------------------------------------------------------------------------------
constexpr int ATT_TILE = 64;         // keys per shared-memory tile
constexpr int ATT_THREADS = 256;
constexpr int ATT_MAX_SPLITS = 64;   // CTAs per KV head at most
constexpr long long ATT_WAIT_LIMIT = 2000000000LL;  // cycles (about a second) before a wait on a copy gives up

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void bar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void bar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool bar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_addr(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded: false after ATT_WAIT_LIMIT cycles.
__device__ __forceinline__ bool bar_wait(uint64_t* bar, uint32_t parity) {
    if (bar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    for (uint32_t spin = 1;; spin++) {
        if (bar_try_wait(bar, parity)) return true;
        if ((spin & 255) == 0 && clock64() - t0 > ATT_WAIT_LIMIT) return false;
    }
}
// Contiguous global -> shared copy (both 16-byte aligned, bytes a multiple of 16), completion on `bar`.
__device__ __forceinline__ void bulk_load(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_addr(dst)), "l"(src),
                 "r"(bytes), "r"(smem_addr(bar))
                 : "memory");
}

__device__ __forceinline__ float4 kv4(const float* p) { return *(const float4*)p; }
__device__ __forceinline__ float4 kv4(const __half* p) {
    uint2 r = *(const uint2*)p;
    float2 a = __half22float2(*(const __half2*)&r.x), b = __half22float2(*(const __half2*)&r.y);
    return make_float4(a.x, a.y, b.x, b.y);
}

template <int HD, int G, typename T>
constexpr size_t attend_smem() {
    size_t tiles = 2 * (size_t)ATT_TILE * HD * sizeof(T);
    size_t red = (size_t)(ATT_THREADS / (HD / 4)) * G * HD * 4;
    size_t first = tiles > red ? tiles : red;
    return first + 16 /* barriers */ + (size_t)G * HD * 4 /* q */ + (size_t)G * ATT_TILE * 4 /* p */ + (size_t)G * ATT_MAX_SPLITS * 4 /* combine weights */
           + 4 * (size_t)G * 4 + 16;
}

// Grid (nkv, splits). CTA (kvh, s) runs the G query heads of KV head kvh over its share of the key tiles with
// an online softmax, writes the unnormalized partial (o, m, l) of each head, and the last CTA of a KV head
// to finish (a counter, no waiting) combines the partials, writes `out` and, if asked, the planes of `out`.
template <int HD, int G, typename T>
__global__ void __launch_bounds__(ATT_THREADS) attend_kernel(const float* __restrict__ q, const T* __restrict__ kc, const T* __restrict__ vc,
                                                             float* __restrict__ out, float* part, uint32_t* counters,
                                                             const uint32_t* __restrict__ sp, DecAttn p, XPlanes xp, uint32_t* status) {
    constexpr int COLS = HD / 4, PARTS = ATT_THREADS / COLS, KPP = ATT_TILE / PARTS;
    constexpr size_t TILE_BYTES = 2 * (size_t)ATT_TILE * HD * sizeof(T);
    constexpr size_t RED_BYTES = (size_t)PARTS * G * HD * 4;
    constexpr size_t FIRST = TILE_BYTES > RED_BYTES ? TILE_BYTES : RED_BYTES;
    extern __shared__ __align__(128) uint8_t smem[];
    T* Ks = (T*)smem;
    T* Vs = Ks + ATT_TILE * HD;
    float* red = (float*)smem;  // reused after the last tile
    uint64_t* bars = (uint64_t*)(smem + FIRST);
    float* qs = (float*)(smem + FIRST + 16);
    float* sc = qs + G * HD;
    float* wts = sc + G * ATT_TILE;
    float* mrun = wts + G * ATT_MAX_SPLITS;
    float* lrun = mrun + G;
    float* alpha = lrun + G;
    int* flags = (int*)(alpha + G);  // [0] abort, [1] last

    pdl_launch_dependents();
    pdl_wait();
    const int tid = threadIdx.x, kvh = blockIdx.x, split = blockIdx.y;
    uint32_t len = sp[0] + 1;
    if (len > p.max_len) len = p.max_len;
    const uint32_t lo = (p.window != 0 && len > p.window) ? len - p.window : 0;
    const uint32_t n = len - lo;
    const uint32_t tiles = (n + ATT_TILE - 1) / ATT_TILE;
    uint32_t ns = min(tiles, gridDim.y);
    const uint32_t per = (tiles + ns - 1) / ns;
    ns = (tiles + per - 1) / per;
    if ((uint32_t)split >= ns) return;
    const int h0 = kvh * G;
    const float NEG = -INFINITY;

    const uint32_t t0 = split * per, t1 = min(tiles, t0 + per);
    auto issue = [&](uint32_t t) {  // one thread: both copies of key tile t
        const uint32_t j0 = lo + t * ATT_TILE, nv = min((uint32_t)ATT_TILE, len - j0);
        const uint32_t bytes = nv * HD * (uint32_t)sizeof(T);
        const size_t at = ((size_t)kvh * p.max_len + j0) * HD;
        bar_expect_tx(&bars[0], bytes);
        bulk_load(Ks, kc + at, bytes, &bars[0]);
        bar_expect_tx(&bars[1], bytes);
        bulk_load(Vs, vc + at, bytes, &bars[1]);
    };
    if (tid == 0) {
        bar_init(&bars[0], 1);
        bar_init(&bars[1], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        issue(t0);  // the first tile is on its way while the queries are staged
        flags[0] = 0;
        flags[1] = 0;
    }
    for (int i = tid; i < G * HD; i += ATT_THREADS) qs[i] = q[(size_t)h0 * HD + i] * p.scale;
    if (tid < G) {
        mrun[tid] = NEG;
        lrun[tid] = 0.0f;
    }
    __syncthreads();

    float4 acc[G];
#pragma unroll
    for (int g = 0; g < G; g++) acc[g] = make_float4(0.f, 0.f, 0.f, 0.f);
    const int part_id = tid / COLS, c4 = tid % COLS;
    const int lane8 = tid & 7, slot = tid >> 3;
    bool ok = true;
    uint32_t phase = 0;
    for (uint32_t t = t0; t < t1; t++) {
        const uint32_t j0 = lo + t * ATT_TILE, nv = min((uint32_t)ATT_TILE, len - j0);
        phase = (t - t0) & 1;
        if (tid == 0 && t > t0) issue(t);
        if (!bar_wait(&bars[0], phase)) flags[0] = 1;
        __syncthreads();
        if (flags[0]) {
            ok = false;
            break;
        }
        // scores: eight lanes per key, two keys per thread group
#pragma unroll
        for (int pass = 0; pass < 2; pass++) {
            const int j = slot + 32 * pass;
            float s[G];
#pragma unroll
            for (int g = 0; g < G; g++) s[g] = 0.0f;
            if ((uint32_t)j < nv) {
                const T* kr = Ks + j * HD;
#pragma unroll
                for (int i = 0; i < HD / 32; i++) {
                    const int d = lane8 * 4 + 32 * i;
                    float4 k4 = kv4(kr + d);
#pragma unroll
                    for (int g = 0; g < G; g++) {
                        float4 q4 = *(const float4*)(qs + g * HD + d);
                        s[g] = fmaf(k4.x, q4.x, s[g]);
                        s[g] = fmaf(k4.y, q4.y, s[g]);
                        s[g] = fmaf(k4.z, q4.z, s[g]);
                        s[g] = fmaf(k4.w, q4.w, s[g]);
                    }
                }
            }
#pragma unroll
            for (int g = 0; g < G; g++) {
                float v = s[g];
                v += __shfl_xor_sync(0xffffffffu, v, 1);
                v += __shfl_xor_sync(0xffffffffu, v, 2);
                v += __shfl_xor_sync(0xffffffffu, v, 4);
                if (lane8 == 0) sc[g * ATT_TILE + j] = (uint32_t)j < nv ? v : NEG;
            }
        }
        __syncthreads();
        // online softmax: warp g owns head g
        if ((tid >> 5) < G) {
            const int g = tid >> 5, lane = tid & 31;
            float a = sc[g * ATT_TILE + lane], b = sc[g * ATT_TILE + 32 + lane];
            float mx = fmaxf(a, b);
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
            const float mo = mrun[g], mn = fmaxf(mo, mx);
            float ea = expf(a - mn), eb = expf(b - mn);
            float sum = ea + eb;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
            sc[g * ATT_TILE + lane] = ea;
            sc[g * ATT_TILE + 32 + lane] = eb;
            if (lane == 0) {
                const float al = expf(mo - mn);  // 0 on the first tile (mo = -inf)
                alpha[g] = al;
                lrun[g] = lrun[g] * al + sum;
                mrun[g] = mn;
            }
        }
        if (!bar_wait(&bars[1], phase)) flags[0] = 1;
        __syncthreads();
        if (flags[0]) {
            ok = false;
            break;
        }
        // values: thread (part, c4) adds its KPP keys of the tile into four dimensions of every head
#pragma unroll
        for (int g = 0; g < G; g++) {
            const float al = alpha[g];
            acc[g].x *= al;
            acc[g].y *= al;
            acc[g].z *= al;
            acc[g].w *= al;
        }
#pragma unroll
        for (int kk = 0; kk < KPP; kk++) {
            const int j = part_id * KPP + kk;
            if ((uint32_t)j < nv) {
                float4 v4 = kv4(Vs + j * HD + c4 * 4);
#pragma unroll
                for (int g = 0; g < G; g++) {
                    const float e = sc[g * ATT_TILE + j];
                    acc[g].x = fmaf(e, v4.x, acc[g].x);
                    acc[g].y = fmaf(e, v4.y, acc[g].y);
                    acc[g].z = fmaf(e, v4.z, acc[g].z);
                    acc[g].w = fmaf(e, v4.w, acc[g].w);
                }
            }
        }
        __syncthreads();  // the tile and the probabilities are free again
    }
    if (!ok) {
        // A copy did not arrive in time: record it, give the copies one more bounded wait so that nothing
        // lands in shared memory that has been handed on, and leave without touching the outputs.
        if (tid == 0) {
            atomicExch(status, 1u);
            bar_wait(&bars[0], phase);
            bar_wait(&bars[1], phase);
        }
        return;
    }

    // partial of this split: sum over the parts, then (o, m, l) per head
#pragma unroll
    for (int g = 0; g < G; g++) *(float4*)(red + ((size_t)part_id * G + g) * HD + c4 * 4) = acc[g];
    __syncthreads();
    for (int idx = tid; idx < G * HD; idx += ATT_THREADS) {
        const int g = idx / HD, d = idx % HD;
        float o = 0.0f;
#pragma unroll
        for (int pp = 0; pp < PARTS; pp++) o += red[((size_t)pp * G + g) * HD + d];
        float* ph = part + ((size_t)(h0 + g) * ATT_MAX_SPLITS + split) * (HD + 2);
        ph[d] = o;
        if (d == 0) {
            ph[HD] = mrun[g];
            ph[HD + 1] = lrun[g];
        }
    }
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        const uint32_t prev = atomicAdd(&counters[kvh], 1u);
        flags[1] = prev == ns - 1;
    }
    __syncthreads();
    if (!flags[1]) return;
    __threadfence();
    // combine (the last CTA of this KV head)
    for (int i = tid; i < G * (int)ns; i += ATT_THREADS) {
        const int g = i / (int)ns;
        const float* ph = part + (size_t)(h0 + g) * ATT_MAX_SPLITS * (HD + 2);
        float M = NEG;
        for (uint32_t s = 0; s < ns; s++) M = fmaxf(M, __ldcg(ph + s * (HD + 2) + HD));
        wts[g * ATT_MAX_SPLITS + (i % (int)ns)] = expf(__ldcg(ph + (i % (int)ns) * (HD + 2) + HD) - M);
    }
    __syncthreads();
    for (int idx = tid; idx < G * HD; idx += ATT_THREADS) {
        const int g = idx / HD, d = idx % HD;
        const float* ph = part + (size_t)(h0 + g) * ATT_MAX_SPLITS * (HD + 2);
        float L = 0.0f, o = 0.0f;
        for (uint32_t s = 0; s < ns; s++) {
            const float wgt = wts[g * ATT_MAX_SPLITS + s];
            L += __ldcg(ph + s * (HD + 2) + HD + 1) * wgt;
            o += __ldcg(ph + s * (HD + 2) + d) * wgt;
        }
        const float r = o / L;
        out[(size_t)h0 * HD + idx] = r;
        if (p.planes) xplanes_block(r, (h0 * HD + idx) >> 5, tid & 31, (int)(p.nh * HD), xp);
    }
    if (tid == 0) counters[kvh] = 0;  // ready for the next launch
}

// ---- greedy token ----------------------------------------------------------------------------------
constexpr int ARGMAX_CTAS = 128;

// First index of the largest logit (ties to the lower index, as a left-to-right scan with `>` finds it).
// The last CTA to finish reduces the partials, stores the token, appends it to the output list and moves
// the step words on: sp[0] (position) and sp[2] (tokens generated) each grow by one.
__global__ void __launch_bounds__(256) argmax_kernel(const float* __restrict__ logits, uint32_t n, float* pval, int* pidx, uint32_t* counter,
                                                     int* token, int* out_tokens, uint32_t* sp) {
    __shared__ float sv[8];
    __shared__ int si[8];
    __shared__ int last;
    pdl_launch_dependents();
    pdl_wait();
    float best = -INFINITY;
    int bi = 0x7fffffff;
    for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
        float v = logits[i];
        if (v > best || (v == best && (int)i < bi)) {
            best = v;
            bi = (int)i;
        }
    }
    auto reduce = [&](float& b, int& ix) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            float ob = __shfl_xor_sync(0xffffffffu, b, o);
            int oi = __shfl_xor_sync(0xffffffffu, ix, o);
            if (ob > b || (ob == b && oi < ix)) {
                b = ob;
                ix = oi;
            }
        }
    };
    reduce(best, bi);
    if ((threadIdx.x & 31) == 0) {
        sv[threadIdx.x >> 5] = best;
        si[threadIdx.x >> 5] = bi;
    }
    __syncthreads();
    if (threadIdx.x < 32) {
        best = threadIdx.x < 8 ? sv[threadIdx.x] : -INFINITY;
        bi = threadIdx.x < 8 ? si[threadIdx.x] : 0x7fffffff;
        reduce(best, bi);
        if (threadIdx.x == 0) {
            pval[blockIdx.x] = best;
            pidx[blockIdx.x] = bi;
            __threadfence();
            last = atomicAdd(counter, 1u) == gridDim.x - 1;
        }
    }
    __syncthreads();
    if (!last || threadIdx.x >= 32) return;
    __threadfence();
    best = -INFINITY;
    bi = 0x7fffffff;
    for (uint32_t i = threadIdx.x; i < gridDim.x; i += 32) {
        float v = __ldcg(pval + i);
        int ix = __ldcg(pidx + i);
        if (v > best || (v == best && ix < bi)) {
            best = v;
            bi = ix;
        }
    }
    reduce(best, bi);
    if (threadIdx.x == 0) {
        if (bi == 0x7fffffff) bi = 0;  // every logit NaN or -inf
        token[0] = bi;
        if (out_tokens) out_tokens[sp[2]] = bi;
        sp[2] += 1;
        sp[0] += 1;
        *counter = 0;
    }
}

// ---- host <-> cache rows, step words ---------------------------------------------------------------
// rows [n][nkv][hd] f32 (the host's LayerCache order) <-> cache [nkv][max_len][hd] at positions pos0 ..
template <typename T, bool TO_CACHE>
__global__ void __launch_bounds__(256) kv_rows_kernel(float* rows, T* cache, uint32_t nkv, uint32_t hd, uint32_t max_len, uint32_t pos0,
                                                      uint32_t n) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (size_t)n * nkv * hd) return;
    uint32_t d = (uint32_t)(i % hd), h = (uint32_t)((i / hd) % nkv), r = (uint32_t)(i / ((size_t)hd * nkv));
    size_t at = ((size_t)h * max_len + pos0 + r) * hd + d;
    if (TO_CACHE) cache[at] = (T)rows[i];
    else rows[i] = (float)cache[at];
}

__global__ void set_step_kernel(uint32_t* sp, uint32_t pos, uint32_t table_pos0, uint32_t count, int* token, int tok) {
    sp[0] = pos;
    sp[1] = table_pos0;
    sp[2] = count;
    sp[3] = 0;
    if (token) token[0] = tok;
}

}  // namespace

cudaError_t launch_kv_rows(float* rows, void* cache, int kv_f16, bool to_cache, uint32_t nkv, uint32_t hd, uint32_t max_len, uint32_t pos0,
                           uint32_t n, cudaStream_t st) {
    size_t total = (size_t)n * nkv * hd;
    if (total == 0) return cudaSuccess;
    unsigned grid = (unsigned)((total + 255) / 256);
    if (kv_f16) {
        if (to_cache) kv_rows_kernel<__half, true><<<grid, 256, 0, st>>>(rows, (__half*)cache, nkv, hd, max_len, pos0, n);
        else kv_rows_kernel<__half, false><<<grid, 256, 0, st>>>(rows, (__half*)cache, nkv, hd, max_len, pos0, n);
    } else {
        if (to_cache) kv_rows_kernel<float, true><<<grid, 256, 0, st>>>(rows, (float*)cache, nkv, hd, max_len, pos0, n);
        else kv_rows_kernel<float, false><<<grid, 256, 0, st>>>(rows, (float*)cache, nkv, hd, max_len, pos0, n);
    }
    return cudaGetLastError();
}

cudaError_t launch_set_step(uint32_t* sp, uint32_t pos, uint32_t table_pos0, uint32_t count, int* token, int tok, cudaStream_t st) {
    set_step_kernel<<<1, 1, 0, st>>>(sp, pos, table_pos0, count, token, tok);
    return cudaGetLastError();
}

cudaError_t launch_norm(const float* x, float* out, const float* w, const DecNorm& p, uint32_t rows, XPlanes xp, cudaStream_t st, bool pdl) {
    if (p.planes && (p.n % 32 || rows != 1)) return cudaErrorInvalidValue;
    unsigned threads = p.n >= 4096 ? 1024 : p.n >= 1024 ? 512 : ((p.n + 31) / 32) * 32;
    return launch_k(norm_kernel, dim3(rows), dim3(threads), 0, st, pdl, x, out, w, p, xp);
}

template <typename T>
static cudaError_t rope_t(const float* qkv, float* qo, void* kc, void* vc, const float* qn, const float* kn, const float* cs, const uint32_t* sp,
                          const DecRope& p, cudaStream_t st, bool pdl) {
    return launch_k(qk_rope_kernel<T>, dim3(p.nh + 2 * p.nkv), dim3(p.hd), 0, st, pdl, qkv, qo, (T*)kc, (T*)vc, qn, kn, cs, sp, p);
}

cudaError_t launch_qk_rope(const float* qkv, float* qo, void* kc, void* vc, int kv_f16, const float* qn, const float* kn, const float* cs,
                           const uint32_t* sp, const DecRope& p, cudaStream_t st, bool pdl) {
    if (p.hd > 256 || p.hd % 32 || 2 * p.half_rot > p.hd) return cudaErrorInvalidValue;
    return kv_f16 ? rope_t<__half>(qkv, qo, kc, vc, qn, kn, cs, sp, p, st, pdl) : rope_t<float>(qkv, qo, kc, vc, qn, kn, cs, sp, p, st, pdl);
}

bool attend_supports(uint32_t nh, uint32_t nkv, uint32_t hd) {
    if (nkv == 0 || nh % nkv) return false;
    uint32_t g = nh / nkv;
    return (hd == 64 || hd == 128) && (g == 1 || g == 2 || g == 4 || g == 8);
}
size_t attend_part_floats(uint32_t nh, uint32_t hd) { return (size_t)nh * ATT_MAX_SPLITS * (hd + 2); }

template <int HD, int G, typename T>
static cudaError_t attend_t(const float* q, const void* kc, const void* vc, float* out, float* part, uint32_t* counters, const uint32_t* sp,
                            const DecAttn& p, XPlanes xp, uint32_t* status, cudaStream_t st, bool pdl) {
    constexpr size_t smem = attend_smem<HD, G, T>();
    static bool set = false;  // per instantiation; the attribute is per function and device-wide values are equal
    if (!set) {
        cudaError_t e = cudaFuncSetAttribute(attend_kernel<HD, G, T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
        set = true;
    }
    uint32_t splits = (p.max_len + ATT_TILE - 1) / ATT_TILE;
    if (splits > ATT_MAX_SPLITS) splits = ATT_MAX_SPLITS;
    if (splits == 0) splits = 1;
    dim3 grid(p.nkv, splits);
    return launch_k(attend_kernel<HD, G, T>, grid, dim3(ATT_THREADS), smem, st, pdl, q, (const T*)kc, (const T*)vc, out, part, counters, sp, p, xp,
                    status);
}

template <int HD, typename T>
static cudaError_t attend_g(uint32_t g, const float* q, const void* kc, const void* vc, float* out, float* part, uint32_t* counters,
                            const uint32_t* sp, const DecAttn& p, XPlanes xp, uint32_t* status, cudaStream_t st, bool pdl) {
    switch (g) {
        case 1: return attend_t<HD, 1, T>(q, kc, vc, out, part, counters, sp, p, xp, status, st, pdl);
        case 2: return attend_t<HD, 2, T>(q, kc, vc, out, part, counters, sp, p, xp, status, st, pdl);
        case 4: return attend_t<HD, 4, T>(q, kc, vc, out, part, counters, sp, p, xp, status, st, pdl);
        case 8: return attend_t<HD, 8, T>(q, kc, vc, out, part, counters, sp, p, xp, status, st, pdl);
    }
    return cudaErrorInvalidValue;
}

cudaError_t launch_attend(const float* q, const void* kc, const void* vc, int kv_f16, float* out, float* part, uint32_t* counters,
                          const uint32_t* sp, const DecAttn& p, XPlanes xp, uint32_t* status, cudaStream_t st, bool pdl) {
    if (!attend_supports(p.nh, p.nkv, p.hd)) return cudaErrorInvalidValue;
    const uint32_t g = p.nh / p.nkv;
    if (p.hd == 64)
        return kv_f16 ? attend_g<64, __half>(g, q, kc, vc, out, part, counters, sp, p, xp, status, st, pdl)
                      : attend_g<64, float>(g, q, kc, vc, out, part, counters, sp, p, xp, status, st, pdl);
    return kv_f16 ? attend_g<128, __half>(g, q, kc, vc, out, part, counters, sp, p, xp, status, st, pdl)
                  : attend_g<128, float>(g, q, kc, vc, out, part, counters, sp, p, xp, status, st, pdl);
}

cudaError_t launch_glu(const float* g, const float* u, float* out, uint32_t n, int gelu, cudaStream_t st, bool pdl) {
    return launch_k(glu_kernel, dim3((n + 255) / 256), dim3(256), 0, st, pdl, g, u, out, n, gelu);
}

cudaError_t launch_argmax(const float* logits, uint32_t n, float* pval, int* pidx, uint32_t* counter, int* token, int* out_tokens, uint32_t* sp,
                          cudaStream_t st, bool pdl) {
    return launch_k(argmax_kernel, dim3(ARGMAX_CTAS), dim3(256), 0, st, pdl, logits, n, pval, pidx, counter, token, out_tokens, sp);
}

}  // namespace b2
