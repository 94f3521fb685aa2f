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

#include "attend_core.cuh"

namespace b2 {

using namespace attend_core;

namespace {

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
// Blocks: nh query heads, then nkv key heads, then nkv value heads; a thread per dimension (rope_head, attend_core.cuh).
template <typename T>
__global__ void __launch_bounds__(256) qk_rope_kernel(const float* __restrict__ qkv, float* __restrict__ qo, T* __restrict__ kc, T* __restrict__ vc,
                                                      const float* __restrict__ qn, const float* __restrict__ kn, const float* __restrict__ cs_table,
                                                      const uint32_t* __restrict__ sp, DecRope p) {
    __shared__ float buf[256];
    __shared__ float red[32];
    pdl_launch_dependents();
    pdl_wait();
    rope_head<T>(blockIdx.x, threadIdx.x, sp[0], sp[1], qkv, qo, kc, vc, qn, kn, cs_table, p, buf, red);
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

// ---- attention: grid (KV heads, splits), one unit per CTA (attend_core.cuh) --------------------------------
// blockIdx.z: the token of a step of several tokens (AttnTokens: its queries, outputs and planes a fixed stride behind token
// 0's, its own step words, partials and counters); the keys of all the step's tokens are in the caches already.
template <int HD, int G, typename T>
__global__ void __launch_bounds__(ATT_THREADS) attend_kernel(const float* __restrict__ q, T* kc, T* vc, float* __restrict__ out, float* part,
                                                             uint32_t* counters, const uint32_t* __restrict__ sp, DecAttn p, XPlanes xp,
                                                             uint32_t* status, FusedRope fr, AttnTokens at) {
    extern __shared__ __align__(128) uint8_t smem[];
    pdl_launch_dependents();
    if (blockIdx.z) {
        const size_t z = blockIdx.z;
        q += z * at.act_stride;
        out += z * at.act_stride;
        part += z * at.part_stride;
        counters += z * p.nkv;
        sp += 4 * z;
        if (fr.qkv) fr.qkv += z * at.act_stride;
        if (xp.planes) {
            xp.planes = (int8_t*)((uint8_t*)xp.planes + z * at.planes_stride);
            xp.sx = (float2*)((uint8_t*)xp.sx + z * at.planes_stride);
            xp.v16 = (int32_t*)((uint8_t*)xp.v16 + z * at.planes_stride);
        }
    }
    // the step words (position, RoPE table base) were written before this step's graph was launched
    attend_unit<HD, G, T>(smem, threadIdx.x, 0, blockIdx.x, blockIdx.y, gridDim.y, sp[0], q, kc, vc, out, part, counters, p, xp, status, nullptr,
                          fr.qkv ? &fr : nullptr, sp[1], true);
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

// ---- all-gather of a row-sharded vector by stores into the peers' buffers ---------------------------------------
// One CTA. The GPUs meet twice: once before anyone writes (every rank is then past the kernels that read the vector's
// old contents), once after (every part has landed everywhere). A meeting = a store of the running epoch into each
// peer's flag word for this rank, then a bounded wait until every peer's word here has reached the epoch.
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) { asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory"); }
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
constexpr long long EXCHANGE_WAIT_LIMIT = 1000000000LL;  // cycles (about half a second)

__device__ __forceinline__ bool peers_meet(const PeerSet& ps, uint32_t* lflags, int bank, uint32_t epoch, int* ok_s,
                                           long long limit = EXCHANGE_WAIT_LIMIT) {
    const uint32_t tid = threadIdx.x;
    if (tid == 0) *ok_s = 1;
    __syncthreads();
    if (tid < ps.world && tid != ps.rank) {
        st_release_sys(ps.flags[tid] + bank + ps.rank, epoch);
        const long long t0 = clock64();
        uint32_t spin = 0;
        while ((int32_t)(ld_acquire_sys(lflags + bank + tid) - epoch) < 0) {
            if ((++spin & 15) == 0 && clock64() - t0 > limit) {
                *ok_s = 0;
                break;
            }
        }
    }
    __syncthreads();
    return *ok_s != 0;
}

__global__ void __launch_bounds__(1024) exchange_kernel(PeerSet ps, size_t off, uint32_t n, uint32_t* lflags, uint32_t* status, int meet_first,
                                                        long long limit) {
    __shared__ int ok_s;
    __shared__ uint32_t epoch_s;
    pdl_launch_dependents();
    pdl_wait();
    if (threadIdx.x == 0) epoch_s = lflags[0] + 1;
    __syncthreads();
    const uint32_t epoch = epoch_s;
    // The first meeting is left out where the plan has shown that no kernel between the previous exchange and this one
    // reads the other ranks' parts of the vector (a peer can be at most one exchange ahead).
    bool ok = meet_first ? peers_meet(ps, lflags, 8, epoch, &ok_s, limit) : true;
    if (ok) {
        const uint32_t part = n / ps.world;  // a multiple of 4 (checked on the host)
        const float4* src = (const float4*)(ps.base[ps.rank] + off + (size_t)ps.rank * part);
        for (uint32_t p = 0; p < ps.world; p++) {
            if (p == ps.rank) continue;
            float4* dst = (float4*)(ps.base[p] + off + (size_t)ps.rank * part);
            for (uint32_t i = threadIdx.x; i < part / 4; i += blockDim.x) dst[i] = __ldcg(src + i);
        }
        __threadfence_system();
        ok = peers_meet(ps, lflags, 16, epoch, &ok_s, limit);
    }
    if (threadIdx.x == 0) {
        lflags[0] = epoch;
        if (!ok) atomicExch(status, 4u);
    }
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

cudaError_t launch_exchange(const PeerSet& ps, size_t off_floats, uint32_t n, uint32_t* lflags, uint32_t* status, cudaStream_t st, bool pdl,
                            bool meet_first, long long wait_limit_cycles) {
    if (ps.world < 2 || ps.world > 8 || n % (4 * ps.world)) return cudaErrorInvalidValue;
    const long long limit = wait_limit_cycles > 0 ? wait_limit_cycles : EXCHANGE_WAIT_LIMIT;
    return launch_k(exchange_kernel, dim3(1), dim3(1024), 0, st, pdl, ps, off_floats, n, lflags, status, meet_first ? 1 : 0, limit);
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
size_t attend_part_floats(uint32_t nh, uint32_t hd) { return (size_t)nh * ATT_MAX_SPLITS * (hd + 4); }

template <int HD, int G, typename T>
static cudaError_t attend_t(const float* q, void* kc, void* vc, float* out, float* part, uint32_t* counters, const uint32_t* sp,
                            const DecAttn& p, XPlanes xp, uint32_t* status, cudaStream_t st, bool pdl, const FusedRope& fr, const AttnTokens& at) {
    constexpr size_t smem = attend_smem<HD, G, T>();
    if (cudaError_t e = ensure_dynamic_smem((const void*)attend_kernel<HD, G, T>, smem, 0); e != cudaSuccess) return e;
    uint32_t splits = (p.max_len + ATT_TILE - 1) / ATT_TILE;
    if (splits > ATT_MAX_SPLITS) splits = ATT_MAX_SPLITS;
    if (splits == 0) splits = 1;
    dim3 grid(p.nkv, splits, (unsigned)std::max(1, at.n));
    return launch_k(attend_kernel<HD, G, T>, grid, dim3(ATT_THREADS), smem, st, pdl, q, (T*)kc, (T*)vc, out, part, counters, sp, p, xp, status, fr, at);
}

template <int HD, typename T>
static cudaError_t attend_g(uint32_t g, const float* q, void* kc, void* vc, float* out, float* part, uint32_t* counters,
                            const uint32_t* sp, const DecAttn& p, XPlanes xp, uint32_t* status, cudaStream_t st, bool pdl, const FusedRope& fr,
                            const AttnTokens& at) {
    switch (g) {
        case 1: return attend_t<HD, 1, T>(q, kc, vc, out, part, counters, sp, p, xp, status, st, pdl, fr, at);
        case 2: return attend_t<HD, 2, T>(q, kc, vc, out, part, counters, sp, p, xp, status, st, pdl, fr, at);
        case 4: return attend_t<HD, 4, T>(q, kc, vc, out, part, counters, sp, p, xp, status, st, pdl, fr, at);
        case 8: return attend_t<HD, 8, T>(q, kc, vc, out, part, counters, sp, p, xp, status, st, pdl, fr, at);
    }
    return cudaErrorInvalidValue;
}

cudaError_t launch_attend(const float* q, void* kc, void* vc, int kv_f16, float* out, float* part, uint32_t* counters,
                          const uint32_t* sp, const DecAttn& p, XPlanes xp, uint32_t* status, cudaStream_t st, bool pdl, const FusedRope* frp,
                          const AttnTokens* atp) {
    if (!attend_supports(p.nh, p.nkv, p.hd)) return cudaErrorInvalidValue;
    AttnTokens at{};
    if (atp) at = *atp;
    if (at.n > 1 && frp) return cudaErrorInvalidValue;  // the tokens of one launch must find each other's keys in the caches
    FusedRope fr{};
    if (frp) {
        fr = *frp;
        if (fr.r.nh != p.nh || fr.r.nkv != p.nkv || fr.r.hd != p.hd || 2 * fr.r.half_rot > p.hd || fr.r.v_norm || fr.r.v_from_k)
            return cudaErrorInvalidValue;
    }
    const uint32_t g = p.nh / p.nkv;
    if (p.hd == 64)
        return kv_f16 ? attend_g<64, __half>(g, q, kc, vc, out, part, counters, sp, p, xp, status, st, pdl, fr, at)
                      : attend_g<64, float>(g, q, kc, vc, out, part, counters, sp, p, xp, status, st, pdl, fr, at);
    return kv_f16 ? attend_g<128, __half>(g, q, kc, vc, out, part, counters, sp, p, xp, status, st, pdl, fr, at)
                  : attend_g<128, float>(g, q, kc, vc, out, part, counters, sp, p, xp, status, st, pdl, fr, at);
}

cudaError_t launch_glu(const float* g, const float* u, float* out, uint32_t n, int gelu, cudaStream_t st, bool pdl) {
    return launch_k(glu_kernel, dim3((n + 255) / 256), dim3(256), 0, st, pdl, g, u, out, n, gelu);
}

cudaError_t launch_argmax(const float* logits, uint32_t n, float* pval, int* pidx, uint32_t* counter, int* token, int* out_tokens, uint32_t* sp,
                          cudaStream_t st, bool pdl) {
    return launch_k(argmax_kernel, dim3(ARGMAX_CTAS), dim3(256), 0, st, pdl, logits, n, pval, pidx, counter, token, out_tokens, sp);
}

}  // namespace b2
