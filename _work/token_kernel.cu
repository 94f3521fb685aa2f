// The persistent token kernel (see token_kernel.h). One CTA of 768 threads per SM, launched cooperatively so that
// all of them are resident; they walk the token's program together.
//
// Waiting. CTAs wait for one another only at grid barriers: an arrival counter in global memory that every CTA's
// first thread increments and then polls. Every poll loop is bounded (clock64): a CTA that waits too long sets the
// abort word, which every other waiter sees, and all CTAs leave the kernel with the status word set.
#include "token_kernel.h"

#include "attend_core.cuh"
#include "dq_core.cuh"
#include "gemv_core.cuh"
#include "gemv_ring.cuh"

namespace b2 {

using namespace gemv_core;
using namespace attend_core;

namespace {

constexpr int TK_THREADS = 768;
constexpr int TK_WARPS = TK_THREADS / 32;
constexpr int TK_GROUPS = TK_THREADS / ATT_THREADS;
constexpr long long TK_BARRIER_LIMIT = 600000000LL;  // cycles (about a third of a second) a CTA waits at a barrier

struct Fixed {  // start of the dynamic shared memory
    TokOp op;   // the op being run (copied from the program)
    float red[32];
    float buf[256];
    float best_v[TK_WARPS];
    int best_i[TK_WARPS];
    int flag;
    int token;
    uint64_t ring_bars[TK_WARPS * 4];  // the warps' ring barriers (up to four slots each)
};
constexpr size_t FIXED_BYTES = (sizeof(Fixed) + 127) / 128 * 128;

__device__ __forceinline__ uint32_t ld_acquire(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// All CTAs of the grid. False: a wait ran out somewhere (the caller returns from the kernel).
__device__ __forceinline__ bool grid_barrier(uint32_t* ctl, uint32_t& target, Fixed* fx) {
    __syncthreads();
    if (threadIdx.x == 0) {
        target += gridDim.x;
        __threadfence();
        atomicAdd(&ctl[0], 1u);
        bool ok = true;
        const long long t0 = clock64();
        uint32_t spin = 0;
        while ((int32_t)(ld_acquire(&ctl[0]) - target) < 0) {
            if ((++spin & 31) == 0) {
                if (ld_acquire(&ctl[1]) != 0) {
                    ok = false;
                    break;
                }
                if (clock64() - t0 > TK_BARRIER_LIMIT) {
                    atomicExch(&ctl[1], 1u);
                    atomicCAS(&ctl[2], 0u, 2u);
                    ok = false;
                    break;
                }
            }
        }
        fx->flag = ok ? 1 : 0;
    }
    __syncthreads();
    return fx->flag != 0;
}

// The shared-memory layout the GEMV code reads (XS, swz): `pl` is [3][K] plane bytes, then {scale, scaled sum} per
// block of 32, then the 16-element integer sums.
__device__ __forceinline__ XS staged(uint8_t* pl, int K) {
    XS xs;
    xs.K = K;
    xs.p0 = pl;
    xs.sx = (const float2*)(pl + 3 * (size_t)K);
    xs.v16 = (const int32_t*)(xs.sx + K / 32);
    xs.xf = nullptr;
    return xs;
}

// Four consecutive values per lane (element k0 .. k0 + 3, k0 a multiple of 4): the eight lanes that hold a block of
// 32 split it together. Same arithmetic per element as xplanes_split; the plane bytes go out as 32-bit words.
__device__ __forceinline__ void stage_quad(float4 t, int k0, int lane, int K, uint8_t* pl) {
    const unsigned m8 = 0xffu << (lane & 24), m4 = 0xfu << (lane & 28);
    const float v[4] = {t.x, t.y, t.z, t.w};
    const float amax = fmaxf(fmaxf(fabsf(t.x), fabsf(t.y)), fmaxf(fabsf(t.z), fabsf(t.w)));
    const float a = __uint_as_float(__reduce_max_sync(m8, __float_as_uint(amax)));
    const float sc = a / XQ_MAX, inv = XQ_MAX / a;
    uint32_t w0 = 0, w1 = 0, w2 = 0;
    int sum = 0;
#pragma unroll
    for (int e = 0; e < 4; e++) {
        int q = a > 0.0f ? __float2int_rn(v[e] * inv) : 0;
        q = max(-(int)XQ_MAX, min((int)XQ_MAX, q));
        const int q0 = ((q + 64) & 127) - 64;
        const int r1 = (q - q0) >> 7;
        const int q1 = ((r1 + 64) & 127) - 64;
        const int q2 = (r1 - q1) >> 7;
        w0 |= (uint32_t)(q0 & 0xff) << (8 * e);
        w1 |= (uint32_t)(q1 & 0xff) << (8 * e);
        w2 |= (uint32_t)(q2 & 0xff) << (8 * e);
        sum += q;
    }
    const int at = (swz(k0 >> 4) << 4) + (k0 & 15);
    *(uint32_t*)(pl + at) = w0;
    *(uint32_t*)(pl + K + at) = w1;
    *(uint32_t*)(pl + 2 * K + at) = w2;
    const int sum16 = __reduce_add_sync(m4, sum), sum32 = __reduce_add_sync(m8, sum);
    float2* sx = (float2*)(pl + 3 * (size_t)K);
    int32_t* v16 = (int32_t*)(sx + K / 32);
    if ((lane & 3) == 0) v16[k0 >> 4] = sum16;
    if ((lane & 7) == 0) sx[k0 >> 5] = make_float2(sc, sc * (float)sum32);
}

// RMSNorm of one row (norm_kernel's arithmetic), every CTA for itself: the row's planes land in shared memory.
// A thread holds two runs of four consecutive values (rows of up to 8 * 768).
__device__ __forceinline__ void norm_stage(const TokOp& op, Fixed* fx, uint8_t* pl, unsigned long long* prof) {
    const long long pt0 = clock64();
    const DecNorm& p = op.norm;
    const int tid = threadIdx.x;
    float4 v[2], wv[2];
    float s = 0.0f;
#pragma unroll
    for (int j = 0; j < 2; j++) {
        const uint32_t i = (tid + j * TK_THREADS) * 4;
        v[j] = i < p.n ? __ldcg((const float4*)(op.x + i)) : make_float4(0.f, 0.f, 0.f, 0.f);
        wv[j] = (i < p.n && op.p0) ? *(const float4*)(op.p0 + i) : make_float4(1.f, 1.f, 1.f, 1.f);
        v[j].x *= p.pre;
        v[j].y *= p.pre;
        v[j].z *= p.pre;
        v[j].w *= p.pre;
        s += v[j].x * v[j].x;
        s += v[j].y * v[j].y;
        s += v[j].z * v[j].z;
        s += v[j].w * v[j].w;
    }
    if (prof && tid == 0) prof[0] += (unsigned long long)(clock64() - pt0);
    const float k = 1.0f / sqrtf(block_sum(s, fx->red) / (float)p.n + p.eps);
    if (prof && tid == 0) prof[1] += (unsigned long long)(clock64() - pt0);
#pragma unroll
    for (int j = 0; j < 2; j++) {
        const uint32_t i = (tid + j * TK_THREADS) * 4;
        if (i < p.n) {  // p.n % 32 == 0: the eight lanes of a block are all here
            float4 t = make_float4(v[j].x * k, v[j].y * k, v[j].z * k, v[j].w * k);
            if (op.p0) t = make_float4(t.x * wv[j].x, t.y * wv[j].y, t.z * wv[j].z, t.w * wv[j].w);
            if (blockIdx.x == 0) *(float4*)(op.y + i) = t;
            stage_quad(t, (int)i, tid & 31, (int)p.n, pl);
        }
    }
    __syncthreads();
}

__device__ __forceinline__ void stage_vector(const float* x, int n, uint8_t* pl) {
    const int tid = threadIdx.x, quads = n / 4;
    for (int q0 = tid; q0 < quads; q0 += TK_THREADS * 4) {  // four loads in flight per lane (the vector sits in L2)
        float4 v[4];
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int q = q0 + j * TK_THREADS;
            v[j] = q < quads ? __ldcg((const float4*)x + q) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int q = q0 + j * TK_THREADS;
            if (q < quads) stage_quad(v[j], q * 4, tid & 31, n, pl);
        }
    }
    __syncthreads();
}

// Planes another phase left in global memory -> this CTA's shared memory (the staging step of gemv_kernel).
__device__ __forceinline__ void copy_planes(const XPlanes& xp, int K, uint8_t* pl) {
    xplanes_stage(xp, K, pl, threadIdx.x, TK_THREADS);
    __syncthreads();
}

// Rows of the matrix spread over every warp of the grid; the arithmetic of gemv_kernel.
template <class F, bool PAIR>
__device__ __forceinline__ void gemv_rows(const TokOp& op, const XS& xs) {
    const WeightDev& w = op.w;
    const int K = (int)w.n_in;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const size_t n_out = w.n_out;
    const int iters = (K + F::ITER_K - 1) / F::ITER_K;
    constexpr int RW = PAIR ? 1 : 2;
    // warps of one CTA take rows far apart, so that the CTAs' share of rows is even for any row count
    const size_t r_first = ((size_t)warp * gridDim.x + blockIdx.x) * RW, r_step = (size_t)gridDim.x * TK_WARPS * RW;
    float* y = op.y;
    for (size_t r0 = r_first; r0 < n_out; r0 += r_step) {
        const size_t rowB = PAIR ? r0 : min(r0 + 1, n_out - 1);
        float accA = 0.0f, accB = 0.0f;
        for (int it = 0; it < iters; it++) {
            if (!F::active(K, it, lane)) continue;
            typename F::Regs ra, rb;
            F::load(w, r0, it, lane, ra);
            F::load(PAIR ? op.w2 : w, rowB, it, lane, rb);
            F::dot2(ra, rb, xs, it, lane, accA, accB);
        }
        accA = warp_sum(accA);
        accB = warp_sum(accB);
        if (lane == 0) {
            if (PAIR) {
                y[r0] = (op.mode == B2_MODE_SILU_PAIR ? silu(accA) : gelu_tanh(accA)) * accB;
            } else {
#pragma unroll
                for (int r = 0; r < 2; r++) {
                    if (r0 + r >= n_out) break;
                    const float a = r ? accB : accA;
                    float* o = y + r0 + r;
                    if (op.mode == B2_MODE_STORE)
                        *o = a;
                    else if (op.mode == B2_MODE_ADD)
                        *o += a;
                    else
                        *o += a * (1.0f / (1.0f + __expf(-op.z[0])));
                }
            }
        }
    }
}

template <class F>
__device__ __forceinline__ void gemv_fmt(const TokOp& op, const XS& xs) {
    if (op.pair) gemv_rows<F, true>(op, xs);
    else gemv_rows<F, false>(op, xs);
}

// The 4-bit formats: weights through the warp's ring of bulk copies (gemv_ring.cuh).
template <class F>
__device__ __forceinline__ bool gemv_ring_fmt(const TokOp& op, const XS& xs, WarpRing& ring) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const size_t rw = op.pair ? 1 : 2;
    const size_t r_first = ((size_t)warp * gridDim.x + blockIdx.x) * rw, r_step = (size_t)gridDim.x * TK_WARPS * rw;
    if (op.pair) return gemv4_ring<F, true>(op.w, op.w2, xs, op.y, (int)op.mode, op.z, ring, r_first, r_step, lane);
    return gemv4_ring<F, false>(op.w, op.w2, xs, op.y, (int)op.mode, op.z, ring, r_first, r_step, lane);
}

template <int HD, int G, typename T>
__device__ __forceinline__ void attend_all(const TokOp& op, const TokenArgs& a, uint32_t pos, uint8_t* work) {
    const DecAttn& p = op.attn;
    uint32_t len = pos + 1;
    if (len > p.max_len) len = p.max_len;
    uint32_t lo, tiles, per, ns;
    attend_splits(len, p.window, a.max_splits, lo, tiles, per, ns);
    const int group = threadIdx.x / ATT_THREADS, gtid = threadIdx.x % ATT_THREADS;
    constexpr size_t GROUP_BYTES = (attend_smem<HD, G, T>() + 127) / 128 * 128;
    uint8_t* gsm = work + (size_t)group * GROUP_BYTES;
    // unit u = (KV head, split); consecutive units go to different SMs
    for (uint32_t u = (uint32_t)group * gridDim.x + blockIdx.x; u < p.nkv * ns; u += TK_GROUPS * gridDim.x)
        attend_unit<HD, G, T>(gsm, gtid, 1 + group, (int)(u / ns), (int)(u % ns), a.max_splits, pos, op.x, (const T*)op.kc, (const T*)op.vc,
                              op.y, a.part, a.att_counters, p, op.xp, &a.ctl[2],
                              (a.prof && blockIdx.x == 0 && group == 0) ? a.prof + 72 : nullptr);
    __syncthreads();
}

template <int HD, typename T>
__device__ __forceinline__ void attend_g(const TokOp& op, const TokenArgs& a, uint32_t pos, uint8_t* work) {
    switch (op.attn.nh / op.attn.nkv) {
        case 1: attend_all<HD, 1, T>(op, a, pos, work); break;
        case 2: attend_all<HD, 2, T>(op, a, pos, work); break;
        case 4: attend_all<HD, 4, T>(op, a, pos, work); break;
    }
}

template <int FMT>
__device__ __forceinline__ void embed_fmt(const WeightDev& w, size_t row, float* out) {
    const size_t chunks = w.n_in / 8;
    for (size_t c = (size_t)blockIdx.x * TK_THREADS + threadIdx.x; c < chunks; c += (size_t)gridDim.x * TK_THREADS) {
        float v[8];
        dequant8<FMT>(w, row, c * 8, v);
        float4* o = (float4*)(out + c * 8);
        o[0] = make_float4(v[0], v[1], v[2], v[3]);
        o[1] = make_float4(v[4], v[5], v[6], v[7]);
    }
}

__device__ __forceinline__ void best_of(float& b, int& ix, float ob, int oi) {
    if (ob > b || (ob == b && oi < ix)) {
        b = ob;
        ix = oi;
    }
}
__device__ __forceinline__ void warp_best(float& b, int& ix) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        float ob = __shfl_xor_sync(0xffffffffu, b, o);
        int oi = __shfl_xor_sync(0xffffffffu, ix, o);
        best_of(b, ix, ob, oi);
    }
}

__global__ void __launch_bounds__(TK_THREADS, 1) token_kernel(TokenArgs a) {
    extern __shared__ __align__(128) uint8_t smem[];
    Fixed* fx = (Fixed*)smem;
    uint8_t* work = smem + FIXED_BYTES;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    uint32_t target = 0;
    // the warp's ring: slots behind the planes (the attention tiles use the same memory at other times)
    WarpRing ring;
    ring.S = (int)a.ring_slots;
    ring.slots = work + a.ring_offset + (size_t)warp * a.ring_slots * RING_SLOT_BYTES;
    ring.bars = fx->ring_bars + warp * 4;
    ring.phases = 0;
    if (lane == 0)
        for (int sl = 0; sl < ring.S; sl++) bar_init(&ring.bars[sl], 1);
    if (tid == 0) asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    __syncthreads();
    for (uint32_t tok = 0; tok < a.n_tokens; tok++) {
        const uint32_t pos = a.pos0 + tok;
        if (a.with_head) {
            // the token's embedding row -> the graph's input (every CTA a slice), then the ops
            int t = tok == 0 ? (int)a.first_token : fx->token;
            const size_t row = (t >= 0 && (size_t)t < a.embed.n_out) ? (size_t)t : 0;
            switch (a.embed.fmt) {
                case B2_FMT_MLX4: embed_fmt<B2_FMT_MLX4>(a.embed, row, a.input); break;
                case B2_FMT_Q4_K: embed_fmt<B2_FMT_Q4_K>(a.embed, row, a.input); break;
                case B2_FMT_Q6_K: embed_fmt<B2_FMT_Q6_K>(a.embed, row, a.input); break;
                case B2_FMT_Q8_0: embed_fmt<B2_FMT_Q8_0>(a.embed, row, a.input); break;
                case B2_FMT_F8E4M3: embed_fmt<B2_FMT_F8E4M3>(a.embed, row, a.input); break;
            }
            if (!grid_barrier(a.ctl, target, fx)) return;
        }
        for (uint32_t pc = 0; pc < a.n_ops; pc++) {
            __syncthreads();  // the previous op is done with fx->op
            for (uint32_t i = tid; i < sizeof(TokOp) / 4; i += TK_THREADS) ((uint32_t*)&fx->op)[i] = ((const uint32_t*)&a.prog[pc])[i];
            __syncthreads();
            const TokOp& op = fx->op;
            const long long prof_t0 = clock64();
            switch (op.kind) {
                case TK_BARRIER:
                    if (!grid_barrier(a.ctl, target, fx)) return;
                    break;
                case TK_NORM_STAGE: norm_stage(op, fx, work, (a.prof && blockIdx.x == 0) ? a.prof + 64 : nullptr); break;
                case TK_STAGE: stage_vector(op.x, (int)op.n, work); break;
                case TK_COPY: copy_planes(op.xp, (int)op.n, work); break;
                case TK_XPLANES:
                    for (uint32_t blk = (uint32_t)warp * gridDim.x + blockIdx.x; blk < op.n / 32; blk += gridDim.x * TK_WARPS)
                        xplanes_block(__ldcg(op.x + blk * 32 + lane), (int)blk, lane, (int)op.n, op.xp);
                    break;
                case TK_GEMV: {
                    const XS xs = staged(work, (int)op.w.n_in);
                    bool ok = true;
                    switch (op.w.fmt) {
                        case B2_FMT_MLX4: ok = gemv_ring_fmt<FmtMLX4>(op, xs, ring); break;
                        case B2_FMT_Q4_K: ok = gemv_ring_fmt<FmtQ4K>(op, xs, ring); break;
                        case B2_FMT_Q6_K: gemv_fmt<FmtQ6K>(op, xs); break;
                        case B2_FMT_Q8_0: gemv_fmt<FmtQ8_0>(op, xs); break;
                    }
                    if (!ok) {  // a copy did not arrive: every CTA leaves at its next barrier
                        atomicExch(&a.ctl[1], 1u);
                        atomicCAS(&a.ctl[2], 0u, 3u);
                    }
                    break;
                }
                case TK_ROPE:
                    for (uint32_t h = blockIdx.x; h < op.rope.nh + 2 * op.rope.nkv; h += gridDim.x) {
                        if (op.kv_f16)
                            rope_head<__half>(h, tid, pos, a.table_pos0, op.x, op.y, (__half*)op.kc, (__half*)op.vc, op.p0, op.p1, a.cs_table, op.rope,
                                              fx->buf, fx->red);
                        else
                            rope_head<float>(h, tid, pos, a.table_pos0, op.x, op.y, (float*)op.kc, (float*)op.vc, op.p0, op.p1, a.cs_table, op.rope,
                                             fx->buf, fx->red);
                    }
                    break;
                case TK_ATTEND:
                    if (op.attn.hd == 64) {
                        if (op.kv_f16) attend_g<64, __half>(op, a, pos, work);
                        else attend_g<64, float>(op, a, pos, work);
                    } else {
                        if (op.kv_f16) attend_g<128, __half>(op, a, pos, work);
                        else attend_g<128, float>(op, a, pos, work);
                    }
                    break;
                case TK_GLU:
                    for (uint32_t i = blockIdx.x * TK_THREADS + tid; i < op.n; i += gridDim.x * TK_THREADS) {
                        const float g = __ldcg(op.x + i);
                        float r;
                        if (op.gelu) {
                            const float K2 = 2.0f * 0.7978846f;
                            const float t = K2 * (g + 0.044715f * g * g * g);
                            r = g / (1.0f + expf(-t));
                        } else {
                            r = g / (1.0f + expf(-g));
                        }
                        op.y[i] = r * __ldcg(op.z + i);
                    }
                    break;
            }
            if (a.prof && blockIdx.x == 0 && tid == 0) {
                a.prof[op.kind & 15] += (unsigned long long)(clock64() - prof_t0);
                a.prof[16 + (op.kind & 15)] += 1;
                if (pc < 32) a.prof[32 + pc] += (unsigned long long)(clock64() - prof_t0);  // the first layer, op by op
            }
        }
        if (a.with_head) {
            // greedy token: every CTA its slice of the logits, partials through global memory, every CTA reduces them
            if (!grid_barrier(a.ctl, target, fx)) return;
            float best = -INFINITY;
            int bi = 0x7fffffff;
            for (uint32_t i = blockIdx.x * TK_THREADS + tid; i < a.n_logits; i += gridDim.x * TK_THREADS) best_of(best, bi, __ldcg(a.logits + i), (int)i);
            warp_best(best, bi);
            if (lane == 0) {
                fx->best_v[warp] = best;
                fx->best_i[warp] = bi;
            }
            __syncthreads();
            if (warp == 0) {
                best = lane < TK_WARPS ? fx->best_v[lane] : -INFINITY;
                bi = lane < TK_WARPS ? fx->best_i[lane] : 0x7fffffff;
                warp_best(best, bi);
                if (lane == 0) {
                    a.argmax_val[blockIdx.x] = best;
                    a.argmax_idx[blockIdx.x] = bi;
                }
            }
            if (!grid_barrier(a.ctl, target, fx)) return;
            if (warp == 0) {
                best = -INFINITY;
                bi = 0x7fffffff;
                for (uint32_t i = lane; i < gridDim.x; i += 32) best_of(best, bi, __ldcg(a.argmax_val + i), __ldcg(a.argmax_idx + i));
                warp_best(best, bi);
                if (lane == 0) {
                    if (bi == 0x7fffffff) bi = 0;  // every logit NaN or -inf
                    fx->token = bi;
                    if (blockIdx.x == 0) {
                        a.token[0] = bi;
                        a.out_tokens[tok] = bi;
                    }
                }
            }
            __syncthreads();
        }
    }
}

template <int HD, typename T>
constexpr size_t att_bytes(uint32_t g) {
    return g == 1 ? attend_smem<HD, 1, T>() : g == 2 ? attend_smem<HD, 2, T>() : attend_smem<HD, 4, T>();
}

}  // namespace

bool token_kernel_attend_ok(uint32_t nh, uint32_t nkv, uint32_t hd) {
    if (nkv == 0 || nh % nkv) return false;
    const uint32_t g = nh / nkv;
    return (hd == 64 || hd == 128) && (g == 1 || g == 2 || g == 4);
}

size_t token_kernel_ring_offset(size_t max_k) { return (xplanes_bytes(max_k) + 127) / 128 * 128; }
size_t token_kernel_ring_bytes(uint32_t slots) { return (size_t)TK_WARPS * slots * RING_SLOT_BYTES; }
size_t token_kernel_fixed_bytes() { return FIXED_BYTES; }

size_t token_kernel_smem(size_t max_k, uint32_t hd, uint32_t g, int kv_f16) {
    size_t att = 0;
    if (hd == 64) att = kv_f16 ? att_bytes<64, __half>(g) : att_bytes<64, float>(g);
    else if (hd == 128) att = kv_f16 ? att_bytes<128, __half>(g) : att_bytes<128, float>(g);
    att = (att + 127) / 128 * 128;  // each group's region starts on a 128-byte boundary
    size_t work = std::max(xplanes_bytes(max_k), TK_GROUPS * att);
    return FIXED_BYTES + (work + 127) / 128 * 128;
}

cudaError_t launch_token_kernel(const TokenArgs& args, size_t smem, int sm_count, cudaStream_t st) {
    static size_t smem_set = 0;
    if (smem > smem_set) {
        cudaError_t e = cudaFuncSetAttribute(token_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
        smem_set = smem;
    }
    int per_sm = 0;
    cudaError_t e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, token_kernel, TK_THREADS, smem);
    if (e != cudaSuccess) return e;
    if (per_sm < 1) return cudaErrorLaunchOutOfResources;
    TokenArgs a = args;
    void* params[] = {&a};
    return cudaLaunchCooperativeKernel((const void*)token_kernel, dim3((unsigned)sm_count), dim3(TK_THREADS), params, smem, st);
}

}  // namespace b2
