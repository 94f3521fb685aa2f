// The decode attention of one (KV head, key split) unit by a group of 256 threads: the body of the attention kernel
// (decode_ops.cu).
#pragma once
#include <cuda_fp16.h>

#include "async_copy.cuh"
#include "kernels.h"
#include "xplanes.cuh"

namespace b2 {
namespace attend_core {

using namespace acopy;

// Sum over the CTA (every thread calls it; threads with nothing to add pass 0). red: 32 floats of shared memory.
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


// One head of the token's attention inputs: h < nh a query head, then nkv key heads, then nkv value heads. Every thread
// of the CTA calls this (it uses the CTA barrier); thread i < hd owns dimension i. Optional per-head RMS norm, RoPE on
// the first 2 * half_rot dimensions (unfused multiplies and adds, as the CPU's apply_rope), queries to `qo`, keys and
// values to row `pos` of the caches [nkv][max_len][hd]. buf: 256 floats of shared memory.
template <typename T>
__device__ __forceinline__ void rope_head(const uint32_t h, const uint32_t i, const uint32_t pos, const uint32_t table_pos0,
                                          const float* qkv, float* qo, T* kc, T* vc,
                                          const float* __restrict__ qn, const float* __restrict__ kn, const float* __restrict__ cs_table,
                                          const DecRope& p, float* buf, float* red) {
    const uint32_t hd = p.hd;
    const bool on = i < hd;
    const uint32_t kind = h < p.nh ? 0 : (h < p.nh + p.nkv ? 1 : 2);
    const uint32_t hh = kind == 0 ? h : (kind == 1 ? h - p.nh : h - p.nh - p.nkv);
    float v = 0.0f;
    // the vector is rewritten between calls by other SMs (persistent kernel): read it from L2
    if (on) v = __ldcg(kind == 0 ? qkv + hh * p.q_stride + i : (kind == 1 || p.v_from_k) ? qkv + p.k_off + hh * hd + i : qkv + p.v_off + hh * hd + i);
    const bool norm = kind == 0 ? qn != nullptr : (kind == 1 ? kn != nullptr : p.v_norm != 0);
    if (norm) {
        float s = block_sum(v * v, red);
        v = v * (1.0f / sqrtf(s / (float)hd + p.eps));
        if (on && kind == 0) v *= qn[i];
        else if (on && kind == 1) v *= kn[i];
    }
    const bool room = pos < p.max_len;  // a full cache: nothing is written (the host refuses the step before this)
    const size_t at = ((size_t)hh * p.max_len + pos) * hd + i;
    if (on && kind != 2) buf[i] = v;
    __syncthreads();
    if (on && room) {
        if (kind == 2) {
            vc[at] = (T)v;
        } else {
            const uint32_t hr = p.half_rot;
            const float* cs = cs_table + (size_t)(pos - table_pos0) * p.cs_stride + p.cs_off;  // cos[hr] then sin[hr] of this position
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
    }
    __syncthreads();  // buf may be reused by the caller's next head
}

// ---- attention -----------------------------------------------------------------------------------
constexpr int ATT_TILE = 64;         // keys per shared-memory tile
constexpr int ATT_THREADS = 256;
constexpr int ATT_MAX_SPLITS = 64;   // CTAs per KV head at most
__device__ __forceinline__ void group_sync(int bar_id) { asm volatile("bar.sync %0, %1;" ::"r"(bar_id), "r"(ATT_THREADS) : "memory"); }
constexpr long long ATT_WAIT_LIMIT = 2000000000LL;  // cycles (about a second) before a wait on a copy gives up

__device__ __forceinline__ float4 kv4(const float* p) { return *(const float4*)p; }
__device__ __forceinline__ float4 kv4(const __half* p) {
    uint2 r = *(const uint2*)p;
    float2 a = __half22float2(*(const __half2*)&r.x), b = __half22float2(*(const __half2*)&r.y);
    return make_float4(a.x, a.y, b.x, b.y);
}

// How the keys lo .. len - 1 are divided: `per` 64-key tiles per split, `ns` splits (<= max_splits).
__device__ __forceinline__ void attend_splits(uint32_t len, uint32_t window, uint32_t max_splits, uint32_t& lo, uint32_t& tiles, uint32_t& per,
                                              uint32_t& ns) {
    lo = (window != 0 && len > window) ? len - window : 0;
    tiles = (len - lo + ATT_TILE - 1) / ATT_TILE;
    ns = min(tiles, max_splits);
    per = (tiles + ns - 1) / ns;
    ns = (tiles + per - 1) / per;
}

template <int HD, int G, typename T>
__host__ __device__ constexpr size_t attend_smem() {
    size_t tiles = 2 * (size_t)ATT_TILE * HD * sizeof(T);
    size_t red = (size_t)(ATT_THREADS / (HD / 4)) * G * HD * 4;
    size_t first = tiles > red ? tiles : red;
    return first + 16 /* barriers */ + (size_t)G * HD * 4 /* q */ + (size_t)G * ATT_TILE * 4 /* p */ + (size_t)G * ATT_MAX_SPLITS * 4 /* combine weights */
           + 4 * (size_t)G * 4 + 16;
}

// A group of 256 threads (a CTA of the attention kernel; `bar_id` names its barrier) as unit (kvh, split): it runs the G
// query heads of KV head kvh over its share of the key tiles with an online softmax, writes the unnormalized partial (o, m, l) of each head, and the last CTA of a KV head
// to finish (a counter, no waiting) combines the partials, writes `out` and, if asked, the planes of `out`.
template <int HD, int G, typename T>
__device__ __forceinline__ void attend_unit(uint8_t* smem, const int tid, const int bar_id, const int kvh, const int split,
                                            const uint32_t max_splits, const uint32_t pos, const float* q,
                                            const T* kc, const T* vc, float* out, float* part,
                                            uint32_t* counters, DecAttn p, XPlanes xp, uint32_t* status,
                                            unsigned long long* prof = nullptr, const FusedRope* fr = nullptr, const uint32_t table_pos0 = 0,
                                            const bool wait_inside = false) {
    const long long pt0 = clock64();
    auto stamp = [&](int i) {
        if (prof && tid == 0) prof[i] += (unsigned long long)(clock64() - pt0);
    };
    constexpr int COLS = HD / 4, PARTS = ATT_THREADS / COLS, KPP = ATT_TILE / PARTS;
    constexpr size_t TILE_BYTES = 2 * (size_t)ATT_TILE * HD * sizeof(T);
    constexpr size_t RED_BYTES = (size_t)PARTS * G * HD * 4;
    constexpr size_t FIRST = TILE_BYTES > RED_BYTES ? TILE_BYTES : RED_BYTES;
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

    uint32_t len = pos + 1;
    if (len > p.max_len) len = p.max_len;
    uint32_t lo, tiles, per, ns;
    attend_splits(len, p.window, max_splits, lo, tiles, per, ns);
    if ((uint32_t)split >= ns) return;
    const int h0 = kvh * G;
    const float NEG = -INFINITY;

    const uint32_t t0 = split * per, t1 = min(tiles, t0 + per);
    // FusedRope: the unit whose keys end at the token's position makes the token's key and value itself (thread d < HD
    // owns dimension d), appends them to the caches and writes them into its last tile, whose copy leaves that row out.
    const bool makes_row = fr != nullptr && t1 == tiles && pos < p.max_len;
    auto rotate = [&](const float* head, int d) {  // dimension d of a head after RoPE (the arithmetic of rope_head)
        const uint32_t hr = fr->r.half_rot;
        float v = __ldcg(head + d);
        if ((uint32_t)d < 2 * hr) {
            const float* cs = fr->cs_table + (size_t)(pos - table_pos0) * fr->r.cs_stride + fr->r.cs_off;
            if (fr->r.interleaved) {
                const uint32_t j = (uint32_t)d >> 1;
                const float c = cs[j], sn = cs[hr + j];
                const float x1 = __ldcg(head + 2 * j), x2 = __ldcg(head + 2 * j + 1);
                v = (d & 1) == 0 ? __fsub_rn(__fmul_rn(x1, c), __fmul_rn(x2, sn)) : __fadd_rn(__fmul_rn(x2, c), __fmul_rn(x1, sn));
            } else {
                const uint32_t j = (uint32_t)d < hr ? (uint32_t)d : (uint32_t)d - hr;
                const float c = cs[j], sn = cs[hr + j];
                const float x1 = __ldcg(head + j), x2 = __ldcg(head + j + hr);
                v = (uint32_t)d < hr ? __fsub_rn(__fmul_rn(x1, c), __fmul_rn(x2, sn)) : __fadd_rn(__fmul_rn(x2, c), __fmul_rn(x1, sn));
            }
        }
        return v;
    };
    // Without FusedRope the token's row was appended by the kernel ahead: the tile that holds it (the last one) is copied
    // only after the wait.
    const bool late_first = wait_inside && fr == nullptr && t0 == tiles - 1;
    auto issue = [&](uint32_t t) {  // one thread: both copies of key tile t
        const uint32_t j0 = lo + t * ATT_TILE;
        uint32_t nv = min((uint32_t)ATT_TILE, len - j0);
        if (makes_row && t == tiles - 1) nv--;  // the token's own row comes from this unit's registers
        const uint32_t bytes = nv * HD * (uint32_t)sizeof(T);
        const size_t at = ((size_t)kvh * p.max_len + j0) * HD;
        bar_expect_tx(&bars[0], bytes);  // with no bytes to wait for this alone completes the phase
        if (bytes) bulk_load(Ks, kc + at, bytes, &bars[0]);
        bar_expect_tx(&bars[1], bytes);
        if (bytes) bulk_load(Vs, vc + at, bytes, &bars[1]);
    };
    if (tid == 0) {
        bar_init(&bars[0], 1);
        bar_init(&bars[1], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        if (!late_first) issue(t0);  // the first tile is on its way while the queries are staged
        flags[0] = 0;
        flags[1] = 0;
    }
    // wait_inside: the caller has not yet waited for the kernel ahead of it in the stream (programmatic dependent launch).
    // The rows of the caches that this unit copies were written by earlier steps (a step is one graph launch, and the
    // token's own row is left out of the copy), so the first tile's copy starts before the wait; the queries, and the
    // token's key and value, come from the kernel ahead and are read after it.
    if (wait_inside) pdl_wait();
    if (tid == 0 && late_first) issue(t0);
    T k_new = (T)0.0f, v_new = (T)0.0f;
    if (makes_row && tid < HD) {
        k_new = (T)rotate(fr->qkv + fr->r.k_off + (size_t)kvh * HD, tid);
        v_new = (T)__ldcg(fr->qkv + fr->r.v_off + (size_t)kvh * HD + tid);
        const size_t at = ((size_t)kvh * p.max_len + pos) * HD + tid;
        const_cast<T*>(kc)[at] = k_new;
        const_cast<T*>(vc)[at] = v_new;
    }
    if (fr) {
        for (int i = tid; i < G * HD; i += ATT_THREADS)
            qs[i] = rotate(fr->qkv + (size_t)(h0 + i / HD) * fr->r.q_stride, i % HD) * p.scale;
    } else {
        for (int i = tid; i < G * HD; i += ATT_THREADS) qs[i] = __ldcg(q + (size_t)h0 * HD + i) * p.scale;
    }
    if (tid < G) {
        mrun[tid] = NEG;
        lrun[tid] = 0.0f;
    }
    group_sync(bar_id);

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
        group_sync(bar_id);
        if (flags[0]) {
            ok = false;
            break;
        }
        if (makes_row && t == tiles - 1) {  // uniform over the unit's threads
            if (tid < HD) {
                Ks[(pos - j0) * HD + tid] = k_new;
                Vs[(pos - j0) * HD + tid] = v_new;
            }
            group_sync(bar_id);
        }
        if (t == t0) stamp(0);
        // scores: eight lanes per key; a thread takes keys `slot` and `slot + 32` together so that one read of the
        // queries serves both (the queries' shared-memory reads are what bounds this step)
        {
            const int ja = slot, jb = slot + 32;
            const bool va = (uint32_t)ja < nv, vb = (uint32_t)jb < nv;
            const T* ka = Ks + ja * HD;
            const T* kb = Ks + jb * HD;
            float sa[G], sb[G];
#pragma unroll
            for (int g = 0; g < G; g++) sa[g] = sb[g] = 0.0f;
#pragma unroll
            for (int i = 0; i < HD / 32; i++) {
                const int d = lane8 * 4 + 32 * i;
                const float4 k4a = va ? kv4(ka + d) : make_float4(0.f, 0.f, 0.f, 0.f);
                const float4 k4b = vb ? kv4(kb + d) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                for (int g = 0; g < G; g++) {
                    const float4 q4 = *(const float4*)(qs + g * HD + d);
                    sa[g] = fmaf(k4a.x, q4.x, sa[g]);
                    sa[g] = fmaf(k4a.y, q4.y, sa[g]);
                    sa[g] = fmaf(k4a.z, q4.z, sa[g]);
                    sa[g] = fmaf(k4a.w, q4.w, sa[g]);
                    sb[g] = fmaf(k4b.x, q4.x, sb[g]);
                    sb[g] = fmaf(k4b.y, q4.y, sb[g]);
                    sb[g] = fmaf(k4b.z, q4.z, sb[g]);
                    sb[g] = fmaf(k4b.w, q4.w, sb[g]);
                }
            }
#pragma unroll
            for (int g = 0; g < G; g++) {
                float v = sa[g], u = sb[g];
                v += __shfl_xor_sync(0xffffffffu, v, 1);
                u += __shfl_xor_sync(0xffffffffu, u, 1);
                v += __shfl_xor_sync(0xffffffffu, v, 2);
                u += __shfl_xor_sync(0xffffffffu, u, 2);
                v += __shfl_xor_sync(0xffffffffu, v, 4);
                u += __shfl_xor_sync(0xffffffffu, u, 4);
                if (lane8 == 0) {
                    sc[g * ATT_TILE + ja] = va ? v : NEG;
                    sc[g * ATT_TILE + jb] = vb ? u : NEG;
                }
            }
        }
        group_sync(bar_id);
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
        if (t == t0) stamp(1);
        if (!bar_wait(&bars[1], phase)) flags[0] = 1;
        group_sync(bar_id);
        if (flags[0]) {
            ok = false;
            break;
        }
        if (t == t0) stamp(2);
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
        group_sync(bar_id);  // the tile and the probabilities are free again
    }
    if (!ok) {
        // A copy did not arrive in time: record it, give the copies one more bounded wait so that nothing
        // lands in shared memory that has been handed on, and leave without touching the outputs.
        if (tid == 0) {
            atomicExch(status, 1u);
            bar_wait(&bars[0], phase);
            bar_wait(&bars[1], phase);
            bar_inval(&bars[0]);
            bar_inval(&bars[1]);
        }
        return;
    }
    stamp(3);
    if (tid == 0) {  // every thread is past its last wait (the loop ends on a group barrier): the words may be reused
        bar_inval(&bars[0]);
        bar_inval(&bars[1]);
    }

    // partial of this split: sum over the parts, then (o, m, l) per head
#pragma unroll
    for (int g = 0; g < G; g++) *(float4*)(red + ((size_t)part_id * G + g) * HD + c4 * 4) = acc[g];
    group_sync(bar_id);
    for (int idx = tid; idx < G * HD; idx += ATT_THREADS) {
        const int g = idx / HD, d = idx % HD;
        float o = 0.0f;
#pragma unroll
        for (int pp = 0; pp < PARTS; pp++) o += red[((size_t)pp * G + g) * HD + d];
        float* ph = part + ((size_t)(h0 + g) * ATT_MAX_SPLITS + split) * (HD + 4);
        ph[d] = o;
        if (d == 0) {
            ph[HD] = mrun[g];
            ph[HD + 1] = lrun[g];
        }
    }
    __threadfence();
    group_sync(bar_id);
    if (tid == 0) {
        const uint32_t prev = atomicAdd(&counters[kvh], 1u);
        flags[1] = prev == ns - 1;
    }
    group_sync(bar_id);
    stamp(4);
    if (!flags[1]) return;
    __threadfence();
    // combine (the last CTA of this KV head). Every load of a partial is issued before it is needed: the (m, l)
    // pairs of all splits go to shared memory first, the partial outputs are read eight splits at a time.
    float* msm = sc;  // [G][ATT_MAX_SPLITS] maxima (the probabilities are no longer needed)
    float* lsm = qs;  // [G][ATT_MAX_SPLITS] sums (nor are the queries)
    for (int i = tid; i < G * (int)ns; i += ATT_THREADS) {
        const int g = i / (int)ns, sp_ = i - g * (int)ns;
        const float* ph = part + ((size_t)(h0 + g) * ATT_MAX_SPLITS + sp_) * (HD + 4);
        msm[g * ATT_MAX_SPLITS + sp_] = __ldcg(ph + HD);
        lsm[g * ATT_MAX_SPLITS + sp_] = __ldcg(ph + HD + 1);
    }
    group_sync(bar_id);
    for (int i = tid; i < G * (int)ns; i += ATT_THREADS) {
        const int g = i / (int)ns, sp_ = i - g * (int)ns;
        float M = NEG;
        for (uint32_t s2 = 0; s2 < ns; s2++) M = fmaxf(M, msm[g * ATT_MAX_SPLITS + s2]);
        wts[g * ATT_MAX_SPLITS + sp_] = expf(msm[g * ATT_MAX_SPLITS + sp_] - M);
    }
    group_sync(bar_id);
    // The partial outputs: G * HD / 4 columns of four values; the threads form R row groups, group rg adds the splits
    // rg, rg + R, ... of its column (six 16-byte loads in flight at a time), and the groups' sums are added in order.
    {
        constexpr int NC = G * HD / 4, R = ATT_THREADS / NC;
        const int c = tid % NC, rg = tid / NC;
        const int g = (c * 4) / HD, d = (c * 4) % HD;
        const float* ph = part + (size_t)(h0 + g) * ATT_MAX_SPLITS * (HD + 4) + d;
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        for (uint32_t s0 = (uint32_t)rg; s0 < ns; s0 += 6 * R) {
            float4 v[6];
#pragma unroll
            for (int b2 = 0; b2 < 6; b2++) {
                const uint32_t s2 = s0 + (uint32_t)b2 * R;
                v[b2] = s2 < ns ? __ldcg((const float4*)(ph + (size_t)s2 * (HD + 4))) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
#pragma unroll
            for (int b2 = 0; b2 < 6; b2++) {
                const uint32_t s2 = s0 + (uint32_t)b2 * R;
                if (s2 < ns) {
                    const float wgt = wts[g * ATT_MAX_SPLITS + s2];
                    acc.x = fmaf(v[b2].x, wgt, acc.x);
                    acc.y = fmaf(v[b2].y, wgt, acc.y);
                    acc.z = fmaf(v[b2].z, wgt, acc.z);
                    acc.w = fmaf(v[b2].w, wgt, acc.w);
                }
            }
        }
        *(float4*)(red + ((size_t)rg * NC + c) * 4) = acc;
        if (tid < G) {  // the denominators
            float L = 0.0f;
            for (uint32_t s2 = 0; s2 < ns; s2++) L += lsm[tid * ATT_MAX_SPLITS + s2] * wts[tid * ATT_MAX_SPLITS + s2];
            mrun[tid] = L;
        }
        group_sync(bar_id);
        for (int idx = tid; idx < G * HD; idx += ATT_THREADS) {
            float o = 0.0f;
#pragma unroll
            for (int r2 = 0; r2 < R; r2++) o += red[(size_t)r2 * NC * 4 + idx];
            const float r = o / mrun[idx / HD];
            out[(size_t)h0 * HD + idx] = r;
            if (p.planes) xplanes_block(r, (h0 * HD + idx) >> 5, tid & 31, (int)(p.nh * HD), xp);
        }
    }
    stamp(5);
    if (prof && tid == 0) prof[6] += 1;
    if (tid == 0) counters[kvh] = 0;  // ready for the next launch
}

}  // namespace attend_core
}  // namespace b2
