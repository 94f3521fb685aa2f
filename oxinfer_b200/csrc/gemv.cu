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
// A warp owns two weight rows at a time (or, for the fused SiLU / GELU pair, the same row of the
// gate and the up matrix): every lane issues the 16-byte weight loads of both before using either,
// and reads its slice of the activation planes from shared memory once for both. The planes are
// staged once per CTA, with their 16-byte slots permuted so that the eight lanes of a shared-memory
// phase, which read 64 bytes each at a 64-byte stride, fall on different banks.
#include <cuda_fp8.h>

#include <algorithm>
#include <cstdio>
#include <cstdlib>

#include "gemv_core.cuh"
#include "gemv_ring.cuh"

namespace b2 {

using namespace gemv_core;

namespace {

constexpr int GEMV_THREADS = 256;
constexpr int GEMV_WARPS = GEMV_THREADS / 32;

// ---- activation planes ----------------------------------------------------------------------
// blockIdx.y: the token of a step of several tokens (its vector, planes and norm sums a fixed stride behind token 0's).
struct TokenStrides {
    size_t x, planes, partial;  // floats, bytes, floats
};
__device__ __forceinline__ XPlanes planes_of_token(XPlanes p, size_t bytes) {
    p.planes = (int8_t*)((uint8_t*)p.planes + bytes);
    p.sx = (float2*)((uint8_t*)p.sx + bytes);
    p.v16 = (int32_t*)((uint8_t*)p.v16 + bytes);
    return p;
}

__global__ void __launch_bounds__(256) xplanes_kernel(const float* __restrict__ x, int K, XPlanes out, TokenStrides ts) {
    int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    pdl_launch_dependents();
    pdl_wait();
    if (warp >= K / 32) return;
    xplanes_block(x[(size_t)blockIdx.y * ts.x + warp * 32 + lane], warp, lane, K, planes_of_token(out, (size_t)blockIdx.y * ts.planes));
}

// planes(x * pre * w) without the norm factor, and each block's sum of squares of x * pre (see NormScale). A warp per block.
__global__ void __launch_bounds__(256) norm_planes_kernel(const float* __restrict__ x, const float* __restrict__ w, float pre, int K, XPlanes out,
                                                          float* __restrict__ partial, TokenStrides ts) {
    pdl_launch_dependents();
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    const float wv = (w && warp < K / 32) ? w[warp * 32 + lane] : 1.0f;  // the weights do not depend on the kernel ahead
    pdl_wait();
    if (warp >= K / 32) return;
    const float v = x[(size_t)blockIdx.y * ts.x + warp * 32 + lane] * pre;
    float s = v * v;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (lane == 0) partial[(size_t)blockIdx.y * ts.partial + warp] = s;
    xplanes_block(v * wv, warp, lane, K, planes_of_token(out, (size_t)blockIdx.y * ts.planes));
}

// The kernel's order of events, chosen for back-to-back launches of a decode step:
//   1. let the next kernel of the stream start launching (programmatic dependent launch),
//   2. issue the loads of the warp's first weights, which depend on nothing the previous kernel wrote,
//   3. wait for the previous kernel (it wrote the planes / the vector), stage them in shared memory,
//   4. stream the rows.
// NT tokens at once (Backend::matvec_rows, up to four; the reference's dmvk_* kernels, src/cuda_decode.cu:176-232): the
// weights are read once and every token keeps its own accumulators, with the single-token arithmetic, so each row of the
// result equals the one-token result bit for bit. Token i's vector / planes sit multi.x_stride after token i - 1's
// (floats for the f32 vector, bytes for the planes), its outputs multi.y_stride floats after.
struct GemvMulti {
    size_t x_stride, y_stride;
    size_t ns_stride;  // floats between the tokens' blocks of norm partial sums (NormScale), when there is a factor
};

template <class F, bool PAIR, bool XF32, int NT>
__global__ void __launch_bounds__(GEMV_THREADS, NT > 2 ? 2 : 3)
gemv_kernel(WeightDev w, WeightDev w2, const float* __restrict__ x, XPlanes xp, float* __restrict__ y, int mode,
            const float* __restrict__ gate, NormScale ns, GemvBatch batch, GemvMulti multi) {
    extern __shared__ __align__(128) uint8_t smem[];
    pdl_launch_dependents();
    if (batch.n) {  // entry blockIdx.y of a batch: its matrix of the stack, its planes, its output
        const size_t b = blockIdx.y, e = (size_t)batch.expert[b];
        w.p0 += e * batch.w_stride;
        w2.p0 += e * batch.w_stride;
        xp = xplanes_at(batch.planes + (size_t)batch.xrow[b] * batch.x_stride, w.n_in);
        y += b * batch.y_stride;
    }
    const int K = (int)w.n_in;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const size_t n_out = w.n_out;
    const int iters = (K + F::ITER_K - 1) / F::ITER_K;
    constexpr int RW = PAIR ? 1 : 2;  // output rows per warp pass
    const size_t r_first = ((size_t)blockIdx.x * GEMV_WARPS + warp) * RW, r_step = (size_t)gridDim.x * GEMV_WARPS * RW;
    typename F::Regs na, nb;
    auto fetch = [&](size_t r0, int it) {
        if (F::active(K, it, lane)) {
            F::load(w, r0, it, lane, na);
            F::load(PAIR ? w2 : w, PAIR ? r0 : min(r0 + 1, n_out - 1), it, lane, nb);
        }
    };
    if (r_first < n_out) fetch(r_first, 0);
    pdl_wait();

    XS xs[NT];
    const size_t per_tok = ((XF32 ? (size_t)K * 4 : xplanes_bytes((size_t)K)) + 127) / 128 * 128;
#pragma unroll
    for (int tk = 0; tk < NT; tk++) {
        uint8_t* sm = smem + (size_t)tk * per_tok;
        xs[tk].K = K;
        if constexpr (XF32) {
            float* xf = (float*)sm;
            const float* xt = x + (size_t)tk * multi.x_stride;
            for (int g = threadIdx.x; g < K / 4; g += GEMV_THREADS) ((float4*)xf)[swz(g)] = ((const float4*)xt)[g];
            xs[tk].xf = xf;
            xs[tk].p0 = nullptr;
            xs[tk].sx = nullptr;
            xs[tk].v16 = nullptr;
        } else {
            const XPlanes xpt = tk == 0 ? xp : xplanes_at((uint8_t*)xp.planes + (size_t)tk * multi.x_stride, (size_t)K);
            xplanes_stage(xpt, K, sm, threadIdx.x, GEMV_THREADS);
            xs[tk].p0 = sm;
            xs[tk].sx = (const float2*)(sm + 3 * (size_t)K);
            xs[tk].v16 = (const int32_t*)(xs[tk].sx + K / 32);
            xs[tk].xf = nullptr;
        }
    }
    __syncthreads();
    float kscale[NT];
#pragma unroll
    for (int tk = 0; tk < NT; tk++) {
        NormScale nt = ns;
        if (nt.partial) nt.partial += (size_t)tk * multi.ns_stride;
        kscale[tk] = norm_scale_factor(nt, lane);
    }
    for (size_t r0 = r_first; r0 < n_out; r0 += r_step) {
        float accA[NT], accB[NT];
#pragma unroll
        for (int tk = 0; tk < NT; tk++) accA[tk] = accB[tk] = 0.0f;
        for (int it = 0; it < iters; it++) {
            if (!F::active(K, it, lane)) continue;
            if (it > 0 || r0 != r_first) fetch(r0, it);  // the first step's loads were issued before the wait
#pragma unroll
            for (int tk = 0; tk < NT; tk++) F::dot2(na, nb, xs[tk], it, lane, accA[tk], accB[tk]);
        }
#pragma unroll
        for (int tk = 0; tk < NT; tk++) {
            const float sa = warp_sum(accA[tk]) * kscale[tk], sb = warp_sum(accB[tk]) * kscale[tk];
            float* yt = y + (size_t)tk * multi.y_stride;
            if (lane == 0) {
                if (PAIR) {
                    yt[r0] = (mode == B2_MODE_SILU_PAIR ? silu(sa) : gelu_tanh(sa)) * sb;
                } else {
#pragma unroll
                    for (int r = 0; r < 2; r++) {
                        if (r0 + r >= n_out) break;
                        const float a = r ? sb : sa;
                        float* o = yt + r0 + r;
                        if (mode == B2_MODE_STORE)
                            *o = a;
                        else if (mode == B2_MODE_ADD)
                            *o += a;
                        else
                            *o += a * (1.0f / (1.0f + __expf(-gate[0])));
                    }
                }
            }
        }
    }
}

// ---- several tokens of a 4-bit product with the integer dots on the tensor cores -------------------------------------------
// The exact products are bound by instruction issue: 0.75 dp4a per weight and token. mma.sync.m16n8k32 (u8 x s8 -> s32)
// makes the same integer sums, which do not depend on the order of their terms: A = the nibbles of 16 weight rows over one
// block of 32 k (a byte each), B = that block of the planes, column n = (token n / 2, plane n & 1) and, in a second
// instruction, (token n / 2, the third plane) in the even columns. A lane (g, c) then holds, for rows g and g + 8 and token c,
// the three plane sums of the block; the float tail per row, token and 64-group is the one-token kernel's own
// (F::tail), fed the same integers, so the results keep their bits.
// The one-token kernel gives the 64-group (block b, group j) to lane 4 (b % 8) + j of the row's warp, which adds its
// groups in the order of b and then takes part in a butterfly sum. Here a CTA takes 16 rows and its warp w the blocks
// b % 8 == w: it keeps the four accumulators 4 w + j of every (row, token) it holds, adding in the same order, and the 32
// accumulators of a (row, token) meet in shared memory, where one thread adds them in the butterfly's order.
__device__ __forceinline__ void imma_16832(int (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

constexpr int IMMA_ROWS = 16, IMMA_THREADS = 256;

__device__ __forceinline__ void cp_async_16(void* smem_dst, const void* src) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(smem_dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
constexpr int IMMA_TILE_BYTES = IMMA_ROWS * 144;  // one 256-block of 16 rows, packed

// HALVES = 2: 16 warps, two groups of 16 rows at a time (for vectors whose planes leave room for one CTA per SM only).
// RING: every warp brings its next (block, matrix) tile of packed weights into its own two shared-memory buffers with cp.async
// while it works on the current one (the kernel is bound by the latency of those loads otherwise).
template <class F, bool PAIR, int NT, int NP, int HALVES, bool RING>
__global__ void __launch_bounds__(IMMA_THREADS * HALVES, HALVES == 1 ? 2 : 1) gemv4_imma_kernel(WeightDev w, WeightDev w2, XPlanes xp, float* __restrict__ y, int mode,
                                                                  NormScale ns, GemvMulti multi) {
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr int NM = PAIR ? 2 : 1;
    pdl_launch_dependents();
    const int K = (int)w.n_in, nblk = K / 256;
    const size_t n_out = w.n_out;
    const int half = (int)(threadIdx.x >> 8), tid = (int)(threadIdx.x & 255);  // the half's own 8 warps
    const int warp = tid >> 5, lane = tid & 31, g = lane >> 2, c = lane & 3;
    pdl_wait();
    const size_t per_tok = (xplanes_bytes((size_t)K) + 127) / 128 * 128;
#pragma unroll
    for (int tk = 0; tk < NT; tk++) {
        const XPlanes xpt = tk == 0 ? xp : xplanes_at((uint8_t*)xp.planes + (size_t)tk * multi.x_stride, (size_t)K);
        xplanes_stage(xpt, K, smem + (size_t)tk * per_tok, threadIdx.x, IMMA_THREADS * HALVES);
    }
    float kscale[NT];
#pragma unroll
    for (int tk = 0; tk < NT; tk++) {
        NormScale nt = ns;
        if (nt.partial) nt.partial += (size_t)tk * multi.ns_stride;
        kscale[tk] = norm_scale_factor(nt, lane);
    }
    __syncthreads();
    // this lane's column of B: token g / 2, plane (g & 1) of the first instruction's two planes; the third plane in even columns
    const bool bcol = (g >> 1) < NT;
    const uint8_t* btok = smem + (size_t)min(g >> 1, NT - 1) * per_tok;
    const uint8_t* bp1 = btok + (size_t)((NP == 3 ? 0 : 1) + (g & 1)) * K;
    const uint8_t* bp2 = btok + (size_t)2 * K;
    const bool b2col = bcol && (g & 1) == 0;
    // this lane's token in the accumulators: c (lanes with c >= NT carry sums that are never stored)
    const float2* sx_t = (const float2*)(smem + (size_t)min(c, NT - 1) * per_tok + 3 * (size_t)K);
    // [matrix][row 16][token 4][accumulator 32] per half, behind the planes
    float* comb = (float*)(smem + (size_t)NT * per_tok) + (size_t)half * NM * IMMA_ROWS * 4 * 32;
    const size_t groups = (n_out + IMMA_ROWS - 1) / IMMA_ROWS;
    auto half_sync = [&] {  // the 256 threads of this half (the halves run on their own, each with its named barrier)
        if (HALVES == 1) __syncthreads();
        else asm volatile("bar.sync %0, 256;" ::"r"(1 + half) : "memory");
    };
    // The planes are staged once per CTA; each half of the CTA then takes groups of 16 rows in turn.
    for (size_t grp = (size_t)blockIdx.x * HALVES + half; grp < groups; grp += (size_t)gridDim.x * HALVES) {
        const size_t row0 = grp * IMMA_ROWS;
        const size_t rows_ld[2] = {min(row0 + g, n_out - 1), min(row0 + g + 8, n_out - 1)};  // rows past the end repeat the last one (never stored)
        float acc[NM][2][4];
#pragma unroll
        for (int m = 0; m < NM; m++)
#pragma unroll
            for (int r = 0; r < 2; r++) acc[m][r][0] = acc[m][r][1] = acc[m][r][2] = acc[m][r][3] = 0.0f;
        // RING: tile (b, m) of this warp = the 144 packed bytes of block b of the group's 16 rows of matrix m
        uint8_t* wbuf = smem + (size_t)NT * per_tok + (size_t)HALVES * NM * IMMA_ROWS * 4 * 32 * sizeof(float) + (size_t)warp * 2 * IMMA_TILE_BYTES;
        auto issue = [&](int b, int m, int buf) {
            const uint8_t* wp = m ? w2.p0 : w.p0;
            for (int q = lane; q < IMMA_ROWS * 9; q += 32) {
                const int row = q / 9, part = q - row * 9;
                cp_async_16(wbuf + (size_t)buf * IMMA_TILE_BYTES + row * 144 + part * 16,
                            wp + (min(row0 + row, n_out - 1) * (size_t)nblk + b) * 144 + part * 16);
            }
            cp_async_commit();
        };
        int buf = 0;
        if (RING && warp < nblk) issue(warp, 0, 0);
        for (int b = warp; b < nblk; b += 8) {
#pragma unroll
            for (int m = 0; m < NM; m++) {  // (a pair: one matrix after the other, so that only one's words are live)
                // the block's loads first, all of them in flight together: two headers and 16 words of nibbles
                Q4Regs hd[2];
                uint32_t wq[2][4][2];  // [row][group][word]: bytes 4 c .. and 16 + 4 c .. of the group's 32
                if constexpr (RING) {
                    const int nb = m == NM - 1 ? b + 8 : b, nm = m == NM - 1 ? 0 : m + 1;  // the tile behind this one
                    if (nb < nblk) {
                        issue(nb, nm, buf ^ 1);
                        cp_async_wait<1>();
                    } else {
                        cp_async_wait<0>();
                    }
                    __syncwarp();  // every lane's copies of this tile have landed
                    const uint8_t* tile = wbuf + (size_t)buf * IMMA_TILE_BYTES;
#pragma unroll
                    for (int r = 0; r < 2; r++) {
                        const uint8_t* blk = tile + (g + 8 * r) * 144;
                        hd[r].hdr = *(const uint4*)blk;
#pragma unroll
                        for (int j = 0; j < 4; j++) {
                            wq[r][j][0] = *(const uint32_t*)(blk + 16 + 32 * j + 4 * c);
                            wq[r][j][1] = *(const uint32_t*)(blk + 32 + 32 * j + 4 * c);
                        }
                    }
                    __syncwarp();  // the buffer may be overwritten by the copies issued in the next round
                    buf ^= 1;
                } else {
#pragma unroll
                    for (int r = 0; r < 2; r++) {
                        const uint8_t* blk = (m ? w2.p0 : w.p0) + (rows_ld[r] * (size_t)nblk + b) * 144;
                        hd[r].hdr = __ldg((const uint4*)blk);
#pragma unroll
                        for (int j = 0; j < 4; j++) {
                            wq[r][j][0] = __ldg((const uint32_t*)(blk + 16 + 32 * j + 4 * c));
                            wq[r][j][1] = __ldg((const uint32_t*)(blk + 32 + 32 * j + 4 * c));
                        }
                    }
                }
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    const int k0 = b * 256 + 64 * j;
                    const float4 sx = *(const float4*)(sx_t + (k0 >> 5));  // {scale, sum} of the two blocks of this lane's token
                    int lo[2], hi[2];
#pragma unroll
                    for (int h = 0; h < 2; h++) {
                        // B: bytes 4 c .. 4 c + 3 and 16 + 4 c .. of the block of 32 (low nibbles: k0, high: k0 + 32)
                        const int ka = k0 + 32 * h;
                        const size_t o0 = ((size_t)swz(ka >> 4) << 4) + 4 * c, o1 = ((size_t)swz((ka >> 4) + 1) << 4) + 4 * c;
                        const uint32_t b10 = bcol ? *(const uint32_t*)(bp1 + o0) : 0u, b11 = bcol ? *(const uint32_t*)(bp1 + o1) : 0u;
                        const uint32_t a[4] = {(wq[0][j][0] >> (4 * h)) & 0x0F0F0F0Fu, (wq[1][j][0] >> (4 * h)) & 0x0F0F0F0Fu,
                                               (wq[0][j][1] >> (4 * h)) & 0x0F0F0F0Fu, (wq[1][j][1] >> (4 * h)) & 0x0F0F0F0Fu};
                        int s1[4] = {0, 0, 0, 0}, s2[4] = {0, 0, 0, 0};
                        imma_16832(s1, a, b10, b11);
                        if (NP == 3) {
                            const uint32_t b20 = b2col ? *(const uint32_t*)(bp2 + o0) : 0u, b21 = b2col ? *(const uint32_t*)(bp2 + o1) : 0u;
                            imma_16832(s2, a, b20, b21);
                        }
                        // columns 2 c, 2 c + 1 of the first instruction = this lane's token, its two planes; column 2 c of the second = the third
                        const int va = NP == 3 ? planes_sum<3>(s1[0], s1[1], s2[0]) : planes_sum<2>(0, s1[0], s1[1]);
                        const int vb = NP == 3 ? planes_sum<3>(s1[2], s1[3], s2[2]) : planes_sum<2>(0, s1[2], s1[3]);
                        if (h) {
                            hi[0] = va;
                            hi[1] = vb;
                        } else {
                            lo[0] = va;
                            lo[1] = vb;
                        }
                    }
                    F::tail(hd[0], j, sx, lo[0], hi[0], acc[m][0][j]);
                    F::tail(hd[1], j, sx, lo[1], hi[1], acc[m][1][j]);
                }
            }
        }
        if (c < NT) {
#pragma unroll
            for (int m = 0; m < NM; m++)
#pragma unroll
                for (int r = 0; r < 2; r++)
#pragma unroll
                    for (int j = 0; j < 4; j++) comb[(((size_t)m * 16 + g + 8 * r) * 4 + c) * 32 + 4 * warp + j] = acc[m][r][j];
        }
        half_sync();
        if (tid < IMMA_ROWS * NT) {
            const int r = tid / NT, tk = tid % NT;
            float tot[NM];
#pragma unroll
            for (int m = 0; m < NM; m++) {
                float a[32];
#pragma unroll
                for (int i = 0; i < 32; i++) a[i] = comb[(((size_t)m * 16 + r) * 4 + tk) * 32 + i];
#pragma unroll
                for (int o = 16; o > 0; o >>= 1)  // the butterfly of warp_sum, as lane 0 sees it
#pragma unroll
                    for (int i = 0; i < o; i++) a[i] += a[i + o];
                float ks = kscale[0];
#pragma unroll
                for (int i = 1; i < NT; i++)
                    if (tk == i) ks = kscale[i];
                tot[m] = a[0] * ks;
            }
            if (row0 + r < n_out) {
                float* o = y + (size_t)tk * multi.y_stride + row0 + r;
                if (PAIR)
                    *o = (mode == B2_MODE_SILU_PAIR ? silu(tot[0]) : gelu_tanh(tot[0])) * tot[NM - 1];
                else if (mode == B2_MODE_STORE)
                    *o = tot[0];
                else
                    *o += tot[0];
            }
        }
        half_sync();  // the accumulators' shared memory is free for the next group
    }
}

// The 4-bit formats: the same products with the weights brought in by bulk copies into per-warp rings (gemv_ring.cuh).
// The first copies are issued before the kernel waits for the one ahead of it in the stream.
constexpr int RING_SLOTS = 3;
constexpr int RING_SLOTS_MAX = 4;
constexpr size_t RING_BYTES = (size_t)GEMV_WARPS * RING_SLOTS * RING_SLOT_BYTES;

// WARPS = 8: rows interleaved over the grid's warps. With an epilogue (EpiPlanes) a CTA owns whole blocks of 32 rows,
// 32 / WARPS per warp; WARPS = 16 then keeps two rows per warp, the depth of the plain form.
template <class F, bool PAIR, int WARPS>
__global__ void __launch_bounds__(WARPS * 32, WARPS == 8 ? 3 : 1)
gemv4_ring_kernel(WeightDev w, WeightDev w2, XPlanes xp, float* __restrict__ y, int mode, const float* __restrict__ gate, uint32_t* status,
                  NormScale ns, EpiPlanes epi, int slots_per_warp) {
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ uint64_t bars[WARPS * RING_SLOTS_MAX];
    __shared__ uint64_t xbars[RING_X_STEPS];
    __shared__ float epi_vals[2 * 32];
    constexpr int THREADS = WARPS * 32;
    pdl_launch_dependents();
    const int K = (int)w.n_in;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    constexpr int RW = PAIR ? 1 : 2;
    const bool with_epi = epi.out.planes != nullptr;
    const uint32_t ni = with_epi ? (uint32_t)max(1, 32 / WARPS / RW) : 1;
    const size_t r_first = with_epi ? (size_t)blockIdx.x * 32 + (size_t)warp * (32 / WARPS) : ((size_t)warp * gridDim.x + blockIdx.x) * RW;
    const size_t r_step = with_epi ? (size_t)gridDim.x * 32 : (size_t)gridDim.x * WARPS * RW;
    const size_t planes_bytes = (xplanes_bytes((size_t)K) + 127) / 128 * 128;
    WarpRing ring;
    ring.S = slots_per_warp;
    ring.slots = smem + planes_bytes + (size_t)warp * slots_per_warp * RING_SLOT_BYTES;
    ring.bars = bars + warp * RING_SLOTS_MAX;
    ring.phases = 0;
    if (lane == 0) {
        for (int sl = 0; sl < slots_per_warp; sl++) acopy::bar_init(&ring.bars[sl], 1);
        if (warp == 0)
            for (int i = 0; i < (K / 256 + 7) / 8; i++) acopy::bar_init(&xbars[i], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        ring_prime<PAIR>(w, w2, ring, r_first, r_step, ni);
    }
    pdl_wait();
    // the planes of x (written by the kernel ahead) -> shared memory, a set of bulk copies per 2048 k: the rows start once
    // the first set has landed
    if (threadIdx.x == 0) ring_stage_planes(xp, K, smem, xbars);
    __syncthreads();  // the barrier words are initialized for every warp
    XS xs;
    xs.K = K;
    xs.p0 = smem;
    xs.sx = (const float2*)(smem + 3 * (size_t)K);
    xs.v16 = (const int32_t*)(xs.sx + K / 32);
    xs.xf = nullptr;
    const float kscale = norm_scale_factor(ns, lane);
    if (!gemv4_ring<F, PAIR>(w, w2, xs, y, mode, gate, ring, r_first, r_step, lane, true, kscale, ni, epi, epi_vals, THREADS, xbars) && status)
        atomicExch(status, 5u);
}

static int env_int(const char* name, int dflt) {
    const char* e = getenv(name);
    return e ? atoi(e) : dflt;
}

template <class F, bool PAIR, int WARPS>
cudaError_t launch_ring_w(const WeightDev& w, const WeightDev* up, XPlanes xp, float* y, int mode, const float* gate, int sm_count,
                          cudaStream_t st, bool pdl, NormScale ns, EpiPlanes epi, int slots) {
    auto kern = gemv4_ring_kernel<F, PAIR, WARPS>;
    const size_t smem = (xplanes_bytes(w.n_in) + 127) / 128 * 128 + (size_t)WARPS * slots * RING_SLOT_BYTES;
    if (smem + 2048 > 227 * 1024) return cudaErrorInvalidValue;
    if (cudaError_t e = ensure_dynamic_smem((const void*)kern, smem); e != cudaSuccess) return e;
    const size_t rows_per_cta = epi.out.planes ? 32 : (size_t)WARPS * (PAIR ? 1 : 2);
    const size_t groups = (w.n_out + rows_per_cta - 1) / rows_per_cta;
    size_t per_sm = (size_t)(224 * 1024) / (smem + 2048);
    const size_t cap = (size_t)(2048 / (WARPS * 32)) < 3 ? (size_t)(2048 / (WARPS * 32)) : 3;
    per_sm = per_sm < 1 ? 1 : (per_sm > cap ? cap : per_sm);
    if (WARPS != 8) per_sm = 1;  // the launch bounds of the wide form
    const size_t grid = groups < (size_t)sm_count * per_sm ? groups : (size_t)sm_count * per_sm;
    return launch_k(kern, dim3((unsigned)grid), dim3(WARPS * 32), smem, st, pdl, w, PAIR ? *up : w, xp, y, mode, gate, (uint32_t*)nullptr, ns, epi,
                    slots);
}

template <class F>
cudaError_t launch_ring_f(const WeightDev& w, const WeightDev* up, XPlanes xp, float* y, int mode, const float* gate, int sm_count,
                          cudaStream_t st, bool pdl, NormScale ns, EpiPlanes epi) {
    const bool pair = mode == B2_MODE_SILU_PAIR || mode == B2_MODE_GELU_PAIR;
    if (epi.out.planes) {
        static const int warps = env_int("B2_EPI_WARPS", 16), slots = std::min(RING_SLOTS_MAX, std::max(2, env_int("B2_EPI_SLOTS", 3)));
        if (warps == 16) {
            const size_t smem = (xplanes_bytes(w.n_in) + 127) / 128 * 128 + (size_t)16 * slots * RING_SLOT_BYTES;
            if (smem + 2048 <= 227 * 1024)
                return pair ? launch_ring_w<F, true, 16>(w, up, xp, y, mode, gate, sm_count, st, pdl, ns, epi, slots)
                            : launch_ring_w<F, false, 16>(w, up, xp, y, mode, gate, sm_count, st, pdl, ns, epi, slots);
        }
    }
    static const int plain_slots = std::min(RING_SLOTS_MAX, std::max(2, env_int("B2_RING_SLOTS", RING_SLOTS)));
    return pair ? launch_ring_w<F, true, 8>(w, up, xp, y, mode, gate, sm_count, st, pdl, ns, epi, plain_slots)
                : launch_ring_w<F, false, 8>(w, up, xp, y, mode, gate, sm_count, st, pdl, ns, epi, plain_slots);
}

// FT<3> reads all three planes of x, FT<2> the upper two (XPlanes::np).
template <template <int> class FT>
cudaError_t launch_ring(const WeightDev& w, const WeightDev* up, XPlanes xp, float* y, int mode, const float* gate, int sm_count,
                        cudaStream_t st, bool pdl, NormScale ns, EpiPlanes epi) {
    return xp.np == 2 ? launch_ring_f<FT<2>>(w, up, xp, y, mode, gate, sm_count, st, pdl, ns, epi)
                      : launch_ring_f<FT<3>>(w, up, xp, y, mode, gate, sm_count, st, pdl, ns, epi);
}

// ---- FP8 e4m3 weights on the tensor cores ---------------------------------------------------------------------
// The float path above spends about three instructions per weight (convert, widen, multiply-add) and reads four
// bytes of x per weight from shared memory: a third of the HBM rate at best. Here the multiply-adds run as
// mma.sync m16n8k16 (f16 operands, f32 accumulate): a warp owns 16 weight rows, A is the weights (hardware
// e4m3x2 -> f16x2, exact), B's column 0 is x rounded to f16 and column 1 the f16 of the rounding remainder, so
// that x enters with 22 bits and the two columns' sums are added at the end; the other six columns are zero.
// The summation index of an MMA may be permuted freely as long as A and B agree, so a lane loads 16 consecutive
// bytes of its row (k = 64 c + 16 t ..) and feeds them to four MMAs. The block scale (one per 128 x 128 block)
// multiplies the accumulators once per 128 k.
__device__ __forceinline__ void mma_f16_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void f8x16_to_h2(const uint4& q, uint32_t (&h)[8]) {
    const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int i = 0; i < 4; i++) {
        __half2_raw lo = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(w[i] & 0xffff), __NV_E4M3);
        __half2_raw hi = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(w[i] >> 16), __NV_E4M3);
        h[2 * i] = *reinterpret_cast<uint32_t*>(&lo);
        h[2 * i + 1] = *reinterpret_cast<uint32_t*>(&hi);
    }
}

constexpr int F8M_CHUNK = 64;  // k per step of a warp: 16 bytes per lane and row

// A CTA owns one 16-row tile at a time; its eight warps split K (whole 128-k scale blocks each) and their partial sums
// meet in shared memory, added in warp order.
__global__ void __launch_bounds__(GEMV_THREADS, 3)
gemv_f8_mma_kernel(WeightDev w, const float* __restrict__ x, float* __restrict__ y, int mode, const float* __restrict__ gate) {
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ float part[GEMV_WARPS][16];
    pdl_launch_dependents();
    const int K = (int)w.n_in;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const size_t n_out = w.n_out;
    __half* xh = (__half*)smem;   // [K] x rounded to f16
    __half* xl = xh + K;          // [K] f16 of the remainder
    // this warp's share of the scale blocks: blocks [kb0, kb1)
    const int nblk = K / 128;
    const int kb0 = (int)((long long)nblk * warp / GEMV_WARPS), kb1 = (int)((long long)nblk * (warp + 1) / GEMV_WARPS);
    const int ch0 = 2 * kb0, ch1 = 2 * kb1;  // chunks of 64 k
    pdl_wait();
    // x times a power of two that brings its largest magnitude into [2^14, 2^15): vectors of any magnitude stay inside f16's
    // range and out of its subnormals; the results are scaled back (exactly) when they are written
    float mx = 0.0f;
    for (int i = threadIdx.x; i < K; i += GEMV_THREADS) mx = fmaxf(mx, fabsf(x[i]));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    if (lane == 0) part[warp][0] = mx;
    __syncthreads();
    mx = part[0][0];
#pragma unroll
    for (int i = 1; i < GEMV_WARPS; i++) mx = fmaxf(mx, part[i][0]);
    __syncthreads();
    float xscale = 1.0f, xinv = 1.0f;
    if (mx > 0.0f && mx < INFINITY) {
        int e;
        frexpf(mx, &e);
        const int up = min(100, max(-100, 15 - e));
        xscale = ldexpf(1.0f, up);
        xinv = ldexpf(1.0f, -up);
    }
    for (int i = threadIdx.x; i < K; i += GEMV_THREADS) {
        const float v = x[i] * xscale;
        const __half h = __float2half_rn(v);
        xh[i] = h;
        xl[i] = __float2half_rn(v - __half2float(h));
    }
    __syncthreads();
    const __half* xb = g == 0 ? xh : xl;  // lanes of column 0 read x, of column 1 the remainder, the rest feed zeros
    const size_t tiles = (n_out + 15) / 16;
    for (size_t tile = blockIdx.x; tile < tiles; tile += gridDim.x) {
        const size_t r0 = tile * 16;
        const size_t rowA = min(r0 + g, n_out - 1), rowB = min(r0 + g + 8, n_out - 1);
        const uint8_t* pa = w.p0 + rowA * (size_t)K + 16 * t;
        const uint8_t* pb = w.p0 + rowB * (size_t)K + 16 * t;
        const float* srow = w.p1 ? (const float*)w.p1 + ((w.bs_row0 + r0) / w.bs_rows) * w.bs_ncb : nullptr;
        float acc[4] = {0.f, 0.f, 0.f, 0.f}, c[4] = {0.f, 0.f, 0.f, 0.f};
        // four chunks of loads in flight ahead of the arithmetic
        uint4 qa[4], qb[4];
#pragma unroll
        for (int i = 0; i < 4; i++)
            if (ch0 + i < ch1) {
                qa[i] = ldg_stream(pa + (size_t)(ch0 + i) * F8M_CHUNK);
                qb[i] = ldg_stream(pb + (size_t)(ch0 + i) * F8M_CHUNK);
            }
        for (int base = ch0; base < ch1; base += 4) {
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const int ch = base + i;
                if (ch >= ch1) break;
                const uint4 ca = qa[i], cb = qb[i];
                if (ch + 4 < ch1) {
                    qa[i] = ldg_stream(pa + (size_t)(ch + 4) * F8M_CHUNK);
                    qb[i] = ldg_stream(pb + (size_t)(ch + 4) * F8M_CHUNK);
                }
                uint32_t ha[8], hb[8];
                f8x16_to_h2(ca, ha);
                f8x16_to_h2(cb, hb);
                uint4 b01 = make_uint4(0, 0, 0, 0), b23 = make_uint4(0, 0, 0, 0);
                if (g < 2) {
                    const uint4* src = (const uint4*)(xb + ch * F8M_CHUNK + 16 * t);
                    b01 = src[0];
                    b23 = src[1];
                }
                const uint32_t bw[8] = {b01.x, b01.y, b01.z, b01.w, b23.x, b23.y, b23.z, b23.w};
#pragma unroll
                for (int m = 0; m < 4; m++) mma_f16_16816(c, ha[2 * m], hb[2 * m], ha[2 * m + 1], hb[2 * m + 1], bw[2 * m], bw[2 * m + 1]);
                if ((ch & 1) == 1) {  // the end of a 128-k scale block
                    const float s = srow ? __ldg(srow + (ch >> 1)) : 1.0f;
                    acc[0] = fmaf(c[0], s, acc[0]);
                    acc[1] = fmaf(c[1], s, acc[1]);
                    acc[2] = fmaf(c[2], s, acc[2]);
                    acc[3] = fmaf(c[3], s, acc[3]);
                    c[0] = c[1] = c[2] = c[3] = 0.f;
                }
            }
        }
        if (t == 0) {  // columns 0 and 1 of rows g and g + 8
            part[warp][g] = acc[0] + acc[1];
            part[warp][g + 8] = acc[2] + acc[3];
        }
        __syncthreads();
        if (threadIdx.x < 16) {
            const size_t r = r0 + threadIdx.x;
            if (r < n_out) {
                float v = 0.0f;
#pragma unroll
                for (int wv = 0; wv < GEMV_WARPS; wv++) v += part[wv][threadIdx.x];
                v *= xinv;
                float* o = y + r;
                if (mode == B2_MODE_STORE)
                    *o = v;
                else if (mode == B2_MODE_ADD)
                    *o += v;
                else
                    *o += v * (1.0f / (1.0f + __expf(-gate[0])));
            }
        }
        __syncthreads();
    }
}

static bool f8_mma_ok(const WeightDev& w, int mode) {
    if (mode == B2_MODE_SILU_PAIR || mode == B2_MODE_GELU_PAIR) return false;
    if (w.n_in % 128 || w.n_in < 128 * GEMV_WARPS || w.n_in * 4 > 200 * 1024) return false;
    if (w.p1 && (w.bs_cols != 128 || w.bs_rows % 16 || w.bs_row0 % 16)) return false;
    return true;
}

static cudaError_t launch_f8_mma(const WeightDev& w, const float* x, float* y, int mode, const float* gate, int sm_count, cudaStream_t st, bool pdl) {
    const size_t smem = w.n_in * 4;  // two f16 copies of x
    // the kernel also has static shared memory: ask early
    if (cudaError_t e = ensure_dynamic_smem((const void*)gemv_f8_mma_kernel, smem, 40 * 1024); e != cudaSuccess) return e;
    const size_t tiles = (w.n_out + 15) / 16;
    size_t per_sm = (size_t)(220 * 1024) / (smem + 2048);
    per_sm = per_sm < 1 ? 1 : (per_sm > 3 ? 3 : per_sm);
    const size_t grid = tiles < (size_t)sm_count * per_sm ? tiles : (size_t)sm_count * per_sm;
    return launch_k(gemv_f8_mma_kernel, dim3((unsigned)grid), dim3(GEMV_THREADS), smem, st, pdl, w, x, y, mode, gate);
}

template <class F, bool XF32, int NT>
cudaError_t launch_fmt_f(const WeightDev& w, const WeightDev* up, const float* x, XPlanes xp, float* y, int mode, const float* gate,
                         int sm_count, cudaStream_t st, bool pdl, NormScale ns, GemvMulti multi) {
    size_t smem = (((XF32 ? w.n_in * 4 : xplanes_bytes(w.n_in)) + 127) / 128 * 128) * NT;
    bool pair = mode == B2_MODE_SILU_PAIR || mode == B2_MODE_GELU_PAIR;
    auto kern = pair ? gemv_kernel<F, true, XF32, NT> : gemv_kernel<F, false, XF32, NT>;
    if (cudaError_t e = ensure_dynamic_smem((const void*)kern, smem); e != cudaSuccess) return e;
    const size_t rows_per_cta = (size_t)GEMV_WARPS * (pair ? 1 : 2);
    size_t groups = (w.n_out + rows_per_cta - 1) / rows_per_cta;
    size_t per_sm = (size_t)(220 * 1024) / (smem + 1024);
    per_sm = per_sm < 1 ? 1 : (per_sm > 3 ? 3 : per_sm);
    size_t grid = groups < (size_t)sm_count * per_sm ? groups : (size_t)sm_count * per_sm;
    return launch_k(kern, dim3((unsigned)grid), dim3(GEMV_THREADS), smem, st, pdl, w, pair ? *up : w, x, xp, y, mode, gate, ns, GemvBatch{}, multi);
}

template <template <int> class FT, bool XF32, int NT = 1>
cudaError_t launch_fmt(const WeightDev& w, const WeightDev* up, const float* x, XPlanes xp, float* y, int mode, const float* gate,
                       int sm_count, cudaStream_t st, bool pdl, NormScale ns, GemvMulti multi = GemvMulti{0, 0, 0}) {
    if (XF32 || xp.np != 2) return launch_fmt_f<FT<3>, XF32, NT>(w, up, x, xp, y, mode, gate, sm_count, st, pdl, ns, multi);
    return launch_fmt_f<FT<XF32 ? 3 : 2>, XF32, NT>(w, up, x, xp, y, mode, gate, sm_count, st, pdl, ns, multi);
}

}  // namespace

bool gemv_supports(const WeightDev& w) {
    switch (w.fmt) {
        case B2_FMT_MLX4:
        case B2_FMT_Q4_K:
        case B2_FMT_Q6_K: return w.n_in % 256 == 0 && xplanes_bytes(w.n_in) <= 200 * 1024;
        case B2_FMT_Q8_0: return w.n_in % 64 == 0 && xplanes_bytes(w.n_in) <= 200 * 1024;
        case B2_FMT_F8E4M3: return w.n_in % 16 == 0 && w.n_in * 4 <= 200 * 1024 && (w.p1 == nullptr || w.bs_cols % 16 == 0);
        default: return false;
    }
}

cudaError_t launch_xplanes(const float* x, size_t K, XPlanes out, cudaStream_t st, bool pdl, int tokens, size_t x_stride, size_t planes_stride) {
    unsigned warps = (unsigned)(K / 32);
    if (tokens < 1) return cudaErrorInvalidValue;
    return launch_k(xplanes_kernel, dim3((warps + 7) / 8, (unsigned)tokens), dim3(256), 0, st, pdl, x, (int)K, out, TokenStrides{x_stride, planes_stride, 0});
}

__global__ void __launch_bounds__(256) xplanes_rows_kernel(const float* __restrict__ x, int rows, int K, uint8_t* planes, size_t stride) {
    pdl_launch_dependents();
    pdl_wait();
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    const int per_row = K / 32;
    if (warp >= rows * per_row) return;
    const int r = warp / per_row, blk = warp - r * per_row;
    xplanes_block(x[(size_t)r * K + blk * 32 + lane], blk, lane, K, xplanes_at(planes + (size_t)r * stride, (size_t)K));
}

cudaError_t launch_xplanes_rows(const float* x, size_t rows, size_t K, uint8_t* planes, size_t stride, cudaStream_t st, bool pdl) {
    if (rows == 0 || K % 32) return cudaErrorInvalidValue;
    const unsigned warps = (unsigned)(rows * (K / 32));
    return launch_k(xplanes_rows_kernel, dim3((warps + 7) / 8), dim3(256), 0, st, pdl, x, (int)rows, (int)K, planes, stride);
}

template <class F>
static cudaError_t launch_batched_fmt(const WeightDev& w, const WeightDev* up, const GemvBatch& b, size_t batch, float* y, int mode, int sm_count,
                                      cudaStream_t st, bool pdl) {
    const bool pair = mode == B2_MODE_SILU_PAIR || mode == B2_MODE_GELU_PAIR;
    auto kern = pair ? gemv_kernel<F, true, false, 1> : gemv_kernel<F, false, false, 1>;
    const size_t smem = (xplanes_bytes(w.n_in) + 127) / 128 * 128;
    if (cudaError_t e = ensure_dynamic_smem((const void*)kern, smem); e != cudaSuccess) return e;
    const size_t rows_per_cta = (size_t)GEMV_WARPS * (pair ? 1 : 2);
    size_t gx = (w.n_out + rows_per_cta - 1) / rows_per_cta;
    const size_t cap = std::max<size_t>(1, (size_t)sm_count * 3 / batch);  // about three CTAs per SM over the whole batch
    if (gx > cap) gx = cap;
    XPlanes none{};
    return launch_k(kern, dim3((unsigned)gx, (unsigned)batch), dim3(GEMV_THREADS), smem, st, pdl, w, pair ? *up : w, (const float*)nullptr, none, y, mode,
                    (const float*)nullptr, NormScale{nullptr, 0, 0.0f, 0.0f}, b, GemvMulti{0, 0, 0});
}

cudaError_t launch_gemv_batched(const WeightDev& w, const WeightDev* up, const GemvBatch& b, size_t batch, float* y, int mode, int np, int sm_count,
                                cudaStream_t st, bool pdl) {
    if (batch == 0 || batch > GEMV_BATCH_MAX || (size_t)b.n != batch || !gemv_supports(w)) return cudaErrorInvalidValue;
    if (w.fmt == B2_FMT_MLX4)
        return np == 2 ? launch_batched_fmt<FmtMLX4_T<2>>(w, up, b, batch, y, mode, sm_count, st, pdl) : launch_batched_fmt<FmtMLX4_T<3>>(w, up, b, batch, y, mode, sm_count, st, pdl);
    if (w.fmt == B2_FMT_Q4_K)
        return np == 2 ? launch_batched_fmt<FmtQ4K_T<2>>(w, up, b, batch, y, mode, sm_count, st, pdl) : launch_batched_fmt<FmtQ4K_T<3>>(w, up, b, batch, y, mode, sm_count, st, pdl);
    return cudaErrorInvalidValue;
}

template <int NT>
static cudaError_t launch_multi_nt(const WeightDev& w, const WeightDev* up, const float* x, XPlanes xp, float* y, int mode, int sm_count,
                                   cudaStream_t st, GemvMulti m, bool pdl, NormScale ns) {
    switch (w.fmt) {
        case B2_FMT_MLX4: return launch_fmt<FmtMLX4_T, false, NT>(w, up, x, xp, y, mode, nullptr, sm_count, st, pdl, ns, m);
        case B2_FMT_Q4_K: return launch_fmt<FmtQ4K_T, false, NT>(w, up, x, xp, y, mode, nullptr, sm_count, st, pdl, ns, m);
        case B2_FMT_Q6_K: return launch_fmt<FmtQ6K_T, false, NT>(w, up, x, xp, y, mode, nullptr, sm_count, st, pdl, ns, m);
        case B2_FMT_Q8_0: return launch_fmt<FmtQ8_0_T, false, NT>(w, up, x, xp, y, mode, nullptr, sm_count, st, pdl, ns, m);
        case B2_FMT_F8E4M3: return launch_fmt<FmtF8_T, true, NT>(w, up, x, xp, y, mode, nullptr, sm_count, st, pdl, ns, m);
        default: return cudaErrorInvalidValue;
    }
}

template <class F, int NT>
static cudaError_t launch_imma_nt(const WeightDev& w, const WeightDev* up, XPlanes xp, float* y, int mode, int sm_count, cudaStream_t st, GemvMulti m,
                                  bool pdl, NormScale ns) {
    const bool pair = mode == B2_MODE_SILU_PAIR || mode == B2_MODE_GELU_PAIR;
    const bool np2 = xp.np == 2;
    const size_t per_tok = (xplanes_bytes(w.n_in) + 127) / 128 * 128;
    const size_t comb = (size_t)(pair ? 2 : 1) * IMMA_ROWS * 4 * 32 * sizeof(float);
    // planes that leave room for one CTA per SM only: 16 warps in that CTA instead of 8
    const bool wide = per_tok * NT + comb + 1024 > 112 * 1024 && per_tok * NT + 2 * comb <= 224 * 1024;
    // room for the warps' weight buffers beside two CTAs per SM: the cp.async form
    const size_t ring_bytes = (size_t)8 * 2 * IMMA_TILE_BYTES;
    static const bool ring_on = env_int("B2_GEMV_IMMA_RING", 1) != 0;
    const bool ring = ring_on && !wide && per_tok * NT + comb + ring_bytes + 1024 <= 112 * 1024;
    const size_t smem = per_tok * NT + (wide ? 2 : 1) * comb + (ring ? ring_bytes : 0);
    if (smem > 224 * 1024) return cudaErrorInvalidValue;
    void (*kern)(WeightDev, WeightDev, XPlanes, float*, int, NormScale, GemvMulti);
    if (wide)
        kern = pair ? (np2 ? gemv4_imma_kernel<F, true, NT, 2, 2, false> : gemv4_imma_kernel<F, true, NT, 3, 2, false>)
                    : (np2 ? gemv4_imma_kernel<F, false, NT, 2, 2, false> : gemv4_imma_kernel<F, false, NT, 3, 2, false>);
    else if (ring)
        kern = pair ? (np2 ? gemv4_imma_kernel<F, true, NT, 2, 1, true> : gemv4_imma_kernel<F, true, NT, 3, 1, true>)
                    : (np2 ? gemv4_imma_kernel<F, false, NT, 2, 1, true> : gemv4_imma_kernel<F, false, NT, 3, 1, true>);
    else
        kern = pair ? (np2 ? gemv4_imma_kernel<F, true, NT, 2, 1, false> : gemv4_imma_kernel<F, true, NT, 3, 1, false>)
                    : (np2 ? gemv4_imma_kernel<F, false, NT, 2, 1, false> : gemv4_imma_kernel<F, false, NT, 3, 1, false>);
    if (cudaError_t e = ensure_dynamic_smem((const void*)kern, smem); e != cudaSuccess) return e;
    const size_t groups = (w.n_out + IMMA_ROWS - 1) / IMMA_ROWS;
    size_t per_sm = (size_t)(224 * 1024) / (smem + 1024);
    per_sm = per_sm < 1 ? 1 : (per_sm > 3 ? 3 : per_sm);
    const size_t halves = wide ? 2 : 1;
    const size_t grid = std::min((groups + halves - 1) / halves, (size_t)sm_count * per_sm);
    return launch_k(kern, dim3((unsigned)grid), dim3((unsigned)(IMMA_THREADS * halves)), smem, st, pdl, w, pair ? *up : w, xp, y, mode, ns, m);
}

// B2_GEMV_IMMA=0: the several-token 4-bit products on the dp4a kernel (for A/B runs; the results are the same bits).
static bool imma_enabled() {
    static const bool on = env_int("B2_GEMV_IMMA", 1) != 0;
    return on;
}

bool gemv_multi_pays(const WeightDev& w, int nt) {
    const bool tensor = imma_enabled() && (w.fmt == B2_FMT_Q4_K || w.fmt == B2_FMT_MLX4);
    return gemv_multi_fits(w, nt) && nt >= (tensor ? 2 : 3);
}

bool gemv_multi_fits(const WeightDev& w, int nt) {
    const size_t per = ((w.fmt == B2_FMT_F8E4M3 ? w.n_in * 4 : xplanes_bytes(w.n_in)) + 127) / 128 * 128;
    return nt >= 1 && nt <= 4 && gemv_supports(w) && per * (size_t)nt <= 200 * 1024;
}

cudaError_t launch_gemv_multi(const WeightDev& w, const WeightDev* up, const float* x, size_t x_stride, XPlanes xp, size_t xp_stride, float* y,
                              size_t y_stride, int nt, int mode, int sm_count, cudaStream_t st, bool pdl, NormScale ns, size_t ns_stride) {
    const bool f8 = w.fmt == B2_FMT_F8E4M3;
    if (!gemv_multi_fits(w, nt) || mode == B2_MODE_ADD_GATED) return cudaErrorInvalidValue;  // no gate pointer travels here
    const GemvMulti m{f8 ? x_stride : xp_stride, y_stride, ns_stride};
    const size_t imma_smem = (xplanes_bytes(w.n_in) + 127) / 128 * 128 * (size_t)nt + 2 * IMMA_ROWS * 4 * 32 * sizeof(float);  // (the pair's)
    if (nt >= 2 && imma_enabled() && (w.fmt == B2_FMT_Q4_K || w.fmt == B2_FMT_MLX4) && imma_smem <= 224 * 1024) {  // the integer dots on the tensor cores
        const bool q4k = w.fmt == B2_FMT_Q4_K;
        switch (nt) {
            case 2: return q4k ? launch_imma_nt<FmtQ4K_T<3>, 2>(w, up, xp, y, mode, sm_count, st, m, pdl, ns) : launch_imma_nt<FmtMLX4_T<3>, 2>(w, up, xp, y, mode, sm_count, st, m, pdl, ns);
            case 3: return q4k ? launch_imma_nt<FmtQ4K_T<3>, 3>(w, up, xp, y, mode, sm_count, st, m, pdl, ns) : launch_imma_nt<FmtMLX4_T<3>, 3>(w, up, xp, y, mode, sm_count, st, m, pdl, ns);
            default: return q4k ? launch_imma_nt<FmtQ4K_T<3>, 4>(w, up, xp, y, mode, sm_count, st, m, pdl, ns) : launch_imma_nt<FmtMLX4_T<3>, 4>(w, up, xp, y, mode, sm_count, st, m, pdl, ns);
        }
    }
    switch (nt) {
        case 1: return launch_multi_nt<1>(w, up, x, xp, y, mode, sm_count, st, m, pdl, ns);
        case 2: return launch_multi_nt<2>(w, up, x, xp, y, mode, sm_count, st, m, pdl, ns);
        case 3: return launch_multi_nt<3>(w, up, x, xp, y, mode, sm_count, st, m, pdl, ns);
        default: return launch_multi_nt<4>(w, up, x, xp, y, mode, sm_count, st, m, pdl, ns);
    }
}

cudaError_t launch_norm_planes(const float* x, const float* w, float pre, size_t K, XPlanes out, float* partial, cudaStream_t st, bool pdl, int tokens,
                               size_t x_stride, size_t planes_stride, size_t partial_stride) {
    if (K == 0 || K % 32 || tokens < 1) return cudaErrorInvalidValue;
    unsigned warps = (unsigned)(K / 32);
    return launch_k(norm_planes_kernel, dim3((warps + 7) / 8, (unsigned)tokens), dim3(256), 0, st, pdl, x, w, pre, (int)K, out, partial,
                    TokenStrides{x_stride, planes_stride, partial_stride});
}

static int ring_level() {  // B2_GEMV_RING: 0 never, 1 in dependent-launch chains (the default), 2 for every launch
    static const int level = env_int("B2_GEMV_RING", 1);
    return level;
}
static bool ring_enabled() { return ring_level() != 0; }
static bool ring_fits(const WeightDev& w) {
    return (w.fmt == B2_FMT_MLX4 || w.fmt == B2_FMT_Q4_K) && xplanes_bytes(w.n_in) + RING_BYTES + 4096 <= 224 * 1024 && w.n_in <= 2048 * RING_X_STEPS;
}
bool gemv_takes_epilogue(const WeightDev& w) { return ring_enabled() && ring_fits(w) && w.n_out % 32 == 0; }

cudaError_t launch_gemv(const WeightDev& w, const WeightDev* up, const float* x, XPlanes xp, float* y, int mode, const float* gate,
                        int sm_count, cudaStream_t st, bool pdl, NormScale ns, EpiPlanes epi, bool plain_form) {
    if (epi.out.planes) {  // only the ring form carries the epilogue, chained or not
        if (!gemv_takes_epilogue(w)) return cudaErrorInvalidValue;
        if (w.fmt == B2_FMT_MLX4) return launch_ring<FmtMLX4_T>(w, up, xp, y, mode, gate, sm_count, st, pdl, ns, epi);
        return launch_ring<FmtQ4K_T>(w, up, xp, y, mode, gate, sm_count, st, pdl, ns, epi);
    }
    // In a chain of dependent launches (a decode step) the ring form wins: its copies start while the kernel ahead still
    // runs. Launched alone, the register-load form's shorter prologue makes it the faster one (measured at 14336 x 4096:
    // 11.2 us against 12.5), so plain launches keep it.
    if (!plain_form && ring_enabled() && (pdl || ring_level() >= 2) && ring_fits(w)) {
        if (w.fmt == B2_FMT_MLX4) return launch_ring<FmtMLX4_T>(w, up, xp, y, mode, gate, sm_count, st, pdl, ns, epi);
        return launch_ring<FmtQ4K_T>(w, up, xp, y, mode, gate, sm_count, st, pdl, ns, epi);
    }
    switch (w.fmt) {
        case B2_FMT_MLX4: return launch_fmt<FmtMLX4_T, false>(w, up, x, xp, y, mode, gate, sm_count, st, pdl, ns);
        case B2_FMT_Q4_K: return launch_fmt<FmtQ4K_T, false>(w, up, x, xp, y, mode, gate, sm_count, st, pdl, ns);
        case B2_FMT_Q6_K: return launch_fmt<FmtQ6K_T, false>(w, up, x, xp, y, mode, gate, sm_count, st, pdl, ns);
        case B2_FMT_Q8_0: return launch_fmt<FmtQ8_0_T, false>(w, up, x, xp, y, mode, gate, sm_count, st, pdl, ns);
        case B2_FMT_F8E4M3: {
            static const bool mma = [] {
                const char* e = getenv("B2_GEMV_F8_MMA");
                return !e || atoi(e) != 0;
            }();
            if (mma && !ns.partial && f8_mma_ok(w, mode)) return launch_f8_mma(w, x, y, mode, gate, sm_count, st, pdl);
            return launch_fmt<FmtF8_T, true>(w, up, x, xp, y, mode, gate, sm_count, st, pdl, ns);
        }
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
    e = launch_xplanes(x_dev, n_in, xp, st);
    if (e != cudaSuccess) return noalloc_fail(err, err_len, B2_ERR_CUDA, "activation planes kernel", e);
    e = launch_gemv(w, nullptr, x_dev, xp, y_dev, B2_MODE_STORE, nullptr, g_noalloc_sms[dev], st);
    if (e != cudaSuccess) return noalloc_fail(err, err_len, B2_ERR_CUDA, "gemv kernel", e);
    return B2_OK;
}
