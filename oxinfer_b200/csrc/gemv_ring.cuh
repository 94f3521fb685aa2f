// The 4-bit matrix-vector product with the weights brought in by bulk copies: every warp owns a small ring of
// shared-memory slots, its first lane issues the copies of the next row-pair steps (two runs of up to 1152 bytes, the
// eight super-blocks of a step for each of the two rows) while the warp computes the current one, and an mbarrier word
// per slot counts the bytes as they land. Loads in flight no longer cost registers and do not stop while the warp
// does arithmetic, which the register-load form (gemv_core.cuh: load, then use) cannot avoid.
#pragma once
#include "async_copy.cuh"
#include "gemv_core.cuh"
#include "xplanes.cuh"

namespace b2 {
namespace gemv_core {

constexpr int RING_ROW_BYTES = 8 * 144;               // one row's super-blocks of a step (2048 weights)
constexpr int RING_SLOT_BYTES = 2 * RING_ROW_BYTES;   // a row pair
constexpr long long RING_WAIT_LIMIT = 600000000LL;    // cycles before a wait on a copy gives up

struct WarpRing {     // one warp's ring; the state lives in the warp's registers between products
    uint8_t* slots;   // S slots of RING_SLOT_BYTES, 128-byte aligned
    uint64_t* bars;   // S barrier words (initialized with count 1)
    uint32_t phases;  // bit s: the parity the next wait on slot s uses
    int S;
};

__device__ __forceinline__ void q4_load_smem(const uint8_t* row_chunk, int lane, Q4Regs& r) {
    const uint8_t* blk = row_chunk + (lane >> 2) * 144;
    r.hdr = *(const uint4*)blk;
    r.q0 = *(const uint4*)(blk + 16 + 32 * (lane & 3));
    r.q1 = *(const uint4*)(blk + 32 + 32 * (lane & 3));
}

// A warp's row sequence: pair-step p covers rows row(p), row(p) + 1 (PAIR: row(p) of both matrices), with
//   row(p) = r_first + (p / ni) * r_step + (p % ni) * (PAIR ? 1 : 2).
// ni == 1 is the plain arithmetic sequence (rows interleaved over the grid's warps); with ni = 2 (PAIR: 4), r_first =
// 32 * CTA + 4 * warp and r_step = 32 * grid, the eight warps of a CTA cover whole blocks of 32 consecutive rows.
template <bool PAIR>
__device__ __forceinline__ size_t ring_row(size_t r_first, size_t r_step, uint32_t ni, uint32_t p) {
    return ni == 1 ? r_first + (size_t)p * r_step : r_first + (size_t)(p / ni) * r_step + (size_t)(p % ni) * (PAIR ? 1 : 2);
}

// The copies of step s of a warp's row sequence (one lane calls it).
template <bool PAIR>
__device__ __forceinline__ void ring_issue(const WeightDev& w, const WeightDev& w2, const WarpRing& ring, size_t r_first, size_t r_step, uint32_t s,
                                           uint32_t ni = 1) {
    using namespace acopy;
    const int nblk = (int)w.n_in / 256, iters = (nblk + 7) / 8;
    const size_t row_bytes = (size_t)nblk * 144, n_out = w.n_out;
    const uint32_t pair = s / (uint32_t)iters, it = s - pair * (uint32_t)iters;
    const size_t r0 = ring_row<PAIR>(r_first, r_step, ni, pair);
    const size_t rowB = PAIR ? r0 : min(r0 + 1, n_out - 1);
    const uint32_t bytes = (uint32_t)min(8, nblk - (int)it * 8) * 144u;
    const int slot = (int)(s % (uint32_t)ring.S);
    uint8_t* dst = ring.slots + slot * RING_SLOT_BYTES;
    bar_expect_tx(&ring.bars[slot], 2 * bytes);
    bulk_load(dst, w.p0 + r0 * row_bytes + (size_t)it * RING_ROW_BYTES, bytes, &ring.bars[slot]);
    bulk_load(dst + RING_ROW_BYTES, (PAIR ? w2.p0 : w.p0) + rowB * row_bytes + (size_t)it * RING_ROW_BYTES, bytes, &ring.bars[slot]);
}

// How many steps a warp's sequence has.
__device__ __forceinline__ uint32_t ring_steps(const WeightDev& w, size_t r_first, size_t r_step, uint32_t ni = 1) {
    const int nblk = (int)w.n_in / 256, iters = (nblk + 7) / 8;
    const uint32_t npairs = r_first < w.n_out ? (uint32_t)((w.n_out - r_first + r_step - 1) / r_step) * ni : 0;
    return npairs * (uint32_t)iters;
}

// The first S - 1 steps' copies (one lane). A kernel may call this before it waits for the kernel ahead of it: the
// weights do not depend on that kernel. gemv4_ring is then told that the ring is primed.
template <bool PAIR>
__device__ __forceinline__ void ring_prime(const WeightDev& w, const WeightDev& w2, const WarpRing& ring, size_t r_first, size_t r_step,
                                           uint32_t ni = 1) {
    const uint32_t T = ring_steps(w, r_first, r_step, ni);
    for (uint32_t s = 0; s + 1 < (uint32_t)ring.S && s < T; s++) ring_issue<PAIR>(w, w2, ring, r_first, r_step, s, ni);
}

// The planes record of x -> shared memory by bulk copies, one set per step of 2048 k (what a warp consumes per ring step)
// with a barrier word each (count 1, initialized by the caller), so the rows start as soon as the first part has landed.
// One thread calls it; gemv4_ring waits on xbars[step].
constexpr int RING_X_STEPS = 32;  // barrier words: K <= 65536
__device__ __forceinline__ void ring_stage_planes(const XPlanes& xp, int K, uint8_t* sm, uint64_t* xbars) {
    using namespace acopy;
    const int iters = (K / 256 + 7) / 8;
    const uint8_t* g = (const uint8_t*)xp.planes;
    const size_t sx_at = 3 * (size_t)K, v16_at = sx_at + 8 * (size_t)(K / 32);
    for (int it = 0; it < iters; it++) {
        const uint32_t k0 = (uint32_t)it * 2048u, kn = min(2048u, (uint32_t)K - k0);
        bar_expect_tx(&xbars[it], 3 * kn + kn / 4 + kn / 4);
#pragma unroll
        for (int p = 0; p < 3; p++) bulk_load(sm + (size_t)p * K + k0, g + (size_t)p * K + k0, kn, &xbars[it]);
        bulk_load(sm + sx_at + k0 / 4, g + sx_at + k0 / 4, kn / 4, &xbars[it]);
        bulk_load(sm + v16_at + k0 / 4, g + v16_at + k0 / 4, kn / 4, &xbars[it]);
    }
}

constexpr int EPI_BARRIER = 7;  // the named barrier the eight warps of a CTA meet at once a block of 32 rows is done

// The split of a finished block of 32 outputs (EpiPlanes) by one warp: `vals` are the block's values in shared memory.
__device__ __forceinline__ void epi_block(const EpiPlanes& epi, const float* vals, int blk, int n_out, int lane) {
    const float v = vals[lane] * epi.pre;
    if (epi.partial) {
        float s = v * v;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
        if (lane == 0) epi.partial[blk] = s;
    }
    xplanes_block(epi.w ? v * epi.w[(size_t)blk * 32 + lane] : v, blk, lane, n_out, epi.out);
}

// Rows of a warp's sequence (ring_row) by one warp. False: a wait on a copy ran into its limit (the caller reports it
// and stops). With an EpiPlanes (`epi_vals`: 2 x 32 floats of CTA-shared memory; ni as described at ring_row, every warp
// of the CTA of `epi_threads` threads calling with the same step count) the warps meet after each block of 32 rows and one of them
// splits it; a warp whose copy wait failed keeps meeting the others without computing, so nobody waits for it in vain.
template <class F, bool PAIR>
__device__ __forceinline__ bool gemv4_ring(const WeightDev& w, const WeightDev& w2, const XS& xs, float* __restrict__ y, const int mode,
                                           const float* __restrict__ gate, WarpRing& ring, const size_t r_first, const size_t r_step,
                                           const int lane, const bool primed = false, const float kscale = 1.0f, const uint32_t ni = 1,
                                           const EpiPlanes epi = EpiPlanes{XPlanes{nullptr, nullptr, nullptr}, nullptr, nullptr, 1.0f},
                                           float* epi_vals = nullptr, const int epi_threads = 256, uint64_t* xbars = nullptr) {
    using namespace acopy;
    const int K = (int)w.n_in, nblk = K / 256, iters = (nblk + 7) / 8;
    const size_t n_out = w.n_out;
    const uint32_t T = ring_steps(w, r_first, r_step, ni);
    const int S = ring.S;
    const bool with_epi = epi.out.planes != nullptr;
    if (lane == 0 && !primed) ring_prime<PAIR>(w, w2, ring, r_first, r_step, ni);
    float accA = 0.0f, accB = 0.0f;
    uint32_t it = 0, pair = 0;
    bool ok = true;
    for (uint32_t s = 0; s < T; s++) {
        if (ok) {
            __syncwarp();  // every lane is done with the slot that is refilled now
            if (lane == 0 && s + (uint32_t)S - 1 < T) ring_issue<PAIR>(w, w2, ring, r_first, r_step, s + (uint32_t)S - 1, ni);
            const int slot = (int)(s % (uint32_t)S);
            if (!bar_wait(&ring.bars[slot], (ring.phases >> slot) & 1u, RING_WAIT_LIMIT)) {
                if (!with_epi) return false;
                ok = false;
            }
            ring.phases ^= 1u << slot;
            if (ok && xbars && !bar_wait(&xbars[it], 0u, RING_WAIT_LIMIT)) {  // this step's part of the planes (ring_stage_planes)
                if (!with_epi) return false;
                ok = false;
            }
            if (ok && F::active(K, (int)it, lane)) {
                const uint8_t* src = ring.slots + slot * RING_SLOT_BYTES;
                Q4Regs ra, rb;
                q4_load_smem(src, lane, ra);
                q4_load_smem(src + RING_ROW_BYTES, lane, rb);
                F::dot2(ra, rb, xs, (int)it, lane, accA, accB);
            }
        }
        if (++it == (uint32_t)iters) {
            const size_t r0 = ring_row<PAIR>(r_first, r_step, ni, pair);
            accA = warp_sum(accA) * kscale;
            accB = warp_sum(accB) * kscale;
            const uint32_t group = pair / ni;
            float* vals = with_epi ? epi_vals + (group & 1u) * 32 + (r0 & 31) : nullptr;
            if (lane == 0 && ok) {
                if (PAIR) {
                    const float a = (mode == B2_MODE_SILU_PAIR ? silu(accA) : gelu_tanh(accA)) * accB;
                    y[r0] = a;
                    if (with_epi) vals[0] = a;
                } else {
#pragma unroll
                    for (int r = 0; r < 2; r++) {
                        if (r0 + r >= n_out) break;
                        float a = r ? accB : accA;
                        float* o = y + r0 + r;
                        if (mode == B2_MODE_ADD)
                            a += *o;
                        else if (mode != B2_MODE_STORE)
                            a = *o + a * (1.0f / (1.0f + __expf(-gate[0])));
                        *o = a;
                        if (with_epi) vals[r] = a;
                    }
                }
            }
            if (with_epi && (pair + 1) % ni == 0) {  // the block of 32 rows is complete once all eight warps are here
                asm volatile("bar.sync %0, %1;" ::"r"(EPI_BARRIER), "r"(epi_threads) : "memory");
                if (group % (uint32_t)(epi_threads >> 5) == (threadIdx.x >> 5))
                    epi_block(epi, epi_vals + (group & 1u) * 32, (int)(r0 >> 5), (int)n_out, lane);
            }
            accA = accB = 0.0f;
            it = 0;
            pair++;
        }
    }
    return ok;
}

}  // namespace gemv_core
}  // namespace b2
