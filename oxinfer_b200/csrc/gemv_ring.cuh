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

// The copies of step s of a warp's row sequence (one lane calls it).
template <bool PAIR>
__device__ __forceinline__ void ring_issue(const WeightDev& w, const WeightDev& w2, const WarpRing& ring, size_t r_first, size_t r_step, uint32_t s) {
    using namespace acopy;
    const int nblk = (int)w.n_in / 256, iters = (nblk + 7) / 8;
    const size_t row_bytes = (size_t)nblk * 144, n_out = w.n_out;
    const uint32_t pair = s / (uint32_t)iters, it = s - pair * (uint32_t)iters;
    const size_t r0 = r_first + (size_t)pair * r_step;
    const size_t rowB = PAIR ? r0 : min(r0 + 1, n_out - 1);
    const uint32_t bytes = (uint32_t)min(8, nblk - (int)it * 8) * 144u;
    const int slot = (int)(s % (uint32_t)ring.S);
    uint8_t* dst = ring.slots + slot * RING_SLOT_BYTES;
    bar_expect_tx(&ring.bars[slot], 2 * bytes);
    bulk_load(dst, w.p0 + r0 * row_bytes + (size_t)it * RING_ROW_BYTES, bytes, &ring.bars[slot]);
    bulk_load(dst + RING_ROW_BYTES, (PAIR ? w2.p0 : w.p0) + rowB * row_bytes + (size_t)it * RING_ROW_BYTES, bytes, &ring.bars[slot]);
}

// How many steps a warp's sequence has.
__device__ __forceinline__ uint32_t ring_steps(const WeightDev& w, size_t r_first, size_t r_step) {
    const int nblk = (int)w.n_in / 256, iters = (nblk + 7) / 8;
    const uint32_t npairs = r_first < w.n_out ? (uint32_t)((w.n_out - r_first + r_step - 1) / r_step) : 0;
    return npairs * (uint32_t)iters;
}

// The first S - 1 steps' copies (one lane). A kernel may call this before it waits for the kernel ahead of it: the
// weights do not depend on that kernel. gemv4_ring is then told that the ring is primed.
template <bool PAIR>
__device__ __forceinline__ void ring_prime(const WeightDev& w, const WeightDev& w2, const WarpRing& ring, size_t r_first, size_t r_step) {
    const uint32_t T = ring_steps(w, r_first, r_step);
    for (uint32_t s = 0; s + 1 < (uint32_t)ring.S && s < T; s++) ring_issue<PAIR>(w, w2, ring, r_first, r_step, s);
}

// EpiPlanes: lane 0 of the calling warp has just written rows r0 .. r0 + n - 1 of y (all in one block of 32). The add
// releases those writes and acquires the other warps'; whoever brings the block's count to 32 splits the block.
__device__ __forceinline__ void epi_rows(const EpiPlanes& epi, const float* y, size_t r0, uint32_t n, int n_out, int lane) {
    const int blk = (int)(r0 >> 5);
    uint32_t done = 0;
    if (lane == 0) {
        asm volatile("atom.add.acq_rel.gpu.global.u32 %0, [%1], %2;" : "=r"(done) : "l"(epi.counters + blk), "r"(n) : "memory");
        done += n;
    }
    done = __shfl_sync(0xffffffffu, done, 0);
    if (done != 32u) return;
    __syncwarp();  // the other lanes' reads come after lane 0's acquire
    const float v = __ldcg(y + (size_t)blk * 32 + lane) * epi.pre;
    if (epi.partial) {
        float s = v * v;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
        if (lane == 0) epi.partial[blk] = s;
    }
    xplanes_block(epi.w ? v * epi.w[(size_t)blk * 32 + lane] : v, blk, lane, n_out, epi.out);
    if (lane == 0) epi.counters[blk] = 0;
}

// Rows r_first, r_first + r_step, ... (pairs of rows, or the same row of w and w2 with PAIR) by one warp.
// False: a wait on a copy ran into its limit (the caller reports it and stops).
template <class F, bool PAIR>
__device__ __forceinline__ bool gemv4_ring(const WeightDev& w, const WeightDev& w2, const XS& xs, float* __restrict__ y, const int mode,
                                           const float* __restrict__ gate, WarpRing& ring, const size_t r_first, const size_t r_step,
                                           const int lane, const bool primed = false, const float kscale = 1.0f,
                                           const EpiPlanes epi = EpiPlanes{nullptr, XPlanes{nullptr, nullptr, nullptr, nullptr}, nullptr, nullptr, 1.0f}) {
    using namespace acopy;
    const int K = (int)w.n_in, nblk = K / 256, iters = (nblk + 7) / 8;
    const size_t n_out = w.n_out;
    const uint32_t T = ring_steps(w, r_first, r_step);
    const int S = ring.S;
    if (lane == 0 && !primed) ring_prime<PAIR>(w, w2, ring, r_first, r_step);
    float accA = 0.0f, accB = 0.0f;
    uint32_t it = 0;
    size_t r0 = r_first;
    for (uint32_t s = 0; s < T; s++) {
        __syncwarp();  // every lane is done with the slot that is refilled now
        if (lane == 0 && s + (uint32_t)S - 1 < T) ring_issue<PAIR>(w, w2, ring, r_first, r_step, s + (uint32_t)S - 1);
        const int slot = (int)(s % (uint32_t)S);
        if (!bar_wait(&ring.bars[slot], (ring.phases >> slot) & 1u, RING_WAIT_LIMIT)) return false;
        ring.phases ^= 1u << slot;
        if (F::active(K, (int)it, lane)) {
            const uint8_t* src = ring.slots + slot * RING_SLOT_BYTES;
            Q4Regs ra, rb;
            q4_load_smem(src, lane, ra);
            q4_load_smem(src + RING_ROW_BYTES, lane, rb);
            F::dot2(ra, rb, xs, (int)it, lane, accA, accB);
        }
        if (++it == (uint32_t)iters) {
            accA = warp_sum(accA) * kscale;
            accB = warp_sum(accB) * kscale;
            if (lane == 0) {
                if (PAIR) {
                    y[r0] = (mode == B2_MODE_SILU_PAIR ? silu(accA) : gelu_tanh(accA)) * accB;
                } else {
#pragma unroll
                    for (int r = 0; r < 2; r++) {
                        if (r0 + r >= n_out) break;
                        const float a = r ? accB : accA;
                        float* o = y + r0 + r;
                        if (mode == B2_MODE_STORE)
                            *o = a;
                        else if (mode == B2_MODE_ADD)
                            *o += a;
                        else
                            *o += a * (1.0f / (1.0f + __expf(-gate[0])));
                    }
                }
            }
            if (epi.counters) epi_rows(epi, y, r0, PAIR ? 1u : (uint32_t)min((size_t)2, n_out - r0), (int)n_out, lane);
            accA = accB = 0.0f;
            it = 0;
            r0 += r_step;
        }
    }
    return true;
}

}  // namespace gemv_core
}  // namespace b2
