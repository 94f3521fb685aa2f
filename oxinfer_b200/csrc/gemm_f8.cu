// FP8 block-scaled GEMM on the 5th-generation tensor cores with FP8 operands on BOTH sides (tcgen05.mma kind::f8f6f4):
//
//   y[m][n] = sum over 128-k blocks b of  sx[m][b] * sw[n / 128][b] * ( sum_{k in b} qx[m][k] * qw[n][k] )
//
// qw: e4m3 weights with one f32 scale per 128 x 128 block (GgufMatrix F8E4M3 + BlockScales, src/ggml.rs:240-293); qx, sx:
// the activations quantized per token and per 128 k to e4m3 with an f32 scale (quantize_act_e4m3_kernel below: scale =
// amax / 448, q = RNE(x / scale) saturating at +-448). The reference itself multiplies FP8 weights by unquantized
// activations (src/ggml.rs:433-443; gemm_tc.cu keeps that definition); this kernel is the large-projection form in which
// both operands stay in FP8 and nothing is expanded on the way to the tensor cores.
//
// One CTA computes 128 tokens x 256 weight rows over the whole K:
//   warp 0      : TMA producer: per 128-k block one box of activations (128 rows x 128 bytes) and one of weights
//                 (256 rows x 128 bytes), both 128-byte swizzled, straight into the MMA's operand layout (4-stage ring).
//   warp 1      : allocates TMEM; one lane issues four tcgen05.mma (M 128, N 256, K 32) per block into one of two
//                 256-column partial accumulators in TMEM (the first of a block overwrites), then commits: the ring slot is
//                 free, the partial is complete.
//   warps 4..11 : promotion. Warps 4..7 own columns 0..127 of the tile, warps 8..11 columns 128..255; a thread owns one token
//                 row (TMEM lane) and keeps its 128 results in registers. Per block it reads the partial sums with
//                 tcgen05.ld, multiplies by sx[token][b] * sw[column half][b] and adds. With 256-row tiles on a 128-row
//                 scale grid the weight scale is one scalar per warp and block. The promotion of block b runs under the
//                 MMAs of block b + 1.
// Every wait is bounded (cycle counter); a wait that gives up records where in the status word, raises the CTA's abort
// flag, in-flight copies are awaited, TMEM is freed and the kernel returns.
#include <cuda.h>
#include <cuda_fp8.h>

#include <algorithm>
#include <cstdio>
#include <cstdlib>

#include "kernels.h"

namespace b2 {

namespace {

constexpr int F8_STAGES = 4;
// The CTA-pair form (cta_group::2): two CTAs of a cluster compute 256 tokens x 256 weight rows. Each keeps 128 tokens (its
// own partial accumulators, promotion and epilogue) and copies HALF of the weight tile; one thread of the even CTA issues
// M = 256 instructions that read A from both CTAs and half of B from each. Per 128-k block a CTA then moves 32 KB through
// shared memory instead of 48 KB, and six stages fit.
constexpr int F8_PAIR_STAGES = 6;
constexpr int F8_MAX_STAGES = 6;
constexpr int F8_TM = 128;    // tokens per CTA
constexpr int F8_TN = 256;    // weight rows per CTA
constexpr int F8_BK = 128;    // k per stage = one scale block = one 128-byte swizzle row
constexpr int F8_A_BYTES = F8_TM * F8_BK;
constexpr int F8_B_BYTES = F8_TN * F8_BK;
constexpr int F8_THREADS = 384;  // warps 0..3: copies, MMAs (two idle); warps 4..11: promotion
constexpr long long F8_WAIT_LIMIT = 4000000000ll;

struct __align__(8) F8Shared {
    uint64_t full[F8_MAX_STAGES];
    uint64_t empty[F8_MAX_STAGES];
    uint64_t pfull[2];
    uint64_t pfree[2];
    uint32_t tmem_base;
    volatile uint32_t abort_flag;
};
constexpr size_t F8_SMEM = 1024 + (size_t)F8_STAGES * (F8_A_BYTES + F8_B_BYTES) + sizeof(F8Shared);
static_assert(F8_SMEM <= 227 * 1024, "shared memory budget");
constexpr size_t F8_PAIR_SMEM = 1024 + (size_t)F8_PAIR_STAGES * (F8_A_BYTES + F8_B_BYTES / 2) + sizeof(F8Shared);
static_assert(F8_PAIR_SMEM <= 227 * 1024, "shared memory budget (pair form)");

__device__ __forceinline__ uint32_t s32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void bar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(s32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void bar_arrive(uint64_t* bar) {
    asm volatile("{\n\t.reg .b64 st;\n\tmbarrier.arrive.shared::cta.b64 st, [%0];\n\t}" ::"r"(s32(bar)) : "memory");
}
__device__ __forceinline__ void bar_expect(uint64_t* bar, uint32_t bytes) {
    asm volatile("{\n\t.reg .b64 st;\n\tmbarrier.arrive.expect_tx.shared::cta.b64 st, [%0], %1;\n\t}" ::"r"(s32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool bar_try(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.b32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok)
                 : "r"(s32(bar)), "r"(parity)
                 : "memory");
    return ok != 0;
}
// The same test with acquire semantics at cluster scope: for barriers that the peer CTA's threads, copies or instructions complete.
__device__ __forceinline__ bool bar_try_cluster(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\tselp.b32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok)
                 : "r"(s32(bar)), "r"(parity)
                 : "memory");
    return ok != 0;
}
// The address, in the cluster's shared window, of CTA `cta`'s copy of a shared-memory object of this CTA.
__device__ __forceinline__ uint32_t cluster_addr(const void* p, uint32_t cta) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(s32(p)), "r"(cta));
    return r;
}
__device__ __forceinline__ void bar_arrive_cluster(uint32_t cluster_bar) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar) : "memory");
}
__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {  // every thread of both CTAs
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
template <bool CLUSTER = false>
__device__ __forceinline__ bool bar_wait(uint64_t* bar, uint32_t parity, F8Shared* sh, GemmStatus* status, uint32_t where, uint32_t iter,
                                         bool heed_abort = true) {
    auto test = [&] { return CLUSTER ? bar_try_cluster(bar, parity) : bar_try(bar, parity); };
    if (test()) return true;
    const long long t0 = clock64();
    for (uint32_t spin = 1;; spin++) {
        if (test()) return true;
        if ((spin & 255) == 0) {
            if (heed_abort && sh->abort_flag) return false;
            if (clock64() - t0 > F8_WAIT_LIMIT) {
                if (atomicCAS(&status->code, 0u, 1u) == 0u) {
                    status->where = 100 + where;
                    status->cta = blockIdx.x;
                    status->iter = iter;
                }
                sh->abort_flag = 1;
                return false;
            }
        }
    }
}
__device__ __forceinline__ void tma_2d(void* dst, const CUtensorMap* map, uint64_t* bar, int x, int y) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(s32(dst)), "l"(map),
                 "r"(s32(bar)), "r"(x), "r"(y)
                 : "memory");
}
// The copy of a CTA pair: the data lands in this CTA's shared memory, the bytes are counted on the barrier at the cluster
// address `cluster_bar` (the even CTA's: its MMA thread waits for both CTAs' tiles on one barrier). No multicast.
__device__ __forceinline__ void tma_2d_pair(void* dst, const CUtensorMap* map, uint32_t cluster_bar, int x, int y) {
    asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(s32(dst)),
                 "l"(map), "r"(cluster_bar), "r"(x), "r"(y)
                 : "memory");
}
// K-major operand tile, 128-byte swizzle: rows 128 bytes apart, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t desc_sw128(uint32_t addr) {
    uint64_t d = 0;
    d |= (uint64_t)((addr >> 4) & 0x3FFF);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}
__device__ __forceinline__ void mma_f8(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// M = 256 over a CTA pair: A rows 0..127 and B rows 0..N/2-1 from the even CTA's shared memory, the others from the odd
// CTA's (same offsets), accumulator rows 0..127 in the even CTA's tensor memory, 128..255 in the odd CTA's.
__device__ __forceinline__ void mma_f8_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// Arrives on the barrier at cluster address `cluster_bar` when the pair's instructions issued so far have completed.
__device__ __forceinline__ void commit_pair(uint32_t cluster_bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(cluster_bar) : "memory");
}
__device__ __forceinline__ void commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(s32(bar)) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, "
        "%22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]),
          "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]),
          "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]),
          "=r"(v[31])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_ld32_nowait(uint32_t taddr, uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, "
        "%22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]),
          "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]),
          "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]),
          "=r"(v[31])
        : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Tile (m, n) of CTA `id`: panels of 16 token tiles, all weight tiles of a panel before the next panel, the panel's token
// tiles fastest. The CTAs that run together then share 16 activation tiles and about nine weight tiles in L2.
__device__ __forceinline__ void tile_of(int id, int m_tiles, int n_tiles, int& m, int& n) {
    constexpr int PM = 16;
    const int per_panel = PM * n_tiles;
    const int panel = id / per_panel, r = id - panel * per_panel;
    const int pm = min(PM, m_tiles - panel * PM);
    n = r / pm;
    m = panel * PM + r - n * pm;
}

// PAIR: launched as clusters of two CTAs (neighbours in x); m_tiles then counts 256-token tiles of the pair.
template <bool PAIR>
__global__ void __launch_bounds__(F8_THREADS, 1)
gemm_f8_tc_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_w, int K, int n_out, int t, int m_tiles,
                  int n_tiles, const float* __restrict__ sx, const float* __restrict__ sw, int sw_ncb, int sw_row0, void* __restrict__ y, int y_dtype,
                  GemmStatus* __restrict__ status) {
    constexpr int F8_STAGES = PAIR ? F8_PAIR_STAGES : b2::F8_STAGES;
    constexpr int F8_B_BYTES = PAIR ? b2::F8_B_BYTES / 2 : b2::F8_B_BYTES;  // bytes of B this CTA holds per stage
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* a_tiles = smem;
    uint8_t* b_tiles = smem + (size_t)F8_STAGES * F8_A_BYTES;
    F8Shared* sh = (F8Shared*)(b_tiles + (size_t)F8_STAGES * F8_B_BYTES);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nb = K / F8_BK;
    // Programmatic dependent launch: the quantized activations and their scales come from the kernel ahead in the stream; the
    // producer and the promotion warps wait for it before they read them, everything else (barriers, tensor memory) does not.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    // pair form: this CTA's rank in its pair; the pair takes the tiles (of 256 tokens) first_tile, first_tile + tile_step, ...
    const uint32_t rank = PAIR ? cluster_rank() : 0u;
    const int first_tile = PAIR ? (int)(blockIdx.x >> 1) : (int)blockIdx.x, tile_step = PAIR ? (int)(gridDim.x >> 1) : (int)gridDim.x;
    // Persistent: CTA c takes tiles c, c + gridDim.x, ... ; the k-block counter `it` runs on across a CTA's tiles, so the ring
    // and the two partial accumulators keep alternating and the next tile's copies and MMAs start under this tile's epilogue.
    const int total_tiles = m_tiles * n_tiles;

    if (threadIdx.x == 0) {
        for (int s = 0; s < F8_STAGES; s++) {
            bar_init(&sh->full[s], 1);
            bar_init(&sh->empty[s], 1);
        }
        for (int i = 0; i < 2; i++) {
            bar_init(&sh->pfull[i], 1);
            bar_init(&sh->pfree[i], PAIR ? 16 : 8);  // the eight promotion warps (pair form: of both CTAs, on the even CTA's barrier)
        }
        sh->abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        if constexpr (PAIR) {  // the same warp of both CTAs
            asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(s32(&sh->tmem_base)), "r"(512u) : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
        } else {
            asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(s32(&sh->tmem_base)), "r"(512u) : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    if constexpr (PAIR)
        cluster_sync_all();  // both CTAs' barriers exist before either signals the other's
    else
        __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = sh->tmem_base;

    // The register file is divided by need: the copy / MMA warpgroup gives registers back, the two promotion warpgroups (128
    // accumulators and 64 staging registers per thread) take them.
    if (warp < 4) {
      asm volatile("setmaxnreg.dec.sync.aligned.u32 40;" ::: "memory");
      if (warp == 0) {
        if (lane == 0) {
            asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_x) : "memory");
            asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_w) : "memory");
            asm volatile("griddepcontrol.wait;" ::: "memory");
            int it = 0;
            bool ok = true;
            for (int tile = first_tile; tile < total_tiles && ok; tile += tile_step) {
                int mt, nt;
                tile_of(tile, m_tiles, n_tiles, mt, nt);
                for (int b = 0; b < nb; b++, it++) {
                    const int s = it % F8_STAGES;
                    const uint32_t ph = (uint32_t)((it / F8_STAGES) & 1);
                    if (!bar_wait<PAIR>(&sh->empty[s], ph ^ 1u, sh, status, 1, (uint32_t)it)) { ok = false; break; }
                    if constexpr (PAIR) {
                        // both CTAs' tiles are counted on the even CTA's barrier, which expects the bytes of both
                        const uint32_t bar0 = cluster_addr(&sh->full[s], 0);
                        if (rank == 0) bar_expect(&sh->full[s], (uint32_t)(2 * (F8_A_BYTES + F8_B_BYTES)));
                        tma_2d_pair(a_tiles + (size_t)s * F8_A_BYTES, &tmap_x, bar0, b * F8_BK, mt * 2 * F8_TM + (int)rank * F8_TM);
                        tma_2d_pair(b_tiles + (size_t)s * F8_B_BYTES, &tmap_w, bar0, b * F8_BK, nt * F8_TN + (int)rank * (F8_TN / 2));
                    } else {
                        bar_expect(&sh->full[s], (uint32_t)(F8_A_BYTES + F8_B_BYTES));
                        tma_2d(a_tiles + (size_t)s * F8_A_BYTES, &tmap_x, &sh->full[s], b * F8_BK, mt * F8_TM);
                        tma_2d(b_tiles + (size_t)s * F8_B_BYTES, &tmap_w, &sh->full[s], b * F8_BK, nt * F8_TN);
                    }
                }
            }
            // let the copies still in flight land before the shared memory is released (pair form: the odd CTA's copies are
            // counted on the even CTA's barriers, and both CTAs meet at the cluster barrier of the teardown after these waits)
            if (sh->abort_flag && rank == 0)
                for (int j = max(0, it - F8_STAGES); j < it; j++)
                    bar_wait<PAIR>(&sh->full[j % F8_STAGES], (uint32_t)((j / F8_STAGES) & 1), sh, status, 2, (uint32_t)j, false);
        }
    } else if (warp == 1) {
        if (lane == 0 && rank == 0) {
            // D f32 (bit 4), A and B e4m3 (format code 0), both K-major, N >> 3 at bit 17, M >> 4 at bit 24
            const uint32_t idesc = (1u << 4) | ((uint32_t)(F8_TN >> 3) << 17) | ((uint32_t)((PAIR ? 2 * F8_TM : F8_TM) >> 4) << 24);
            const uint64_t a_base = desc_sw128(s32(a_tiles)), b_base = desc_sw128(s32(b_tiles));
            bool ok = true;
            int n_mine = 0;
            for (int tile = first_tile; tile < total_tiles; tile += tile_step) n_mine++;
            const int n_it = n_mine * nb;
            for (int it = 0; it < n_it && ok; it++) {
                const int s = it % F8_STAGES, buf = it & 1;
                if (!bar_wait<PAIR>(&sh->full[s], (uint32_t)((it / F8_STAGES) & 1), sh, status, 3, (uint32_t)it)) { ok = false; break; }
                // the partial accumulator `buf` was last used by block it - 2: wait until its promotion has read it
                if (it >= 2 && !bar_wait<PAIR>(&sh->pfree[buf], (uint32_t)(((it >> 1) - 1) & 1), sh, status, 4, (uint32_t)it)) { ok = false; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint64_t ad = a_base + (uint64_t)((uint32_t)s * (F8_A_BYTES >> 4));
                const uint64_t bd = b_base + (uint64_t)((uint32_t)s * (F8_B_BYTES >> 4));
#pragma unroll
                for (int kk = 0; kk < F8_BK / 32; kk++) {  // 32 bytes of k per instruction: the descriptors advance by 2 x 16 bytes
                    if constexpr (PAIR)
                        mma_f8_pair(tmem_base + (uint32_t)(buf * F8_TN), ad + 2 * kk, bd + 2 * kk, idesc, kk > 0 ? 1u : 0u);
                    else
                        mma_f8(tmem_base + (uint32_t)(buf * F8_TN), ad + 2 * kk, bd + 2 * kk, idesc, kk > 0 ? 1u : 0u);
                }
                if constexpr (PAIR) {  // each CTA's producer and promotion warps wait on their own copies of the barriers
                    commit_pair(cluster_addr(&sh->empty[s], 0));
                    commit_pair(cluster_addr(&sh->empty[s], 1));
                    commit_pair(cluster_addr(&sh->pfull[buf], 0));
                    commit_pair(cluster_addr(&sh->pfull[buf], 1));
                } else {
                    commit(&sh->empty[s]);
                    commit(&sh->pfull[buf]);
                }
            }
        }
      }
    } else {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 232;" ::: "memory");
        // ---- promotion and epilogue ----
        const int pw = warp - 4;             // 0..7
        const int quarter = warp & 3;        // the TMEM lanes this warp may touch: 32 * (warp % 4)
        const int chalf = pw >> 2;           // column half of the tile
        float acc[128];
        bool ok = true;
        int it = 0;
        asm volatile("griddepcontrol.wait;" ::: "memory");  // the activations' scales (sx) come from the kernel ahead
        const uint32_t pfree_even = PAIR ? cluster_addr(&sh->pfree[0], 0) : 0u;  // the even CTA's pfree[0]
        for (int tile = first_tile; tile < total_tiles && ok; tile += tile_step) {
            int mt, nt;
            tile_of(tile, m_tiles, n_tiles, mt, nt);
            const int m0 = PAIR ? mt * 2 * F8_TM + (int)rank * F8_TM : mt * F8_TM, n0 = nt * F8_TN;
            const int token = m0 + quarter * 32 + lane;
            const int tok_c = min(token, t - 1);
            const float* sx_row = sx + (size_t)tok_c * nb;
            // (a column half wholly past n_out, in the last tile of a ragged matrix, reads the last valid scale row: its sums are zero)
            const float* sw_row = sw ? sw + (size_t)min((sw_row0 + n0 + chalf * 128) / 128, (sw_row0 + n_out - 1) / 128) * sw_ncb : nullptr;
#pragma unroll
            for (int i = 0; i < 128; i++) acc[i] = 0.0f;
            float c_next = __ldg(sx_row) * (sw_row ? __ldg(sw_row) : 1.0f);
            for (int b = 0; b < nb; b++, it++) {
                const int buf = it & 1;
                const float c = c_next;
                if (b + 1 < nb) c_next = __ldg(sx_row + b + 1) * (sw_row ? __ldg(sw_row + b + 1) : 1.0f);
                if (!bar_wait<PAIR>(&sh->pfull[buf], (uint32_t)((it >> 1) & 1), sh, status, 5, (uint32_t)it)) { ok = false; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(buf * F8_TN + chalf * 128);
                // two loads in flight: the next 32 columns travel while this chunk's multiply-adds issue
                uint32_t va[32], vb[32];
                tmem_ld32_nowait(taddr, va);
                tmem_ld32_nowait(taddr + 32u, vb);
                tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 32; i++) acc[i] = fmaf(__uint_as_float(va[i]), c, acc[i]);
                tmem_ld32_nowait(taddr + 64u, va);
#pragma unroll
                for (int i = 0; i < 32; i++) acc[32 + i] = fmaf(__uint_as_float(vb[i]), c, acc[32 + i]);
                tmem_ld32_nowait(taddr + 96u, vb);
                tmem_ld_wait();
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                __syncwarp();
                if (lane == 0) {  // the partial is in registers: the MMAs of block it + 2 may overwrite it
                    if constexpr (PAIR)
                        bar_arrive_cluster(pfree_even + (uint32_t)buf * 8u);
                    else
                        bar_arrive(&sh->pfree[buf]);
                }
#pragma unroll
                for (int i = 0; i < 32; i++) acc[64 + i] = fmaf(__uint_as_float(va[i]), c, acc[64 + i]);
#pragma unroll
                for (int i = 0; i < 32; i++) acc[96 + i] = fmaf(__uint_as_float(vb[i]), c, acc[96 + i]);
            }
            ok = __all_sync(0xffffffffu, ok) && !sh->abort_flag;
            if (ok && token < t) {
                const int nbase = n0 + chalf * 128;
                if (y_dtype == B2_BF16) {
                    __nv_bfloat16* o = (__nv_bfloat16*)y + (size_t)token * n_out + nbase;
                    if (nbase + 128 <= n_out && (n_out & 7) == 0) {
#pragma unroll
                        for (int i = 0; i < 16; i++) {
                            uint32_t pk[4];
#pragma unroll
                            for (int j = 0; j < 4; j++) {
                                __nv_bfloat162 h = __floats2bfloat162_rn(acc[8 * i + 2 * j], acc[8 * i + 2 * j + 1]);
                                pk[j] = *reinterpret_cast<uint32_t*>(&h);
                            }
                            ((uint4*)o)[i] = make_uint4(pk[0], pk[1], pk[2], pk[3]);
                        }
                    } else {
#pragma unroll
                        for (int i = 0; i < 128; i++)
                            if (nbase + i < n_out) o[i] = __float2bfloat16_rn(acc[i]);
                    }
                } else {
                    float* o = (float*)y + (size_t)token * n_out + nbase;
                    if (nbase + 128 <= n_out && (n_out & 3) == 0) {
#pragma unroll
                        for (int i = 0; i < 32; i++) ((float4*)o)[i] = make_float4(acc[4 * i], acc[4 * i + 1], acc[4 * i + 2], acc[4 * i + 3]);
                    } else {
#pragma unroll
                        for (int i = 0; i < 128; i++)
                            if (nbase + i < n_out) o[i] = acc[i];
                    }
                }
            }
        }
    }

    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    if constexpr (PAIR)
        cluster_sync_all();  // neither CTA's shared or tensor memory goes away while the other may still signal or read it
    else
        __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if constexpr (PAIR)
            asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
        else
            asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
    }
}

// Per token and per block of 128 k: scale = amax / 448 (1 for an all-zero block), q = e4m3(x / scale), round to nearest
// even, saturating at +-448; NaN stays NaN (0x7f). A warp per block: four values per lane.
__device__ __forceinline__ float as_float(float v) { return v; }
__device__ __forceinline__ float as_float(__nv_bfloat16 v) { return __bfloat162float(v); }
__device__ __forceinline__ float as_float(__half v) { return __half2float(v); }

template <typename T>
__global__ void __launch_bounds__(256) quantize_act_e4m3_kernel(const T* __restrict__ x, size_t t, int K, uint8_t* __restrict__ q, float* __restrict__ sx) {
    // (a dependent launch: the GEMM behind it may set itself up; the GEMM ahead of it may still be reading q and sx)
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const size_t blk = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    const int nb = K / 128;
    if (blk >= t * (size_t)nb) return;
    const size_t row = blk / nb;
    const int b = (int)(blk - row * nb);
    const T* p = x + row * (size_t)K + (size_t)b * 128 + lane * 4;
    float v[4];
#pragma unroll
    for (int i = 0; i < 4; i++) v[i] = as_float(p[i]);
    float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    const float s = amax > 0.0f ? __fdiv_rn(amax, 448.0f) : 1.0f;
    uint32_t pk = 0;
#pragma unroll
    for (int i = 0; i < 4; i++)
        pk |= (uint32_t)__nv_cvt_float_to_fp8(__fdiv_rn(v[i], s), __NV_SATFINITE, __NV_E4M3) << (8 * i);
    *(uint32_t*)(q + row * (size_t)K + (size_t)b * 128 + lane * 4) = pk;
    if (lane == 0) sx[row * nb + b] = s;
}

typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                             const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeFn encode_fn() {
    static EncodeFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess) fn = (EncodeFn)p;
    }
    return fn;
}

}  // namespace

bool gemm_f8_supports(const WeightDev& w, size_t t) {
    return w.fmt == B2_FMT_F8E4M3 && t >= 1 && w.n_in % 128 == 0 && w.n_in >= 128 && ((uintptr_t)w.p0 & 15) == 0 &&
           (w.p1 == nullptr || (w.bs_rows == 128 && w.bs_cols == 128 && w.bs_row0 % 128 == 0));
}

size_t gemm_f8_scratch_bytes(size_t t, size_t K) { return (t * K + 255) / 256 * 256 + t * (K / 128) * 4; }

cudaError_t launch_quantize_act_e4m3(const void* x, int x_dtype, size_t t, size_t K, uint8_t* q, float* sx, cudaStream_t st) {
    if (t == 0 || K % 128) return cudaErrorInvalidValue;
    const size_t warps = t * (K / 128);
    const unsigned grid = (unsigned)((warps + 7) / 8);
    if (x_dtype == B2_F32)
        return launch_k(quantize_act_e4m3_kernel<float>, dim3(grid), dim3(256), 0, st, true, (const float*)x, t, (int)K, q, sx);
    else if (x_dtype == B2_BF16)
        return launch_k(quantize_act_e4m3_kernel<__nv_bfloat16>, dim3(grid), dim3(256), 0, st, true, (const __nv_bfloat16*)x, t, (int)K, q, sx);
    else if (x_dtype == B2_F16)
        return launch_k(quantize_act_e4m3_kernel<__half>, dim3(grid), dim3(256), 0, st, true, (const __half*)x, t, (int)K, q, sx);
    else
        return cudaErrorInvalidValue;
    return cudaGetLastError();
}

cudaError_t launch_gemm_f8(const WeightDev& w, const uint8_t* qx, const float* sx, size_t t, void* y, int y_dtype, GemmStatus* status_dev,
                           cudaStream_t st, char* err, size_t errlen) {
    EncodeFn enc = encode_fn();
    if (!enc) {
        snprintf(err, errlen, "cuTensorMapEncodeTiled is not available from the driver");
        return cudaErrorNotSupported;
    }
    // B2_F8_PAIR=1 selects the CTA-pair form for more than one 128-token tile. Off by default: with two partial accumulators
    // the MMA -> promotion -> MMA chain of a block crosses SMs twice in that form, and it measures 6.8 ms against 3.2 ms at
    // 8192 x 12288 x 28672 (bit-identical results).
    const char* pe = getenv("B2_F8_PAIR");
    const bool pair = t > (size_t)F8_TM && pe && atoi(pe) != 0;
    CUtensorMap tx, tw;
    cuuint32_t estr[2] = {1, 1};
    {
        cuuint64_t dims[2] = {(cuuint64_t)w.n_in, (cuuint64_t)t};
        cuuint64_t strides[1] = {(cuuint64_t)w.n_in};
        cuuint32_t box[2] = {(cuuint32_t)F8_BK, (cuuint32_t)F8_TM};
        CUresult r = enc(&tx, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, (void*)qx, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                         CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) {
            snprintf(err, errlen, "cuTensorMapEncodeTiled(qx) failed with CUresult %d", (int)r);
            return cudaErrorInvalidValue;
        }
    }
    {
        cuuint64_t dims[2] = {(cuuint64_t)w.n_in, (cuuint64_t)w.n_out};
        cuuint64_t strides[1] = {(cuuint64_t)w.n_in};
        cuuint32_t box[2] = {(cuuint32_t)F8_BK, (cuuint32_t)(pair ? F8_TN / 2 : F8_TN)};
        CUresult r = enc(&tw, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, (void*)w.p0, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                         CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) {
            snprintf(err, errlen, "cuTensorMapEncodeTiled(w) failed with CUresult %d", (int)r);
            return cudaErrorInvalidValue;
        }
    }
    const int n_tiles = (int)((w.n_out + F8_TN - 1) / F8_TN);
    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (pair) {
        auto kern = gemm_f8_tc_kernel<true>;
        if (cudaError_t e = ensure_dynamic_smem((const void*)kern, F8_PAIR_SMEM, 0); e != cudaSuccess) return e;
        const int pm_tiles = (int)((t + 2 * F8_TM - 1) / (2 * F8_TM));
        const int pairs = std::min(pm_tiles * n_tiles, sms / 2);  // persistent: one CTA per SM, two SMs per pair
        cudaLaunchConfig_t cfg{};
        cfg.gridDim = dim3((unsigned)(2 * pairs));
        cfg.blockDim = dim3(F8_THREADS);
        cfg.dynamicSmemBytes = F8_PAIR_SMEM;
        cfg.stream = st;
        cudaLaunchAttribute attr{};
        attr.id = cudaLaunchAttributeClusterDimension;
        attr.val.clusterDim.x = 2;  // a CTA pair is formed along x
        attr.val.clusterDim.y = 1;
        attr.val.clusterDim.z = 1;
        cfg.attrs = &attr;
        cfg.numAttrs = 1;
        return cudaLaunchKernelEx(&cfg, kern, tx, tw, (int)w.n_in, (int)w.n_out, (int)t, pm_tiles, n_tiles, sx, (const float*)w.p1, (int)w.bs_ncb,
                                  (int)w.bs_row0, y, y_dtype, status_dev);
    }
    if (cudaError_t e = ensure_dynamic_smem((const void*)gemm_f8_tc_kernel<false>, F8_SMEM, 0); e != cudaSuccess) return e;
    const int m_tiles = (int)((t + F8_TM - 1) / F8_TM);
    const int grid = m_tiles * n_tiles < sms ? m_tiles * n_tiles : sms;  // persistent: one CTA per SM
    return launch_k(gemm_f8_tc_kernel<false>, dim3((unsigned)grid), dim3(F8_THREADS), F8_SMEM, st, true, tx, tw, (int)w.n_in, (int)w.n_out, (int)t, m_tiles,
                    n_tiles, sx, (const float*)w.p1, (int)w.bs_ncb, (int)w.bs_row0, y, y_dtype, status_dev);
}

}  // namespace b2
