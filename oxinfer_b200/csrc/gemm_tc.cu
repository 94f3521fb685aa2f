// Prefill dequant-GEMM for Q4_K weights on the 5th-generation tensor cores (tcgen05 + TMEM).
//
//   y[t][n_out] = x[t][K] * W^T,  W in GGUF Q4_K super-blocks (src/ggml.rs:750-773).
//
// It replaces the reference's CPU prefill path for GGUF weights (dequantize 8 rows + f32 FMA tiles,
// src/kernels.rs:1998-2038) and plays the role of gemm_q4a / gemm_body (src/cuda.rs:185-232), which
// has no GGUF arm at all (src/cuda.rs:1011).
//
// One CTA computes a tile of TM = 128 * m_halves tokens x tile_n weight rows over the whole K:
//   warp 0       : TMA producer. Two streams of cp.async.bulk.tensor copies: the activation tiles
//                  (f16, 64 k x TM tokens, 128-byte swizzle) into a 3-stage ring, and the PACKED weight
//                  tile of one super-block column (144 bytes x tile_n rows, unswizzled) into a raw
//                  staging buffer, one super-block ahead of the dequantizers.
//   warp 1       : allocates TMEM; one lane issues tcgen05.mma.kind::f16 (M = 128 tokens per
//                  instruction, N = tile_n weight rows, K = 16), accumulating in TMEM, and frees each
//                  ring slot with tcgen05.commit.
//   warps 2..17  : dequantizers. Two threads own each weight row of the tile (low / high nibbles of a
//                  64-group): per super-block they copy the row's 144 packed bytes from the staging
//                  buffer to registers, release the buffer, and expand one 64-group per pipeline stage
//                  to f16 with packed half2 arithmetic (w = d*sc*q - dmin*m), writing the K-major,
//                  128-byte-swizzled B operand tile. After the main loop the same warps read the
//                  accumulators back with tcgen05.ld and store y.
// tile_n is chosen on the host (a multiple of 16, at most 240) so that the grid fills the SMs in one
// wave; the last tile may be ragged (TMA zero-fills rows past n_out, which dequantize to zeros).
// Operands are f16 rather than bf16: Q4_K values carry more than 8 significant bits, and bf16
// activations convert to f16 exactly in the range that matters.
// The same kernel is instantiated for the repacked MLX 4-bit blocks, FP8 e4m3 with block scales, Q8_0 (int8 rows + f16
// block scales) and Q6_K (rows of low nibbles and of high bit pairs + i8 scales + f16 d): only the weight copies and the
// dequantizers' expansion differ (the arms of `if constexpr (FMT == ...)`).
//
// Every wait is bounded: a wait that exceeds its cycle limit records where it gave up in a status
// word, raises a CTA-wide abort flag, and every role then falls through to the common teardown
// (in-flight copies are awaited, TMEM is freed) so that the kernel always returns.
#include <cuda.h>
#include <cuda_fp8.h>

#include <cstdio>
#include <cstdlib>
#include <cstring>

#include "kernels.h"

namespace b2 {

namespace {

constexpr int STAGES = 3;
constexpr int STAGE_K = 64;                // f16 elements per row per stage = one 128-byte swizzle row
constexpr int MAX_TILE_N = 240;
constexpr int A_STAGE_BYTES = 256 * 128;   // up to 256 tokens
constexpr int B_STAGE_BYTES = MAX_TILE_N * 128;
constexpr int RAW_BYTES = MAX_TILE_N * 144;  // one super-block column of the weight tile, packed
constexpr int GEMM_THREADS = 608;          // activation producer, MMA issuer, 16 dequant / epilogue warps, weight producer
constexpr long long WAIT_LIMIT_CYCLES = 4000000000ll;  // about two seconds of SM clock

struct F8Scales {  // block scales of an FP8 matrix (formats.cuh); s == nullptr for the 4-bit formats.
                   // Q8_0: s = the f16 block scales [n_out][ncb]. Q6_K: s = the i8 scales [n_out][K / 16], s2 = the f16 d [n_out][K / 256].
    const float* s;
    const void* s2;
    int rows, ncb, row0;
    float pre;  // power of two folded into the f16 weights (keeps small scales out of f16's subnormals); the
                // epilogue multiplies the outputs by 1 / pre
};

// The CTA-pair form (cta_group::2): two CTAs of a cluster share every weight tile. Each expands half of its rows (at most
// 128) and keeps 256 tokens of its own; one thread of the even CTA issues M = 256 instructions that read A from both CTAs
// and B half from each, so a CTA's shared memory is read for half a B tile per instruction instead of a whole one, and a
// weight is expanded once per 512 tokens instead of once per 256. Stages are 32 KB (A) + 16 KB (B): four of them fit.
constexpr int PAIR_STAGES = 4;
constexpr int PAIR_MAX_TILE_N = 240;                       // the pair's tile; a CTA expands half of it
constexpr int PAIR_B_STAGE_BYTES = PAIR_MAX_TILE_N / 2 * 128;
constexpr int PAIR_RAW_BYTES = PAIR_MAX_TILE_N / 2 * 144;  // one of two staging buffers (the copy of super-block sb + 2 flies while sb + 1 is expanded)
constexpr int MAX_STAGES = 4;
constexpr int Q6K_MAX_TILE_N = 208;

struct __align__(8) Shared {
    uint64_t a_full[MAX_STAGES];
    uint64_t b_full[MAX_STAGES];
    uint64_t empty[MAX_STAGES];
    uint64_t raw_full[2];
    uint64_t raw_empty[2];
    uint64_t acc_full;
    uint32_t tmem_base;
    volatile uint32_t abort_flag;
};

constexpr size_t GEMM_SMEM = 1024 /*alignment slack*/ + (size_t)STAGES * (A_STAGE_BYTES + B_STAGE_BYTES) + RAW_BYTES + sizeof(Shared);
static_assert(GEMM_SMEM <= 227 * 1024, "shared memory budget");
constexpr size_t PAIR_SMEM = 1024 + (size_t)PAIR_STAGES * (A_STAGE_BYTES + PAIR_B_STAGE_BYTES) + 2 * PAIR_RAW_BYTES + sizeof(Shared);
static_assert(PAIR_SMEM <= 227 * 1024, "shared memory budget (pair form)");

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("{\n\t.reg .b64 st;\n\tmbarrier.arrive.shared::cta.b64 st, [%0];\n\t}" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("{\n\t.reg .b64 st;\n\tmbarrier.arrive.expect_tx.shared::cta.b64 st, [%0], %1;\n\t}" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.b32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}

// The same test with acquire semantics at cluster scope: for barriers that a peer CTA's threads or copies complete.
__device__ __forceinline__ bool mbar_try_wait_cluster(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\tselp.b32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// The address, in the cluster's shared window, of the CTA of rank `cta`'s copy of a shared-memory object of this CTA.
__device__ __forceinline__ uint32_t cluster_addr(const void* p, uint32_t cta) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_u32(p)), "r"(cta));
    return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_bar) {
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

// Bounded wait. Returns false when the CTA is aborting or the limit passed (in which case it records
// `where` and raises the abort flag). `heed_abort` = false is for the teardown waits. The limit is
// counted on the SM's own cycle counter (a cheap register read; the global nanosecond timer costs
// about a microsecond per read, as long as a whole pipeline stage).
template <bool CLUSTER = false>
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, Shared* sh, GemmStatus* status, uint32_t where, uint32_t iter,
                                          bool heed_abort = true) {
    auto test = [&] { return CLUSTER ? mbar_try_wait_cluster(bar, parity) : mbar_try_wait(bar, parity); };
    if (test()) return true;
    const long long t0 = clock64();
    for (uint32_t spin = 1;; spin++) {
        if (test()) return true;
        if ((spin & 255) == 0) {
            if (heed_abort && sh->abort_flag) return false;
            if (clock64() - t0 > WAIT_LIMIT_CYCLES) {
                if (atomicCAS(&status->code, 0u, 1u) == 0u) {
                    status->where = where;
                    status->cta = blockIdx.x + gridDim.x * blockIdx.y;
                    status->iter = iter;
                }
                sh->abort_flag = 1;
                return false;
            }
        }
    }
}

__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, uint64_t* bar, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(smem_u32(dst)),
        "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y)
        : "memory");
}

// The copy of a CTA pair: the data lands in this CTA's shared memory, the bytes are counted on the barrier at the cluster
// address `cluster_bar` (the even CTA's: its MMA thread waits for both CTAs' tiles on one barrier).
__device__ __forceinline__ void tma_load_2d_pair(void* dst, const CUtensorMap* map, uint32_t cluster_bar, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(smem_u32(dst)),
        "l"(map), "r"(cluster_bar), "r"(x), "r"(y)
        : "memory");
}

// K-major operand tile, 128-byte swizzle, rows 128 bytes apart, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t addr) {
    uint64_t d = 0;
    d |= (uint64_t)((addr >> 4) & 0x3FFF);         // start address
    d |= (uint64_t)1 << 16;                        // leading byte offset (unused for swizzled K-major)
    d |= (uint64_t)(1024 >> 4) << 32;              // stride byte offset: 8 rows * 128 B
    d |= (uint64_t)1 << 46;                        // descriptor version (Blackwell)
    d |= (uint64_t)2 << 61;                        // SWIZZLE_128B
    return d;
}

__device__ __forceinline__ void mma_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// M = 256 over a CTA pair: A rows 0..127 and B rows 0..N/2-1 from the even CTA's shared memory, the rest from the odd CTA's
// (same offsets in both), accumulator rows 0..127 in the even CTA's tensor memory, 128..255 in the odd CTA's.
__device__ __forceinline__ void mma_f16_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// Arrives, when the pair's instructions issued so far have completed, on the barrier at cluster address `cluster_bar`
// (issued once per CTA of the pair: each CTA's producers and epilogue wait on their own copy of the barrier).
__device__ __forceinline__ void mma_commit_pair(uint32_t cluster_bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(cluster_bar) : "memory");
}
__device__ __forceinline__ void mma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&v)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]),
          "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ uint32_t h2_bits(__half2 h) { return *reinterpret_cast<uint32_t*>(&h); }

// TT: the instantiation that takes two-term operands (a_lo_row_arg, w_terms); the one-term kernel carries none of that code.
// PAIR: the CTA-pair form (4-bit formats, one-term operands, no K split, dense launches of an even number of 256-token
// tiles): launched as clusters of two CTAs along x = the token tiles; tile_n is then the pair's tile width.
template <int FMT, bool SPLIT, bool TT, bool PAIR = false>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_q4k_tc_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_w,
                   const __grid_constant__ CUtensorMap tmap_y, int K, int n_out, int t,
                   int tile_n, int m_halves, void* __restrict__ y, int y_dtype_arg, GemmStatus* __restrict__ status, int dbg_arg,
                   const int* __restrict__ tile_expert, F8Scales f8, int k_splits, const float* __restrict__ row_unscale, int a_lo_row_arg, int w_terms,
                   const CUtensorMap* __restrict__ y_more, int n_more) {
    // y_more[0 .. n_more): tensor maps (in global memory) of the other ranks' copies of y, for a row-sharded product whose
    // result every rank wants whole: each staging tile is stored once per destination.
    const int a_lo_row0 = TT ? a_lo_row_arg : 0;
    // Programmatic dependent launch: the kernel behind this one in the stream may start launching now, and this kernel may
    // itself have started before the kernel ahead of it finished. What that kernel wrote is the activations (and their row
    // factors, which the epilogue reads after every activation tile has been consumed): only the activation producer waits
    // for it; the barriers, the tensor memory, the packed weights and their expansion do not depend on it.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    // The timing switches (see debug_switches below) exist only in builds made with -DB2_DEBUG: a production library
    // must not change its results because of an environment variable.
#ifdef B2_DEBUG
    const int dbg = dbg_arg;
#else
    constexpr int dbg = 0;
    (void)dbg_arg;
#endif
    // A "raw block" is what one weight copy brings per row: a 144-byte 4-bit block (256 k, four pipeline
    // stages) or 128 e4m3 bytes (128 k = one column of FP8 scale blocks, two stages).
    // Q8_0 rows are 128 int8 per copy like the FP8 rows; a Q6_K copy brings a row's 128 bytes of low nibbles and, through a
    // second tensor map (y_more[n_more]), its 64 bytes of high bit pairs (the planes of formats.cuh), 256 k = four stages.
    constexpr bool BYTE_ROWS = FMT == B2_FMT_F8E4M3 || FMT == B2_FMT_Q8_0;
    constexpr bool PRE_SCALED = BYTE_ROWS || FMT == B2_FMT_Q6_K;  // the f16 weights carry the factor f8.pre, the epilogue takes it out
    constexpr int RAW_ROW = BYTE_ROWS ? 128 : (FMT == B2_FMT_Q6_K ? 192 : 144);
    constexpr int RAW_ST = BYTE_ROWS ? 2 : 4;
    // bit 8 of the output type: f32 rows that are not 16-byte multiples (n_out % 4 != 0) cannot be described to the copy
    // engine; the epilogue then stores them directly
    const int y_dtype = y_dtype_arg & 0xff;
    const bool y_direct = (y_dtype_arg & 0x100) != 0;
    const long long dbg_k0 = clock64();
    const bool dbg_cta = (dbg & 32768) && blockIdx.x == (PAIR ? 0 : 1) && blockIdx.y == (PAIR ? 1 : 0);
    static_assert(!PAIR || (!SPLIT && !TT && (FMT == B2_FMT_Q4_K || FMT == B2_FMT_MLX4)), "the pair form takes one-term 4-bit operands without a K split");
    constexpr int STAGES = PAIR ? PAIR_STAGES : b2::STAGES;
    // (Q6_K: tiles of at most 208 rows, so that the three B stages leave room for 192 packed bytes per row)
    constexpr int B_STAGE_BYTES = PAIR ? PAIR_B_STAGE_BYTES : (FMT == B2_FMT_Q6_K ? Q6K_MAX_TILE_N * 128 : b2::B_STAGE_BYTES);
    constexpr int RAW_BYTES = PAIR ? PAIR_RAW_BYTES : (FMT == B2_FMT_Q6_K ? Q6K_MAX_TILE_N * 192 : b2::RAW_BYTES);
    static_assert(1024 + STAGES * (A_STAGE_BYTES + B_STAGE_BYTES) + (PAIR ? 2 : 1) * RAW_BYTES + sizeof(Shared) <= (PAIR ? PAIR_SMEM : GEMM_SMEM),
                  "the format's buffers fit the launch's shared memory");
    constexpr int NRAW = PAIR ? 2 : 1;  // staging buffers of packed weights
    // dequantizer sets: groups of warps that take the pipeline stages in turn, one thread per weight row of the CTA's tile
    constexpr int NSETS = PAIR ? 4 : 2, SET_THREADS = 512 / NSETS, SET_WARPS = SET_THREADS / 32;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* a_tiles = smem;
    uint8_t* b_tiles = smem + (size_t)STAGES * A_STAGE_BYTES;
    uint8_t* raw = b_tiles + (size_t)STAGES * B_STAGE_BYTES;
    Shared* sh = (Shared*)(raw + NRAW * RAW_BYTES);
    // pair form: this CTA's rank in its pair (the even CTA issues the instructions) and the rows of the pair's tile it expands
    const uint32_t rank = PAIR ? cluster_rank() : 0u;
    const int my_rows = PAIR ? tile_n / 2 : tile_n;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // K may be divided between the CTAs of blockIdx.z (k_splits of them, whole super-blocks each): every CTA accumulates
    // its share and the epilogue adds the shares into a zeroed y (TMA reduce). sb0: this CTA's first super-block.
    // (SPLIT is a template parameter so that the unsplit kernel carries none of this.)
    const int nsb = SPLIT ? K / (64 * RAW_ST) / k_splits : K / (64 * RAW_ST), nks = nsb * RAW_ST;
    const int sb0 = SPLIT ? (int)blockIdx.z * nsb : 0;
    // (pair form: the two CTAs of a pair are neighbours in x, the dimension a CTA pair is formed along, so there the token
    // tiles run along x and the weight tiles along y)
    const int n0 = (PAIR ? blockIdx.y : blockIdx.x) * tile_n;
    const int m0 = (PAIR ? blockIdx.x : blockIdx.y) * 128 * m_halves;
    // grouped (MoE) launches: the weights of all experts are stacked, n_out rows each, and every token tile
    // belongs to one expert
    const int w_row0 = tile_expert ? tile_expert[blockIdx.y] * n_out : 0;
    // w_terms == 2 (Q4_K, tile_n <= 112): every weight goes into the B operand as two f16 terms, hi in rows 0 .. tile_n - 1 of
    // the stage and lo (what the rounding of hi left of the exact f32 value) in rows 128 .. 128 + tile_n - 1; both are
    // multiplied by the activations into the same accumulator. In each dequantizer set warps 0..3 then write the hi terms of
    // rows 0..127 and warps 4..7 the lo terms of the same rows.
    const bool w2 = TT && w_terms == 2;
    const int row_warps = (my_rows + 31) / 32;
    const int set_warps = w2 ? 2 * row_warps : row_warps;  // live warps in each dequantizer set

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) {
            mbar_init(&sh->a_full[s], 1);
            mbar_init(&sh->b_full[s], (uint32_t)(PAIR ? 2 * set_warps : set_warps));  // pair form: both CTAs' warps arrive on the even CTA's
            mbar_init(&sh->empty[s], 1);
        }
        for (int b = 0; b < NRAW; b++) {
            mbar_init(&sh->raw_full[b], 1);
            mbar_init(&sh->raw_empty[b], (uint32_t)(NSETS * set_warps));
        }
        mbar_init(&sh->acc_full, 1);
        sh->abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        if constexpr (PAIR) {  // the same warp of both CTAs
            asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sh->tmem_base)), "r"(512u)
                         : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
        } else {
            asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sh->tmem_base)), "r"(512u)
                         : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
        }
    }
    tc_fence_before();
    if constexpr (PAIR)
        cluster_sync_all();  // both CTAs' barriers exist before either signals the other's
    else
        __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = sh->tmem_base;

    if (warp == 0) {
        // ---------------- TMA producers: warp 0 streams the activations, warp 18 the packed weights ----------------
        if (lane == 0) {
            asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_x) : "memory");
            // a_lo_row0 > 0 (128-token tiles only): the activations come as two f16 terms, x = hi + lo, with the lo rows stored
            // a_lo_row0 rows below the hi rows; both halves of the stage are filled and both feed the same accumulator, so the
            // activations enter the product with 22 significant bits instead of 11.
            const uint32_t a_bytes = (uint32_t)(128 * (a_lo_row0 > 0 ? 2 : m_halves) * 128);
            int a_issued = 0;
            asm volatile("griddepcontrol.wait;" ::: "memory");  // the activations are complete (see the top of the kernel)
            for (int ks = 0; ks < nks; ks++) {
                const int s = ks % STAGES;
                const uint32_t ph = (uint32_t)((ks / STAGES) & 1);
                if (!mbar_wait<PAIR>(&sh->empty[s], ph ^ 1u, sh, status, 1, (uint32_t)ks)) break;
                if (dbg & 16) {
                    mbar_arrive(&sh->a_full[s]);
                } else {
                    if constexpr (PAIR) {
                        // both CTAs' tiles are counted on the even CTA's barrier, which expects the bytes of both
                        if (rank == 0) mbar_arrive_expect_tx(&sh->a_full[s], 2 * a_bytes);
                        tma_load_2d_pair(a_tiles + (size_t)s * A_STAGE_BYTES, &tmap_x, cluster_addr(&sh->a_full[s], 0), ks * STAGE_K, m0);
                        a_issued = ks + 1;
                        continue;
                    }
                    mbar_arrive_expect_tx(&sh->a_full[s], a_bytes);
                    tma_load_2d(a_tiles + (size_t)s * A_STAGE_BYTES, &tmap_x, &sh->a_full[s], (sb0 * RAW_ST + ks) * STAGE_K, m0);
                    if (a_lo_row0 > 0)
                        tma_load_2d(a_tiles + (size_t)s * A_STAGE_BYTES + 128 * 128, &tmap_x, &sh->a_full[s], (sb0 * RAW_ST + ks) * STAGE_K, a_lo_row0 + m0);
                    a_issued = ks + 1;
                }
            }
            if (sh->abort_flag && (!PAIR || rank == 0)) {
                // Let the copies still in flight land before the CTA's shared memory is released. (Pair form: the odd CTA's
                // copies are counted on the even CTA's barriers; both CTAs meet at the cluster barrier of the teardown, which
                // the even CTA reaches only after these waits.)
                for (int ks = max(0, a_issued - STAGES); ks < a_issued; ks++)
                    mbar_wait<PAIR>(&sh->a_full[ks % STAGES], (uint32_t)((ks / STAGES) & 1), sh, status, 2, (uint32_t)ks, false);
            }
        }
    } else if (warp == 18) {
        if (lane == 0) {
            asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_w) : "memory");
            const uint32_t w_bytes = (uint32_t)(my_rows * RAW_ROW);
            int w_issued = 0;
            for (int sb = 0; sb < nsb; sb++) {
                // the staging buffer is free once every dequant warp has taken its copy of super-block sb - 1,
                // which they do at the start of that super-block: this copy runs a whole super-block ahead
                const int rb = sb % NRAW;
                if (!mbar_wait(&sh->raw_empty[rb], (uint32_t)(((sb / NRAW) & 1) ^ 1), sh, status, 8, (uint32_t)sb)) break;
                if (dbg & 2) {
                    mbar_arrive(&sh->raw_full[rb]);
                    continue;
                }
                mbar_arrive_expect_tx(&sh->raw_full[rb], w_bytes);
                if constexpr (FMT == B2_FMT_Q6_K) {  // [rows][128] low nibbles, then [rows][64] high bit pairs
                    tma_load_2d(raw, &tmap_w, &sh->raw_full[rb], (sb0 + sb) * 128, n0);
                    tma_load_2d(raw + (size_t)my_rows * 128, y_more + n_more, &sh->raw_full[rb], (sb0 + sb) * 64, n0);
                    w_issued = sb + 1;
                    continue;
                }
                tma_load_2d(raw + (size_t)rb * RAW_BYTES, &tmap_w, &sh->raw_full[rb], (sb0 + sb) * RAW_ROW, w_row0 + n0 + (int)rank * my_rows);
                w_issued = sb + 1;
            }
            if (sh->abort_flag)
                for (int sb = max(0, w_issued - NRAW); sb < w_issued; sb++)
                    mbar_wait(&sh->raw_full[sb % NRAW], (uint32_t)((sb / NRAW) & 1), sh, status, 9, (uint32_t)sb, false);
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0 && rank == 0) {
            const uint32_t idesc = (1u << 4) | ((uint32_t)(tile_n >> 3) << 17) | (((PAIR ? 256u : 128u) >> 4) << 24);
            bool ok = true;
            const long long dbg_t0 = clock64();
            long long dbg_wa = 0, dbg_wb = 0;
            const uint64_t a_desc_base = smem_desc_sw128(smem_u32(a_tiles)), b_desc_base = smem_desc_sw128(smem_u32(b_tiles));
            for (int ks = 0; ks < nks && ok; ks++) {
                int s = ks % STAGES;
                uint32_t ph = (uint32_t)((ks / STAGES) & 1);
                const long long w0 = dbg_cta ? clock64() : 0;
                if (!mbar_wait<PAIR>(&sh->a_full[s], ph, sh, status, 3, (uint32_t)ks)) { ok = false; break; }
                const long long w1 = dbg_cta ? clock64() : 0;
                if (!mbar_wait<PAIR>(&sh->b_full[s], ph, sh, status, 4, (uint32_t)ks)) { ok = false; break; }
                const bool dbg_alt = dbg_cta && (dbg & 16384);  // report the issue / commit time instead of the two waits
                if (dbg_cta && !dbg_alt) { dbg_wa += w1 - w0; dbg_wb += clock64() - w1; }
                const long long i0 = dbg_alt ? clock64() : 0;
                tc_fence_after();
                // descriptors differ from the stage-0 ones only in the start-address field (units of 16 bytes)
                const uint64_t adesc0 = a_desc_base + (uint64_t)((uint32_t)s * (A_STAGE_BYTES >> 4));
                const uint64_t bdesc0 = b_desc_base + (uint64_t)((uint32_t)s * (B_STAGE_BYTES >> 4));
                if constexpr (PAIR) {
#pragma unroll
                    for (int kk = 0; kk < STAGE_K / 16; kk++) {
                        if (dbg & 4) break;
                        mma_f16_pair(tmem_base, adesc0 + 2 * kk, bdesc0 + 2 * kk, idesc, (ks > 0 || kk > 0) ? 1u : 0u);
                        mma_f16_pair(tmem_base + 256u, adesc0 + 2 * kk + ((128 * 128) >> 4), bdesc0 + 2 * kk, idesc, (ks > 0 || kk > 0) ? 1u : 0u);
                    }
                    const long long i1 = dbg_alt ? clock64() : 0;
                    mma_commit_pair(cluster_addr(&sh->empty[s], 0));
                    mma_commit_pair(cluster_addr(&sh->empty[s], 1));
                    if (dbg_alt) { dbg_wa += i1 - i0; dbg_wb += clock64() - i1; }
                    continue;
                }
#pragma unroll
                for (int kk = 0; kk < STAGE_K / 16; kk++) {
                    if (!(dbg & 4)) {
                        mma_f16(tmem_base, adesc0 + 2 * kk, bdesc0 + 2 * kk, idesc, (ks > 0 || kk > 0) ? 1u : 0u);
                        if (m_halves == 2) mma_f16(tmem_base + 256u, adesc0 + 2 * kk + ((128 * 128) >> 4), bdesc0 + 2 * kk, idesc, (ks > 0 || kk > 0) ? 1u : 0u);
                        if (a_lo_row0 > 0) mma_f16(tmem_base, adesc0 + 2 * kk + ((128 * 128) >> 4), bdesc0 + 2 * kk, idesc, 1u);
                        if (w2) {  // the weights' lo terms against the activations' hi terms (lo x lo is below f32's own rounding)
                            mma_f16(tmem_base, adesc0 + 2 * kk, bdesc0 + 2 * kk + ((128 * 128) >> 4), idesc, 1u);
                            if (m_halves == 2) mma_f16(tmem_base + 256u, adesc0 + 2 * kk + ((128 * 128) >> 4), bdesc0 + 2 * kk + ((128 * 128) >> 4), idesc, 1u);
                        }
                    }
                }
                const long long i1 = dbg_alt ? clock64() : 0;
                mma_commit(&sh->empty[s]);
                if (dbg_alt) { dbg_wa += i1 - i0; dbg_wb += clock64() - i1; }
            }
            if constexpr (PAIR) {
                mma_commit_pair(cluster_addr(&sh->acc_full, 0));
                mma_commit_pair(cluster_addr(&sh->acc_full, 1));
            } else {
                mma_commit(&sh->acc_full);
            }
            if (dbg_cta) { status->where = (uint32_t)(clock64() - dbg_t0); status->iter = (uint32_t)nks; status->t[0] = (uint32_t)(dbg_t0 - dbg_k0); status->t[1] = (uint32_t)(clock64() - dbg_k0); status->t[5] = (uint32_t)dbg_wa; status->t[6] = (uint32_t)dbg_wb; }
            if (!ok) mbar_wait(&sh->acc_full, 0, sh, status, 5, 0, false);  // drain what was issued before teardown
        }
    } else {
        // ---------------- dequantizers, then epilogue ----------------
        // Two sets of eight warps take the pipeline stages in turn (set 0 the even k-stages, set 1 the odd
        // ones), one thread per weight row: a warp then has two stage times for the serial chain
        // "expand 64 weights, wait for the slot, store, fence, arrive", and half as many waits per weight.
        const int dq_warp = warp - 2;
        const int dt = threadIdx.x - 64;
        const int set = dt / SET_THREADS;
        const int r = w2 ? (dt & 127) : (dt & (SET_THREADS - 1));  // weight row of this CTA's tile
        const bool is_lo = w2 && (dt & 128);
        bool ok = true;
        if ((w2 ? (dq_warp & 3) : (dq_warp & (SET_WARPS - 1))) < row_warps) {
            const bool in_tile = r < my_rows;
            const uint32_t b_full_even = PAIR ? cluster_addr(&sh->b_full[0], 0) : 0u;  // the even CTA's b_full[0]
            const uint32_t row_off = (uint32_t)(r + (is_lo ? 128 : 0)) * 128u;
            const uint32_t swz = (uint32_t)(r & 7);
            const uint4* my_raw0 = (const uint4*)(raw + (size_t)(in_tile ? r : 0) * (FMT == B2_FMT_Q6_K ? 128 : RAW_ROW));
            for (int sb = 0; sb < nsb && ok; sb++) {
                const int rb = sb % NRAW;
                const uint4* my_raw = (const uint4*)((const uint8_t*)my_raw0 + (size_t)rb * RAW_BYTES);
                // this row's packed super-block: staging buffer -> registers (only the two 64-groups this set
                // expands), then release the buffer
                if (!mbar_wait(&sh->raw_full[rb], (uint32_t)((sb / NRAW) & 1), sh, status, 10, (uint32_t)sb)) {
                    ok = false;
                    break;
                }
                if constexpr (FMT == B2_FMT_Q6_K) {
                    // Stage j of the super-block = elements 64 j .. 64 j + 63 = half n = j / 2 of the block, its low (j even) or
                    // high (j odd) nibbles with bit pairs (0, 2) or (4, 6) of the half's 32 qh bytes (src/ggml.rs Q6_K decode):
                    // element e < 32: ql[64 n + e] and qh[32 n + e] >> 4 odd; e >= 32: ql[64 n + e] and qh[32 n + e - 32] >> (4 odd + 2).
                    // The staged tiles are swizzled by the copy engine: 16-byte chunk c of a ql row at c ^ (r & 7), of a qh row at
                    // c ^ ((r >> 1) & 3). w = f16(d sc pre) * (q - 32), q - 32 exact in f16.
                    const uint4* my_qh = (const uint4*)(raw + (size_t)my_rows * 128 + (size_t)(in_tile ? r : 0) * 64);
                    const uint32_t swh = (uint32_t)((r >> 1) & 3);
                    const size_t wrow = (size_t)(n0 + r);
                    const bool live = in_tile && n0 + r < n_out;
                    const float d = live ? __half2float(__ushort_as_half(__ldg((const unsigned short*)f8.s2 + wrow * (size_t)(K / 256) + sb0 + sb))) : 0.0f;
#pragma unroll
                    for (int jj = 0; jj < 2; jj++) {
                        const int j = set + 2 * jj, n = j >> 1, odd = j & 1;
                        uint4 ql4[4], qh4[2];
#pragma unroll
                        for (int c = 0; c < 4; c++) ql4[c] = my_raw[((uint32_t)(4 * n + c)) ^ swz];
#pragma unroll
                        for (int c = 0; c < 2; c++) qh4[c] = my_qh[((uint32_t)(2 * n + c)) ^ swh];
                        if (jj == 1) {  // the row's last read of this super-block's staging buffer
                            __syncwarp();
                            if (lane == 0) mbar_arrive(&sh->raw_empty[rb]);
                        }
                        const uint32_t sc4 = live ? __ldg((const uint32_t*)((const int8_t*)f8.s + wrow * (size_t)(K / 16) + (size_t)(sb0 + sb) * 16 + 4 * j)) : 0u;
                        __half2 mul[4];
#pragma unroll
                        for (int i = 0; i < 4; i++) mul[i] = __float2half2_rn(d * (float)(int8_t)(sc4 >> (8 * i)) * f8.pre);
                        const int ks = sb * 4 + j;
                        const int s = ks % STAGES;
                        const uint32_t ph = (uint32_t)((ks / STAGES) & 1);
                        const uint32_t qlw[16] = {ql4[0].x, ql4[0].y, ql4[0].z, ql4[0].w, ql4[1].x, ql4[1].y, ql4[1].z, ql4[1].w,
                                                  ql4[2].x, ql4[2].y, ql4[2].z, ql4[2].w, ql4[3].x, ql4[3].y, ql4[3].z, ql4[3].w};
                        const uint32_t qhw[8] = {qh4[0].x, qh4[0].y, qh4[0].z, qh4[0].w, qh4[1].x, qh4[1].y, qh4[1].z, qh4[1].w};
                        const __half2 bias = __float2half2_rn(1056.0f);  // 1024 (the exponent trick) + 32
                        uint32_t o[32];
#pragma unroll
                        for (int i = 0; i < 16; i++) {  // word i: elements 4 i .. 4 i + 3 of the stage
                            const uint32_t nib = odd ? (qlw[i] >> 4) & 0x0F0F0F0Fu : qlw[i] & 0x0F0F0F0Fu;
                            const uint32_t hb = ((qhw[i & 7] >> (4 * odd + 2 * (i >> 3))) & 0x03030303u) << 4;
                            const uint32_t q4 = nib | hb;
                            uint32_t p0 = __byte_perm(q4, 0, 0x4140) | 0x64006400u, p1 = __byte_perm(q4, 0, 0x4342) | 0x64006400u;
                            o[2 * i] = h2_bits(__hmul2(__hsub2(*reinterpret_cast<__half2*>(&p0), bias), mul[i >> 2]));
                            o[2 * i + 1] = h2_bits(__hmul2(__hsub2(*reinterpret_cast<__half2*>(&p1), bias), mul[i >> 2]));
                        }
                        if (!mbar_wait<PAIR>(&sh->empty[s], ph ^ 1u, sh, status, 6, (uint32_t)ks)) {
                            ok = false;
                            break;
                        }
                        if (in_tile && !(dbg & 1)) {
                            uint8_t* dst = b_tiles + (size_t)s * B_STAGE_BYTES + row_off;
#pragma unroll
                            for (int c = 0; c < 8; c++)
                                *(uint4*)(dst + ((((uint32_t)c) ^ swz) << 4)) = make_uint4(o[4 * c], o[4 * c + 1], o[4 * c + 2], o[4 * c + 3]);
                        }
                        fence_proxy_async();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(&sh->b_full[s]);
                    }
                    continue;
                }
                if constexpr (BYTE_ROWS) {
                    // 64 e4m3 bytes of this set's stage (the raw tile is 128-byte swizzled: chunk c of row r sits
                    // at c ^ (r & 7)), the block scale of this row and k-block, then hardware e4m3x2 -> f16x2
                    // and one multiply by the scale per pair.
                    uint4 qb[4];
#pragma unroll
                    for (int c = 0; c < 4; c++) qb[c] = my_raw[((uint32_t)(4 * set + c)) ^ swz];
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&sh->raw_empty[rb]);
                    const int ks = sb * 2 + set;
                    const int s = ks % STAGES;
                    const uint32_t ph = (uint32_t)((ks / STAGES) & 1);
                    uint32_t o[32];
                    if constexpr (FMT == B2_FMT_Q8_0) {
                        // 64 int8 of this set's stage = two blocks of 32 with an f16 scale each (src/ggml.rs Q8_0 decode): byte b ^ 0x80
                        // under the exponent 0x64 is the f16 1024 + (q + 128), minus 1152 = q exactly, times f16(d pre)
                        uint32_t d2 = 0u;
                        if (in_tile && n0 + r < n_out)
                            d2 = __ldg((const uint32_t*)((const unsigned short*)f8.s + (size_t)(n0 + r) * (size_t)f8.ncb + (size_t)(sb0 + sb) * 4 + set * 2));
                        const __half2 m0 = __float2half2_rn(__half2float(__ushort_as_half((unsigned short)(d2 & 0xffffu))) * f8.pre);
                        const __half2 m1 = __float2half2_rn(__half2float(__ushort_as_half((unsigned short)(d2 >> 16))) * f8.pre);
                        const __half2 bias = __float2half2_rn(1152.0f);
#pragma unroll
                        for (int c = 0; c < 4; c++) {
                            const uint32_t wds[4] = {qb[c].x, qb[c].y, qb[c].z, qb[c].w};
#pragma unroll
                            for (int i = 0; i < 4; i++) {
                                const uint32_t u = wds[i] ^ 0x80808080u;
                                uint32_t p0 = __byte_perm(u, 0, 0x4140) | 0x64006400u, p1 = __byte_perm(u, 0, 0x4342) | 0x64006400u;
                                o[8 * c + 2 * i] = h2_bits(__hmul2(__hsub2(*reinterpret_cast<__half2*>(&p0), bias), c < 2 ? m0 : m1));
                                o[8 * c + 2 * i + 1] = h2_bits(__hmul2(__hsub2(*reinterpret_cast<__half2*>(&p1), bias), c < 2 ? m0 : m1));
                            }
                        }
                    }
                    float scale = 1.0f;
                    if (FMT == B2_FMT_F8E4M3 && f8.s && in_tile && n0 + r < n_out) scale = __ldg(f8.s + (size_t)((f8.row0 + n0 + r) / f8.rows) * f8.ncb + sb0 + sb);
                    const __half2 sc2 = __float2half2_rn(scale * f8.pre);
#pragma unroll
                    for (int c = 0; c < 4; c++) {
                        if (FMT != B2_FMT_F8E4M3) break;
                        const uint32_t wds[4] = {qb[c].x, qb[c].y, qb[c].z, qb[c].w};
#pragma unroll
                        for (int i = 0; i < 4; i++) {
                            __half2_raw h01 = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(wds[i] & 0xffff), __NV_E4M3);
                            __half2_raw h23 = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(wds[i] >> 16), __NV_E4M3);
                            o[8 * c + 2 * i] = h2_bits(__hmul2(*reinterpret_cast<__half2*>(&h01), sc2));
                            o[8 * c + 2 * i + 1] = h2_bits(__hmul2(*reinterpret_cast<__half2*>(&h23), sc2));
                        }
                    }
                    if (!mbar_wait<PAIR>(&sh->empty[s], ph ^ 1u, sh, status, 6, (uint32_t)ks)) {
                        ok = false;
                        break;
                    }
                    if (in_tile && !(dbg & 1)) {
                        uint8_t* dst = b_tiles + (size_t)s * B_STAGE_BYTES + row_off;
#pragma unroll
                        for (int c = 0; c < 8; c++)
                            *(uint4*)(dst + ((((uint32_t)c) ^ swz) << 4)) = make_uint4(o[4 * c], o[4 * c + 1], o[4 * c + 2], o[4 * c + 3]);
                    }
                    fence_proxy_async();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&sh->b_full[s]);
                    continue;
                }
                const uint4 hdr = my_raw[0];
                uint4 q[2 * (4 / NSETS)];
#pragma unroll
                for (int jj = 0; jj < 4 / NSETS; jj++) {
                    q[2 * jj] = my_raw[1 + 2 * (set + NSETS * jj)];
                    q[2 * jj + 1] = my_raw[2 + 2 * (set + NSETS * jj)];
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(&sh->raw_empty[rb]);
#pragma unroll
                for (int jj = 0; jj < 4 / NSETS; jj++) {
                    const int j = set + NSETS * jj;
                    const int ks = sb * 4 + j;
                    const int s = ks % STAGES;
                    const uint32_t ph = (uint32_t)((ks / STAGES) & 1);
                    // low nibbles: 0x6400 | n = 1024 + n; high nibbles stay in place: 0x6400 | (n << 4) = 1024 + 16 n.
                    // Both formats take two fmas per pair, t = h * c1 + c2 (an exact small integer) and
                    // w = t * dmul + add:
                    //   Q4_K : t = n * sc    (c1 = sc or sc/16, c2 = -1024 sc or -64 sc), w = t * d - f16(dmin * m)
                    //   MLX-4: t = n - 8     (c1 = 1 or 1/16,   c2 = -1032 or -72),      w = t * f16(scale) + f16(offset)
                    // so only the min / offset term and the result are rounded.
                    __half2 dmul, c1lo, c2lo, c1hi, c2hi, addlo, addhi;
                    if constexpr (FMT == B2_FMT_MLX4) {
                        const uint32_t sw = (j & 2) ? hdr.y : hdr.x, bw = (j & 2) ? hdr.w : hdr.z;
                        const float off = bf16_bits_to_f32((bw >> (16 * (j & 1))) & 0xffffu);
                        dmul = __half2half2(__ushort_as_half((unsigned short)((sw >> (16 * (j & 1))) & 0xffffu)));
                        c1lo = __float2half2_rn(1.0f);
                        c2lo = __float2half2_rn(-1032.0f);
                        c1hi = __float2half2_rn(0.0625f);
                        c2hi = __float2half2_rn(-72.0f);
                        addlo = addhi = __float2half2_rn(off);
                    } else {
                        uint32_t sc0, mn0, sc1, mn1;
                        q4k_scale_min(2 * j, hdr.y, hdr.z, hdr.w, sc0, mn0);
                        q4k_scale_min(2 * j + 1, hdr.y, hdr.z, hdr.w, sc1, mn1);
                        const float dmin = __half2float(__ushort_as_half((unsigned short)(hdr.x >> 16)));
                        dmul = __half2half2(__ushort_as_half((unsigned short)(hdr.x & 0xffff)));
                        c1lo = __float2half2_rn((float)sc0);
                        c2lo = __float2half2_rn(-1024.0f * (float)sc0);
                        c1hi = __float2half2_rn(0.0625f * (float)sc1);
                        c2hi = __float2half2_rn(-64.0f * (float)sc1);
                        addlo = __float2half2_rn(-(dmin * (float)mn0));
                        addhi = __float2half2_rn(-(dmin * (float)mn1));
                    }
                    const uint32_t qw[8] = {q[2 * jj].x,     q[2 * jj].y,     q[2 * jj].z,     q[2 * jj].w,
                                            q[2 * jj + 1].x, q[2 * jj + 1].y, q[2 * jj + 1].z, q[2 * jj + 1].w};
                    uint32_t lo[16], hi[16];
#pragma unroll
                    for (int i = 0; i < 8; i++) {
                        // bytes 4i .. 4i+3 of the group -> k = 4i .. 4i+3 (low nibbles) and 32 + 4i .. (high nibbles)
                        uint32_t p0 = __byte_perm(qw[i], 0, 0x4140), p1 = __byte_perm(qw[i], 0, 0x4342);
                        uint32_t l0 = (p0 & 0x000F000Fu) | 0x64006400u, l1 = (p1 & 0x000F000Fu) | 0x64006400u;
                        uint32_t h0 = (p0 & 0x00F000F0u) | 0x64006400u, h1 = (p1 & 0x00F000F0u) | 0x64006400u;
                        lo[2 * i] = h2_bits(__hfma2(__hfma2(*reinterpret_cast<__half2*>(&l0), c1lo, c2lo), dmul, addlo));
                        lo[2 * i + 1] = h2_bits(__hfma2(__hfma2(*reinterpret_cast<__half2*>(&l1), c1lo, c2lo), dmul, addlo));
                        hi[2 * i] = h2_bits(__hfma2(__hfma2(*reinterpret_cast<__half2*>(&h0), c1hi, c2hi), dmul, addhi));
                        hi[2 * i + 1] = h2_bits(__hfma2(__hfma2(*reinterpret_cast<__half2*>(&h1), c1hi, c2hi), dmul, addhi));
                    }
                    if constexpr (FMT == B2_FMT_Q4_K) {
                        if (is_lo) {
                            // the second term: the exact f32 weight of the reference's decode, d1 * q - m1 with both roundings
                            // (src/ggml.rs:750-773), minus the f16 the hi warps wrote (the same arithmetic as above)
                            uint32_t sc0, mn0, sc1, mn1;
                            q4k_scale_min(2 * j, hdr.y, hdr.z, hdr.w, sc0, mn0);
                            q4k_scale_min(2 * j + 1, hdr.y, hdr.z, hdr.w, sc1, mn1);
                            const float d = __half2float(__ushort_as_half((unsigned short)(hdr.x & 0xffff)));
                            const float dmin = __half2float(__ushort_as_half((unsigned short)(hdr.x >> 16)));
                            const float d1l = __fmul_rn(d, (float)sc0), m1l = __fmul_rn(dmin, (float)mn0);
                            const float d1h = __fmul_rn(d, (float)sc1), m1h = __fmul_rn(dmin, (float)mn1);
#pragma unroll
                            for (int i = 0; i < 8; i++) {
#pragma unroll
                                for (int e = 0; e < 2; e++) {  // bytes 4i + 2e, 4i + 2e + 1 of the group
                                    const uint32_t b0 = (qw[i] >> (16 * e)) & 0xffu, b1 = (qw[i] >> (16 * e + 8)) & 0xffu;
                                    const float2 hl = __half22float2(*reinterpret_cast<const __half2*>(&lo[2 * i + e]));
                                    const float2 hh = __half22float2(*reinterpret_cast<const __half2*>(&hi[2 * i + e]));
                                    const float vl0 = __fsub_rn(__fmul_rn(d1l, __uint_as_float(0x4B000000u | (b0 & 15u)) - 8388608.0f), m1l);
                                    const float vl1 = __fsub_rn(__fmul_rn(d1l, __uint_as_float(0x4B000000u | (b1 & 15u)) - 8388608.0f), m1l);
                                    const float vh0 = __fsub_rn(__fmul_rn(d1h, __uint_as_float(0x4B000000u | (b0 >> 4)) - 8388608.0f), m1h);
                                    const float vh1 = __fsub_rn(__fmul_rn(d1h, __uint_as_float(0x4B000000u | (b1 >> 4)) - 8388608.0f), m1h);
                                    lo[2 * i + e] = h2_bits(__floats2half2_rn(vl0 - hl.x, vl1 - hl.y));
                                    hi[2 * i + e] = h2_bits(__floats2half2_rn(vh0 - hh.x, vh1 - hh.y));
                                }
                            }
                        }
                    }
                    if (!mbar_wait<PAIR>(&sh->empty[s], ph ^ 1u, sh, status, 6, (uint32_t)ks)) {
                        ok = false;
                        break;
                    }
                    if (in_tile && !(dbg & 1)) {
                        uint8_t* dst = b_tiles + (size_t)s * B_STAGE_BYTES + row_off;
#pragma unroll
                        for (int c = 0; c < 4; c++) {
                            *(uint4*)(dst + ((((uint32_t)c) ^ swz) << 4)) = make_uint4(lo[4 * c], lo[4 * c + 1], lo[4 * c + 2], lo[4 * c + 3]);
                            *(uint4*)(dst + ((((uint32_t)(c + 4)) ^ swz) << 4)) = make_uint4(hi[4 * c], hi[4 * c + 1], hi[4 * c + 2], hi[4 * c + 3]);
                        }
                    }
                    fence_proxy_async();
                    __syncwarp();
                    if (lane == 0) {
                        if constexpr (PAIR)
                            mbar_arrive_cluster(b_full_even + (uint32_t)s * 8u);
                        else
                            mbar_arrive(&sh->b_full[s]);
                    }
                }
            }
        }
        // Epilogue: warp (warp % 4) may touch TMEM lanes 32 (warp % 4) .. +32. Sixteen warps: four per
        // lane quarter, split over the two accumulator halves and the even / odd 16-column chunks.
        const int quarter = warp & 3;
        const int half = (dq_warp >> 2) & 1;
        const int cpar = dq_warp >> 3;
        if (half < m_halves) {
            bool acc_ok = mbar_wait<PAIR>(&sh->acc_full, 0, sh, status, 7, 0) && !sh->abort_flag;
            acc_ok = __all_sync(0xffffffffu, acc_ok);
            if (dbg_cta && threadIdx.x == 64) status->t[2] = (uint32_t)(clock64() - dbg_k0);
            if (acc_ok) {
                tc_fence_after();
                const int token0 = m0 + half * 128 + quarter * 32;
                const int token = token0 + lane;
                // the activations of a token row may have been scaled by a power of two on their way to f16 (to_f16_rows):
                // its results are scaled back here, exactly
                const bool scaled = PRE_SCALED || row_unscale != nullptr;
                const float out_scale = (PRE_SCALED ? 1.0f / f8.pre : 1.0f) * ((row_unscale && token < t) ? __ldg(row_unscale + token) : 1.0f);
                const uint32_t taddr0 = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(half * 256);
                int c0 = cpar * 32;
                if (y_dtype == B2_F32 && !y_direct && !(dbg & 64)) {
                    // f32 output through shared memory and TMA stores: each warp owns two 4 KB staging tiles
                    // (32 tokens x 32 columns, 128-byte swizzle) in the now idle pipeline buffers, fills one
                    // from TMEM, and lets the copy engine write it out while it fills the other. The tensor
                    // map clips rows past t and columns past n_out.
                    uint8_t* stage = smem + (size_t)dq_warp * 8192;
                    int it = 0;
                    for (; c0 + 32 <= tile_n; c0 += 64, it++) {
                        uint8_t* buf = stage + (it & 1) * 4096;
                        if (it >= 2) {  // the store issued two rounds ago has finished reading this tile
                            if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
                            __syncwarp();
                        }
                        uint32_t v[16], u[16];
                        tmem_ld16(taddr0 + (uint32_t)c0, v);
                        tmem_ld16(taddr0 + (uint32_t)c0 + 16u, u);
                        if (scaled) {
#pragma unroll
                            for (int i = 0; i < 16; i++) {
                                v[i] = __float_as_uint(__uint_as_float(v[i]) * out_scale);
                                u[i] = __float_as_uint(__uint_as_float(u[i]) * out_scale);
                            }
                        }
                        uint8_t* rowp = buf + lane * 128;
                        const uint32_t sw = (uint32_t)(lane & 7);
#pragma unroll
                        for (int pce = 0; pce < 4; pce++) {
                            *(uint4*)(rowp + ((((uint32_t)pce) ^ sw) << 4)) = make_uint4(v[4 * pce], v[4 * pce + 1], v[4 * pce + 2], v[4 * pce + 3]);
                            *(uint4*)(rowp + ((((uint32_t)(pce + 4)) ^ sw) << 4)) = make_uint4(u[4 * pce], u[4 * pce + 1], u[4 * pce + 2], u[4 * pce + 3]);
                        }
                        fence_proxy_async();
                        __syncwarp();
                        if (lane == 0 && !(dbg & 8)) {
                            if (SPLIT)
                                asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3}], [%1];" ::"l"(&tmap_y),
                                             "r"(smem_u32(buf)), "r"(n0 + c0), "r"(token0)
                                             : "memory");
                            else
                                asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(&tmap_y),
                                             "r"(smem_u32(buf)), "r"(n0 + c0), "r"(token0)
                                             : "memory");
                            for (int d = 0; d < n_more; d++)  // the same tile into the peers' y, through their mapped memory
                                asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(y_more + d),
                                             "r"(smem_u32(buf)), "r"(n0 + c0), "r"(token0)
                                             : "memory");
                            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                        }
                    }
                    // a 16-column tail (tile_n not a multiple of 32) goes to the warps whose turn it would be
                    c0 = ((tile_n & 31) && ((tile_n >> 5) & 1) == cpar) ? (tile_n & ~31) : tile_n;
                }
                const int step = (y_dtype == B2_F32 && !y_direct && !(dbg & 64)) ? tile_n : 64;
                for (; c0 < tile_n; c0 += step) {
                  for (int cc = c0; cc < min(c0 + 32, tile_n); cc += 16) {
                    uint32_t v[16];
                    tmem_ld16(taddr0 + (uint32_t)cc, v);
                    if (scaled) {
#pragma unroll
                        for (int i = 0; i < 16; i++) v[i] = __float_as_uint(__uint_as_float(v[i]) * out_scale);
                    }
                    if (token < t && !(dbg & 8)) {
                        int n = n0 + cc;
                        if (y_dtype == B2_F32) {
                            float* o = (float*)y + (size_t)token * n_out + n;
                            if (SPLIT) {  // this CTA's share of K: added to the other share (y starts at zero)
#pragma unroll
                                for (int i = 0; i < 16; i++)
                                    if (n + i < n_out) atomicAdd(o + i, __uint_as_float(v[i]));
                            } else if (n + 16 <= n_out && (n_out & 3) == 0) {
#pragma unroll
                                for (int i = 0; i < 4; i++)
                                    ((float4*)o)[i] = make_float4(__uint_as_float(v[4 * i]), __uint_as_float(v[4 * i + 1]),
                                                                  __uint_as_float(v[4 * i + 2]), __uint_as_float(v[4 * i + 3]));
                            } else {
#pragma unroll
                                for (int i = 0; i < 16; i++)
                                    if (n + i < n_out) o[i] = __uint_as_float(v[i]);
                            }
                        } else {
                            __nv_bfloat16* o = (__nv_bfloat16*)y + (size_t)token * n_out + n;
                            if (n + 16 <= n_out && (n_out & 7) == 0) {
                                uint32_t pk[8];
#pragma unroll
                                for (int i = 0; i < 8; i++) {
                                    __nv_bfloat162 b = __floats2bfloat162_rn(__uint_as_float(v[2 * i]), __uint_as_float(v[2 * i + 1]));
                                    pk[i] = *reinterpret_cast<uint32_t*>(&b);
                                }
                                ((uint4*)o)[0] = make_uint4(pk[0], pk[1], pk[2], pk[3]);
                                ((uint4*)o)[1] = make_uint4(pk[4], pk[5], pk[6], pk[7]);
                            } else {
#pragma unroll
                                for (int i = 0; i < 16; i++)
                                    if (n + i < n_out) o[i] = __float2bfloat16_rn(__uint_as_float(v[i]));
                            }
                        }
                    }
                  }
                }
                // the staging tiles must have been read out before the CTA's shared memory goes away
                if (lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
                __syncwarp();
            }
        }
    }

    if (dbg_cta && threadIdx.x == 64) status->t[3] = (uint32_t)(clock64() - dbg_k0);
    tc_fence_before();
    if constexpr (PAIR)
        cluster_sync_all();  // neither CTA's shared or tensor memory goes away while the other may still signal or read it
    else
        __syncthreads();
    if (dbg_cta && threadIdx.x == 64) status->t[4] = (uint32_t)(clock64() - dbg_k0);
    if (warp == 1) {
        tc_fence_after();
        if constexpr (PAIR)
            asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
        else
            asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
    }
}

// One token row to f16 operands, scaled by a power of two so that its largest magnitude lands in [2^14, 2^15): rows
// of any magnitude (the reference's own tests use rows scaled by 1e-3 .. 2e5, src/cuda.rs:1579-1700) neither overflow
// f16 nor sink into its subnormals, and since the factor is a power of two the rounding is the same relative rounding
// at every magnitude. unscale[row] = 1 / factor is what the GEMM's epilogue multiplies the row's results by (exact).
// lo_off > 0: the remainder x * factor - f16(x * factor) is written lo_off elements behind each value (two-term activations).
// One CTA per row; NaN elements stay NaN, a row with an infinity is passed through unscaled.
__device__ __forceinline__ float load_as_float(const float* p) { return *p; }
__device__ __forceinline__ float load_as_float(const __nv_bfloat16* p) { return __bfloat162float(*p); }
__device__ __forceinline__ float load_as_float(const __half* p) { return __half2float(*p); }

template <typename T>
__global__ void __launch_bounds__(256) to_f16_rows_kernel(const T* __restrict__ x, int K, __half* __restrict__ out, float* __restrict__ unscale,
                                                          size_t lo_off, size_t x_ld) {
    __shared__ float red[8];
    // (a dependent launch: the GEMM behind it may set itself up meanwhile; the GEMM ahead of it may still be reading `out`)
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const T* xr = x + (size_t)blockIdx.x * x_ld;
    __half* o = out + (size_t)blockIdx.x * K;
    float mx = 0.0f;
    for (int i = threadIdx.x; i < K; i += 256) mx = fmaxf(mx, fabsf(load_as_float(xr + i)));
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, d));
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = mx;
    __syncthreads();
    mx = red[0];
#pragma unroll
    for (int i = 1; i < 8; i++) mx = fmaxf(mx, red[i]);
    float s = 1.0f, inv = 1.0f;
    if (mx > 0.0f && mx < INFINITY) {
        int e;
        frexpf(mx, &e);                       // mx = m 2^e, m in [0.5, 1)
        const int up = min(100, max(-100, 15 - e));
        s = ldexpf(1.0f, up);
        inv = ldexpf(1.0f, -up);
    }
    for (int i = threadIdx.x * 2; i < K; i += 512) {  // K is even (a multiple of 64)
        const float a = load_as_float(xr + i) * s, b = load_as_float(xr + i + 1) * s;
        const __half2 h = __floats2half2_rn(a, b);
        *(__half2*)(o + i) = h;
        if (lo_off) {  // the second term: what the rounding to f16 left over (exact in f32, rounded once more)
            const float2 hf = __half22float2(h);
            *(__half2*)(o + lo_off + i) = __floats2half2_rn(a - hf.x, b - hf.y);
        }
    }
    if (threadIdx.x == 0) unscale[blockIdx.x] = inv;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
    }
    return fn;
}

// Only in builds made with -DB2_DEBUG (make EXTRA=-DB2_DEBUG), B2_GEMM_DEBUG selects diagnostic switches for timing
// experiments (the results are WRONG when any of the first five is set): 1 skip the dequantizers' shared-memory
// stores, 2 skip the weight copies, 4 skip the MMAs, 8 skip the epilogue's stores, 16 skip the activation copies;
// 64 epilogue by direct stores instead of TMA stores; 32768 make CTA (1, 0) write cycle stamps of its phases into the
// status word. The shipped library ignores the variable.
int debug_switches() {
#ifdef B2_DEBUG
    const char* e = getenv("B2_GEMM_DEBUG");
    return e ? atoi(e) : 0;
#else
    return 0;
#endif
}

}  // namespace

struct GemmPlan {
    CUtensorMap tmap_x, tmap_w, tmap_y;
    const int* tile_expert = nullptr;  // grouped launches: expert of each token tile (device)
    size_t experts = 1;
    const void* x16;
    const void* wptr;
    const void* y;
    int y_dtype;
    size_t t, K, n_out;
    int tile_n, m_halves, n_tiles, m_tiles;
    int k_splits = 1;
    bool y_direct = false;  // f32 output whose rows the copy engine cannot take (stride not a multiple of 16 bytes)
    CUtensorMap* y_more = nullptr;  // device array of n_more tensor maps: the peers' copies of y (GemmPeerY)
    int n_more = 0;
    size_t y_ld = 0;
    float* more_ptr[7] = {};
    bool pair = false;     // the CTA-pair form: clusters of two CTAs along the token tiles, tile_n the pair's width
    bool pair_asked = false;  // B2_GEMM_PAIR when the plan was made (a cached plan is reused only under the same setting)
    int w_terms = 1;       // 2: two-term weights (Q4_K, tile_n <= 112)
    size_t a_lo_row0 = 0;  // two-term activations: the lo rows start this many rows below the hi rows (0: one term)
    int split_asked = 1;  // B2_GEMM_SPLIT_K when the plan was made (a cached plan is reused only under the same setting)
};

bool gemm_tc_supports(const WeightDev& w, size_t t) {
    if (w.fmt == B2_FMT_F8E4M3) return w.n_in % 128 == 0 && t >= 1 && ((uintptr_t)w.p0 & 15) == 0 && (w.p1 == nullptr || w.bs_cols == 128);
    if (w.fmt == B2_FMT_Q8_0) return w.n_in % 128 == 0 && t >= 1 && ((uintptr_t)w.p0 & 15) == 0 && ((uintptr_t)w.p1 & 3) == 0;
    if (w.fmt == B2_FMT_Q6_K) return w.n_in % 256 == 0 && t >= 1 && (((uintptr_t)w.p0 | (uintptr_t)w.p1) & 15) == 0 && ((uintptr_t)w.p2 & 3) == 0;
    return (w.fmt == B2_FMT_Q4_K || w.fmt == B2_FMT_MLX4) && w.n_in % 256 == 0 && t >= 1 && ((uintptr_t)w.p0 & 15) == 0;
}

// B2_GEMM_PAIR=1 selects the CTA-pair form where a launch qualifies. It is off by default: at the benchmark shape it
// measures 60.7 us against 57.2 us for the single-CTA form (same build), with bit-identical results.
static bool pair_form_enabled() {
    const char* e = getenv("B2_GEMM_PAIR");
    return e && atoi(e) != 0;
}

static int split_k_asked() {
    const char* e = getenv("B2_GEMM_SPLIT_K");
    return e ? atoi(e) : 1;
}

// Tile width (weight rows per CTA): the multiple of 16 up to MAX_TILE_N that minimizes the time of the slowest SM,
// waves x (time of one CTA), over the grid ceil(n_out / tile_n) * m_tiles. A CTA's time is mostly its k loop, whose stage
// time hardly depends on the width (1108 cycles per stage at 208 rows, 1152 at 104), plus an epilogue that grows with
// the width; in units of rows the measurements fit (tile_n + 13 per k stage), with widths above 208 costing about five
// times as much per extra row (58-60 us at 240 against 54 at 208 for 64 stages). So the count of waves decides first.
static int pick_tile_n(size_t n_out, int m_tiles, int sm_count, size_t K, int widest = MAX_TILE_N, int step = 16) {
    // B2_GEMM_TILE_N forces a width (tests and tuning sweeps).
    if (const char* env = getenv("B2_GEMM_TILE_N")) {
        int v = atoi(env);
        if (v >= 16 && v <= widest && v % step == 0) return v;
    }
    const double per_cta = 24.0 + 13.0 * (double)(K / 64);
    int best = widest;
    double best_cost = 1e30;
    for (int tn = widest; tn >= 64; tn -= step) {
        size_t tiles = (n_out + tn - 1) / tn * (size_t)m_tiles;
        size_t waves = (tiles + sm_count - 1) / sm_count;
        double cost = (double)waves * (tn + per_cta + (tn > 208 ? 4.0 * (tn - 208) : 0.0));
        if (cost < best_cost - 1e-9) {
            best_cost = cost;
            best = tn;
        }
    }
    return best;
}

// Q6_K's qh plane [n_out][K / 4] bytes: boxes of 64 bytes x tile rows, 64-byte swizzle (conflict-free 16-byte reads by row).
static CUresult encode_q6k_qh(EncodeTiledFn enc, CUtensorMap* m, const WeightDev& w, int tile_n) {
    cuuint64_t dims[2] = {(cuuint64_t)(w.n_in / 4), (cuuint64_t)w.n_out};
    cuuint64_t strides[1] = {(cuuint64_t)(w.n_in / 4)};
    cuuint32_t box[2] = {64u, (cuuint32_t)tile_n};
    cuuint32_t estr[2] = {1, 1};
    return enc(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, (void*)w.p1, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B,
               CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
}

cudaError_t gemm_tc_plan_create(const WeightDev& w, const void* x16, size_t t, void* y, int y_dtype, GemmPlan** out, char* err,
                                size_t errlen, size_t experts, const int* tile_expert, int force_m_halves, size_t a_lo_row0, int w_terms,
                                const GemmPeerY* peer_y) {
    EncodeTiledFn enc = encode_tiled_fn();
    const bool gathered = peer_y && peer_y->ld != 0;
    if (gathered && (y_dtype != B2_F32 || experts != 1 || tile_expert || peer_y->n_more < 0 || peer_y->n_more > 7 || peer_y->ld < w.n_out ||
                     peer_y->ld % 4 || w.n_out % 4 || ((uintptr_t)y & 15))) {
        snprintf(err, errlen, "a gathered product needs a dense f32 result with 16-byte aligned column blocks");
        return cudaErrorInvalidValue;
    }

    if (!enc) {
        snprintf(err, errlen, "cuTensorMapEncodeTiled is not available from the driver");
        return cudaErrorNotSupported;
    }
    GemmPlan* p = new GemmPlan();
    p->x16 = x16;
    p->wptr = w.p0;
    p->y = y;
    p->y_dtype = y_dtype;
    p->t = t;
    p->K = w.n_in;
    p->n_out = w.n_out;
    p->experts = experts;
    p->tile_expert = tile_expert;
    p->m_halves = force_m_halves ? force_m_halves : (t > 128 ? 2 : 1);
    p->a_lo_row0 = a_lo_row0;
    if (a_lo_row0 && (p->m_halves != 1 || a_lo_row0 % 128 || a_lo_row0 < t)) {
        snprintf(err, errlen, "two-term activations need 128-token tiles and the lo rows on a 128-row boundary behind the hi rows");
        delete p;
        return cudaErrorInvalidValue;
    }
    int tm = 128 * p->m_halves;
    p->m_tiles = (int)((t + tm - 1) / tm);
    int sm_count = 148;
    int dev = 0;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev);
    if (w_terms == 2 && w.fmt != B2_FMT_Q4_K) w_terms = 1;  // the other formats' weights round to f16 far below the bound
    p->w_terms = w_terms;
    // (a gathered product stores every tile through the copy engine, whose staging tiles are 32 columns wide)
    const bool new_fmt = w.fmt == B2_FMT_Q6_K || w.fmt == B2_FMT_Q8_0;
    if (new_fmt && (experts != 1 || tile_expert || a_lo_row0 || w_terms == 2)) {
        snprintf(err, errlen, "Q6_K / Q8_0 products are dense, with one-term operands");
        delete p;
        return cudaErrorInvalidValue;
    }
    // (a Q6_K row brings 192 packed bytes per super-block against Q4_K's 144: narrower tiles fit the same staging buffer)
    const int widest = w.fmt == B2_FMT_Q6_K ? (gathered ? 192 : Q6K_MAX_TILE_N) : (gathered ? 224 : MAX_TILE_N);
    p->tile_n = pick_tile_n(w.n_out, p->m_tiles, sm_count, w.n_in, w_terms == 2 ? (gathered ? 96 : 112) : widest, gathered ? 32 : 16);
    // K in two halves (B2_GEMM_SPLIT_K=2; off by default because a row's bits then depend on whether its launch was
    // split, and row shards must equal the unsharded rows): a CTA's time goes with its number of k stages and hardly
    // with its width, so a grid that fills half the SMs or less runs nearly twice as fast as twice as many CTAs of half
    // the depth. Two shares only: their sum does not depend on the order the two reductions land in. f32 output, dense.
    {
        const int want = split_k_asked();
        p->split_asked = want;
        const int sb_k = w.fmt == B2_FMT_F8E4M3 ? 128 : 256;
        const size_t nsb_all = w.n_in / sb_k;
        if (want == 2 && !new_fmt && y_dtype == B2_F32 && !a_lo_row0 && w_terms == 1 && !tile_expert && !gathered && nsb_all % 2 == 0 && nsb_all >= 8) {
            const int tn2 = pick_tile_n(w.n_out, p->m_tiles * 2, sm_count, w.n_in / 2);
            const size_t tiles1 = (w.n_out + p->tile_n - 1) / p->tile_n * (size_t)p->m_tiles;
            const size_t tiles2 = (w.n_out + tn2 - 1) / tn2 * (size_t)p->m_tiles * 2;
            const size_t waves1 = (tiles1 + sm_count - 1) / sm_count, waves2 = (tiles2 + sm_count - 1) / sm_count;
            if (waves2 <= waves1) {  // the split grid is no deeper in waves: half the stages per CTA
                p->k_splits = 2;
                p->tile_n = tn2;
            }
        }
    }
    // The CTA-pair form: dense one-term 4-bit launches of more than one 256-token tile. The token tiles are rounded up to an
    // even count (a CTA whose tokens are all out of range multiplies zeros and stores nothing).
    p->pair_asked = pair_form_enabled();
    p->pair = p->pair_asked && !gathered && (w.fmt == B2_FMT_Q4_K || w.fmt == B2_FMT_MLX4) && !tile_expert && experts == 1 && !a_lo_row0 && w_terms == 1 &&
              p->k_splits == 1 && p->m_halves == 2 && p->m_tiles >= 2;
    if (p->pair) {
        p->m_tiles = (p->m_tiles + 1) / 2 * 2;
        p->tile_n = pick_tile_n(w.n_out, p->m_tiles, sm_count, w.n_in, PAIR_MAX_TILE_N);
    }
    p->n_tiles = (int)((w.n_out + p->tile_n - 1) / p->tile_n);
    {
        cuuint64_t dims[2] = {(cuuint64_t)w.n_in, (cuuint64_t)(a_lo_row0 ? a_lo_row0 + t : t)};
        cuuint64_t strides[1] = {(cuuint64_t)w.n_in * 2};
        cuuint32_t box[2] = {(cuuint32_t)STAGE_K, (cuuint32_t)tm};
        cuuint32_t estr[2] = {1, 1};
        CUresult r = enc(&p->tmap_x, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, (void*)x16, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                         CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) {
            snprintf(err, errlen, "cuTensorMapEncodeTiled(x) failed with CUresult %d", (int)r);
            delete p;
            return cudaErrorInvalidValue;
        }
    }
    {
        // the packed weights as a byte matrix [n_out][row_bytes]; one box = one super-block column of the tile
        const bool f8 = w.fmt == B2_FMT_F8E4M3 || new_fmt;  // rows of bytes, 128 per copy, swizzled
        size_t row_bytes = w.fmt == B2_FMT_Q6_K ? w.n_in / 2 : f8 ? w.n_in : w.n_in / 256 * 144;
        cuuint64_t dims[2] = {(cuuint64_t)row_bytes, (cuuint64_t)(w.n_out * experts)};
        cuuint64_t strides[1] = {(cuuint64_t)row_bytes};
        cuuint32_t box[2] = {f8 ? 128u : 144u, (cuuint32_t)(p->pair ? p->tile_n / 2 : p->tile_n)};
        cuuint32_t estr[2] = {1, 1};
        CUresult r = enc(&p->tmap_w, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, (void*)w.p0, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                         f8 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) {
            snprintf(err, errlen, "cuTensorMapEncodeTiled(w) failed with CUresult %d", (int)r);
            delete p;
            return cudaErrorInvalidValue;
        }
    }
    p->tmap_y = p->tmap_x;  // placeholder when the epilogue stores directly (bf16 output)
    p->y_direct = y_dtype == B2_F32 && !gathered && (w.n_out % 4 != 0 || ((uintptr_t)y & 15) != 0);
    if (y_dtype == B2_F32 && !p->y_direct) {
        // the f32 output [t][n_out] (a gathered product: this shard's n_out columns of rows `ld` apart); one box = a warp's
        // 32 tokens x 32 columns staging tile
        const size_t ld = gathered ? peer_y->ld : w.n_out;
        cuuint64_t dims[2] = {(cuuint64_t)w.n_out, (cuuint64_t)t};
        cuuint64_t strides[1] = {(cuuint64_t)ld * 4};
        cuuint32_t box[2] = {32, 32};
        cuuint32_t estr[2] = {1, 1};
        CUresult r = enc(&p->tmap_y, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, y, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                         CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) {
            snprintf(err, errlen, "cuTensorMapEncodeTiled(y) failed with CUresult %d", (int)r);
            delete p;
            return cudaErrorInvalidValue;
        }
        if (gathered && peer_y->n_more > 0) {
            CUtensorMap maps[8];
            for (int d = 0; d < peer_y->n_more; d++) {
                if (((uintptr_t)peer_y->more[d] & 15) != 0) r = CUDA_ERROR_INVALID_VALUE;
                if (r == CUDA_SUCCESS)
                    r = enc(&maps[d], CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, peer_y->more[d], dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
                p->more_ptr[d] = peer_y->more[d];
            }
            const int extra = w.fmt == B2_FMT_Q6_K ? 1 : 0;  // the qh plane's map goes behind the peers'
            if (extra && r == CUDA_SUCCESS) r = encode_q6k_qh(enc, &maps[peer_y->n_more], w, p->tile_n);
            cudaError_t ce = r == CUDA_SUCCESS ? cudaMalloc((void**)&p->y_more, sizeof(CUtensorMap) * (peer_y->n_more + extra)) : cudaErrorInvalidValue;
            if (ce == cudaSuccess) ce = cudaMemcpy(p->y_more, maps, sizeof(CUtensorMap) * (peer_y->n_more + extra), cudaMemcpyHostToDevice);
            if (ce != cudaSuccess) {
                snprintf(err, errlen, "tensor maps of the peers' y could not be made (CUresult %d, %s)", (int)r, cudaGetErrorString(ce));
                if (p->y_more) cudaFree(p->y_more);
                delete p;
                return cudaErrorInvalidValue;
            }
            p->n_more = peer_y->n_more;
        }
        p->y_ld = gathered ? ld : 0;
    }
    if (w.fmt == B2_FMT_Q6_K && !p->y_more) {  // the second weight plane's tensor map, read from global memory by the kernel
        CUtensorMap m;
        CUresult r = encode_q6k_qh(enc, &m, w, p->tile_n);
        cudaError_t ce = r == CUDA_SUCCESS ? cudaMalloc((void**)&p->y_more, sizeof(CUtensorMap)) : cudaErrorInvalidValue;
        if (ce == cudaSuccess) ce = cudaMemcpy(p->y_more, &m, sizeof m, cudaMemcpyHostToDevice);
        if (ce != cudaSuccess) {
            snprintf(err, errlen, "the tensor map of the Q6_K high-bit plane could not be made (CUresult %d, %s)", (int)r, cudaGetErrorString(ce));
            if (p->y_more) cudaFree(p->y_more);
            delete p;
            return cudaErrorInvalidValue;
        }
    }
    *out = p;
    return cudaSuccess;
}

void gemm_tc_plan_destroy(GemmPlan* p) {
    if (p && p->y_more) cudaFree(p->y_more);
    delete p;
}

bool gemm_tc_plan_matches(const GemmPlan* p, const WeightDev& w, const void* x16, size_t t, const void* y, int y_dtype, size_t a_lo_row0,
                          int w_terms, int m_halves, const GemmPeerY* peer_y) {
    if (w_terms == 2 && w.fmt != B2_FMT_Q4_K) w_terms = 1;
    if (p) {  // the same destinations
        const size_t ld = peer_y ? peer_y->ld : 0;
        const int nm = peer_y && peer_y->ld ? peer_y->n_more : 0;
        if (p->y_ld != ld || p->n_more != nm) return false;
        for (int d = 0; d < nm; d++)
            if (p->more_ptr[d] != peer_y->more[d]) return false;
    }
    return p && p->experts == 1 && p->a_lo_row0 == a_lo_row0 && p->w_terms == w_terms && (m_halves == 0 || p->m_halves == m_halves) && p->y == y && p->y_dtype == y_dtype && p->x16 == x16 && p->wptr == w.p0 && p->t == t && p->K == w.n_in && p->n_out == w.n_out &&
           p->split_asked == split_k_asked() && p->pair_asked == pair_form_enabled();
}

cudaError_t launch_gemm_tc(GemmPlan* p, const WeightDev& w, size_t t, void* y, int y_dtype, GemmStatus* status_dev, int /*sm_count*/,
                           cudaStream_t st, const float* row_unscale) {
    const bool split = p->k_splits > 1;
    const bool tt = p->a_lo_row0 > 0 || p->w_terms == 2;
    using Kern = void (*)(CUtensorMap, CUtensorMap, CUtensorMap, int, int, int, int, int, void*, int, GemmStatus*, int, const int*, F8Scales, int, const float*,
                          int, int, const CUtensorMap*, int);
    Kern kern;
    if (tt)  // two-term operands never come with a K split
        kern = w.fmt == B2_FMT_MLX4 ? gemm_q4k_tc_kernel<B2_FMT_MLX4, false, true>
               : w.fmt == B2_FMT_F8E4M3 ? gemm_q4k_tc_kernel<B2_FMT_F8E4M3, false, true> : gemm_q4k_tc_kernel<B2_FMT_Q4_K, false, true>;
    else
        kern = w.fmt == B2_FMT_Q6_K     ? gemm_q4k_tc_kernel<B2_FMT_Q6_K, false, false>
               : w.fmt == B2_FMT_Q8_0   ? gemm_q4k_tc_kernel<B2_FMT_Q8_0, false, false>
               : w.fmt == B2_FMT_MLX4   ? (split ? gemm_q4k_tc_kernel<B2_FMT_MLX4, true, false> : gemm_q4k_tc_kernel<B2_FMT_MLX4, false, false>)
               : w.fmt == B2_FMT_F8E4M3 ? (split ? gemm_q4k_tc_kernel<B2_FMT_F8E4M3, true, false> : gemm_q4k_tc_kernel<B2_FMT_F8E4M3, false, false>)
                                        : (split ? gemm_q4k_tc_kernel<B2_FMT_Q4_K, true, false> : gemm_q4k_tc_kernel<B2_FMT_Q4_K, false, false>);
    F8Scales f8{w.fmt == B2_FMT_F8E4M3 ? (const float*)w.p1 : nullptr, nullptr, (int)w.bs_rows, (int)w.bs_ncb, (int)w.bs_row0, 256.0f};
    if (w.fmt == B2_FMT_Q8_0) f8 = F8Scales{(const float*)w.p1, nullptr, 1, (int)(w.n_in / 32), 0, 256.0f};
    if (w.fmt == B2_FMT_Q6_K) f8 = F8Scales{(const float*)w.p2, (const void*)w.p3, 1, 0, 0, 256.0f};
    if (p->pair) {
        kern = w.fmt == B2_FMT_MLX4 ? gemm_q4k_tc_kernel<B2_FMT_MLX4, false, false, true> : gemm_q4k_tc_kernel<B2_FMT_Q4_K, false, false, true>;
        if (cudaError_t e = ensure_dynamic_smem((const void*)kern, PAIR_SMEM); e != cudaSuccess) return e;
        cudaLaunchConfig_t cfg{};
        cfg.gridDim = dim3((unsigned)p->m_tiles, (unsigned)p->n_tiles, 1);
        cfg.blockDim = dim3(GEMM_THREADS);
        cfg.dynamicSmemBytes = PAIR_SMEM;
        cfg.stream = st;
        cudaLaunchAttribute attr[2] = {};
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 2;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[1].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 2;
        cudaError_t le = cudaLaunchKernelEx(&cfg, kern, p->tmap_x, p->tmap_w, p->tmap_y, (int)w.n_in, (int)w.n_out, (int)t, p->tile_n, p->m_halves, y,
                                  y_dtype | (p->y_direct ? 0x100 : 0), status_dev, debug_switches(), (const int*)nullptr, f8, 1, row_unscale, 0, 1, (const CUtensorMap*)nullptr, 0);
        return le;
    }
    if (cudaError_t e = ensure_dynamic_smem((const void*)kern, GEMM_SMEM); e != cudaSuccess) return e;
    dim3 grid((unsigned)p->n_tiles, (unsigned)p->m_tiles, (unsigned)p->k_splits);
    if (p->k_splits > 1) {  // the shares are added into y
        cudaError_t e = cudaMemsetAsync(y, 0, t * w.n_out * sizeof(float), st);
        if (e != cudaSuccess) return e;
    }
    // (a dependent launch: see the top of the kernel)
    return launch_k(kern, grid, dim3(GEMM_THREADS), GEMM_SMEM, st, true, p->tmap_x, p->tmap_w, p->tmap_y, (int)w.n_in, (int)w.n_out, (int)t, p->tile_n, p->m_halves, y,
                    y_dtype | (p->y_direct ? 0x100 : 0), status_dev, debug_switches(), p->tile_expert, f8, p->k_splits, row_unscale, (int)p->a_lo_row0, p->w_terms,
                    (const CUtensorMap*)p->y_more, p->n_more);
}

cudaError_t launch_to_f16(const void* x, int x_dtype, size_t t, size_t K, void* x16, float* unscale, cudaStream_t st, size_t lo_row0, size_t x_ld) {
    if (t == 0 || K % 2) return cudaErrorInvalidValue;
    const size_t lo_off = lo_row0 * K;
    if (x_ld == 0) x_ld = K;
    if (x_dtype == B2_F32)
        return launch_k(to_f16_rows_kernel<float>, dim3((unsigned)t), dim3(256), 0, st, true, (const float*)x, (int)K, (__half*)x16, unscale, lo_off, x_ld);
    else if (x_dtype == B2_BF16)
        return launch_k(to_f16_rows_kernel<__nv_bfloat16>, dim3((unsigned)t), dim3(256), 0, st, true, (const __nv_bfloat16*)x, (int)K, (__half*)x16, unscale, lo_off, x_ld);
    else if (x_dtype == B2_F16)
        return launch_k(to_f16_rows_kernel<__half>, dim3((unsigned)t), dim3(256), 0, st, true, (const __half*)x, (int)K, (__half*)x16, unscale, lo_off, x_ld);
    else
        return cudaErrorInvalidValue;
    return cudaGetLastError();
}

}  // namespace b2
