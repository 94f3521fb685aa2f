// Host-callable launchers of the CUDA kernels (one translation unit per kernel family).
#pragma once
#include <map>
#include <mutex>
#include <utility>

#include "formats.cuh"

namespace b2 {

// A kernel that wants more dynamic shared memory than the default must be told so with cudaFuncSetAttribute, and that
// setting belongs to the (kernel, device) pair: a process may hold contexts on several GPUs (b2_open per ordinal), and
// each of them needs its own call. Remembers the largest size asked so far per pair, so that the common launch costs a
// map lookup. `dflt`: what the kernel may use without asking (less than 48 KB where it also has static shared memory).
inline cudaError_t ensure_dynamic_smem(const void* kern, size_t bytes, size_t dflt = 48 * 1024) {
    if (bytes <= dflt) return cudaSuccess;
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    static std::mutex mu;
    static std::map<std::pair<const void*, int>, size_t> asked;
    std::lock_guard<std::mutex> lock(mu);
    size_t& cur = asked[std::make_pair(kern, dev)];
    if (bytes <= cur) return cudaSuccess;
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
    if (e == cudaSuccess) cur = bytes;
    return e;
}

// Launch with or without the programmatic-dependent-launch attribute. With it the kernel may begin while the
// kernel ahead of it in the stream is still running; every kernel launched this way calls pdl_wait() (xplanes.cuh)
// before it reads what that kernel wrote or writes anything.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_k(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, bool pdl, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kern, KArgs(args)...);
}

// ---- dq.cu: bit-exact dequantization --------------------------------------------------------
// Rows [r0, r0 + nrows) of `w` to f32, row-major [nrows][n_in]. With `row_dev`, r0 is read from that
// device word when the kernel runs (a token's embedding row inside a captured graph).
cudaError_t launch_dequantize(const WeightDev& w, size_t r0, size_t nrows, float* out, cudaStream_t st, const int* row_dev = nullptr,
                              bool pdl = false);
// Raw GGUF Q6_K / Q8_0 rows (device) -> the split planes described in formats.cuh.
cudaError_t launch_repack_q6k(const uint8_t* raw, size_t n_out, size_t n_in, uint8_t* ql, uint8_t* qh, int8_t* sc, uint16_t* d,
                              cudaStream_t st);
cudaError_t launch_repack_mlx4(const uint32_t* w, const uint16_t* scales, const uint16_t* biases, size_t n_out, size_t n_in, uint8_t* out,
                               cudaStream_t st);
// Q4Matrix with offsets (q in Q4_0 order, f16 scale per 32, bf16 offset per `group`, a multiple of 64) -> the same blocks
// launch_repack_mlx4 makes; *mismatch (device, zeroed by the caller) is set if a 64-group's two scales differ.
cudaError_t launch_repack_q4a(const uint8_t* q, const uint16_t* scales, const uint16_t* offsets, size_t n_out, size_t n_in, size_t group,
                              uint8_t* out, int* mismatch, cudaStream_t st);
cudaError_t launch_repack_q8_0(const uint8_t* raw, size_t n_out, size_t n_in, int8_t* qs, uint16_t* d, cudaStream_t st);

// ---- gemv.cu: one-token dequant matrix-vector products ---------------------------------------
// Activation vector split into three int8 planes per block of 32 (x ~= xs * (q0 + 32 q1 + 8192 q2),
// 21 significant bits per block; q1 and q2 alone carry 16), plus block scales and sums. The record in global memory is the image the product
// kernels keep in shared memory, so staging it is a plain copy (bulk copies in the ring form). For n_in = K, in bytes:
//   planes 3K | sx 8K/32 | v16 4K/16
// Element k of plane p sits at p * K + 16 * xplanes_slot(k / 16) + k % 16: the 16-byte slots of each 64 bytes are
// permuted so that the product kernels' shared-memory reads spread over the banks.
struct XPlanes {
    int8_t* planes;   // [3][K], slots permuted
    float2* sx;       // [K/32]  (block scale, scale * sum of the block's integers = the quantized block sum)
    int32_t* v16;     // [K/16]  integer sums of each 16 elements
    int np;           // planes a product reads: 2 = the upper two (16 bits), anything else = all three (21 bits, the default)
};
// Slot g -> g with its low two bits xor-ed by bits 3 and 4: lanes L = 0..7 of a phase that read slots 4 L + i (a 64-byte
// stride) then cover all eight 16-byte bank groups for every i.
__host__ __device__ inline int xplanes_slot(int g) { return g ^ ((((g >> 3) & 1) << 1) | ((g >> 4) & 1)); }
__host__ __device__ inline size_t xplanes_bytes(size_t K) { return 3 * K + 4 * (K / 32) * 2 + 4 * (K / 16); }
__host__ __device__ inline XPlanes xplanes_at(void* base, size_t K) {
    XPlanes p;
    uint8_t* b = (uint8_t*)base;
    p.planes = (int8_t*)b;
    p.sx = (float2*)(b + 3 * K);
    p.v16 = (int32_t*)(b + 3 * K + 8 * (K / 32));
    p.np = 0;
    return p;
}
// tokens > 1: token i's vector x_stride floats and its planes planes_stride bytes behind token 0's, one launch for all.
cudaError_t launch_xplanes(const float* x, size_t K, XPlanes out, cudaStream_t st, bool pdl = false, int tokens = 1, size_t x_stride = 0,
                           size_t planes_stride = 0);
// A vector whose RMS-norm factor is applied after the product instead of before the split: the planes hold the split of
// x * w (no factor), `partial` holds the sum of squares of every block of 32 of x, and the product kernel multiplies its
// sums by k = 1 / sqrt(sum(partial) * inv_n + eps). The split of a block does not depend on a common factor, so this
// equals the product over the normalized vector up to rounding; it lets the norm run as independent warps on many SMs
// instead of one CTA that must first reduce the whole row. partial == nullptr: no factor.
struct NormScale {
    const float* partial;
    uint32_t count;
    float inv_n, eps;
};
// planes(x * pre * w) and the blocks' sums of squares of x * pre; K a multiple of 32, w may be null.
// tokens > 1 as for launch_xplanes; token i's sums partial_stride floats behind token 0's.
cudaError_t launch_norm_planes(const float* x, const float* w, float pre, size_t K, XPlanes out, float* partial, cudaStream_t st, bool pdl = false,
                               int tokens = 1, size_t x_stride = 0, size_t planes_stride = 0, size_t partial_stride = 0);
// What a product may do with its finished output, so that the kernel which would split it for the next product is not
// launched: the CTAs then own whole blocks of 32 consecutive rows (four per warp), the warps leave their results in
// shared memory, and after a CTA barrier one warp writes the planes of y * pre * w (w may be null) and, with `partial`,
// the block's sum of squares of y * pre: what launch_xplanes / launch_norm_planes would have written, bit for bit.
// n_out must be a multiple of 32. out.planes == nullptr: nothing.
struct EpiPlanes {
    XPlanes out;
    const float* w;
    float* partial;
    float pre;
};
// Whether launch_gemv takes an EpiPlanes for this matrix (the 4-bit formats whose planes and rings fit in shared memory).
bool gemv_takes_epilogue(const WeightDev& w);
// y[n_out] = mode(W x [, U x]). `xp` holds the planes of x (launch_xplanes); the
// FP8 kernel reads `x` (f32) directly and ignores `xp`. plain_form: never the ring form (a lone product behind its own plane
// kernel: launched as that kernel's dependent, the register-load form fetches its first weights while the planes are made).
cudaError_t launch_gemv(const WeightDev& w, const WeightDev* up, const float* x, XPlanes xp, float* y, int mode, const float* gate,
                        int sm_count, cudaStream_t st, bool pdl = false, NormScale ns = NormScale{nullptr, 0, 0.0f, 0.0f},
                        EpiPlanes epi = EpiPlanes{XPlanes{nullptr, nullptr, nullptr}, nullptr, nullptr, 1.0f},
                        bool plain_form = false);
// A batch of products in one launch (the routed experts of a few tokens): entry b multiplies matrix expert[b] of a stack
// of equally shaped 4-bit matrices (w describes matrix 0; w_stride bytes apart) by the planes block xrow[b] (x_stride
// bytes apart, laid out as xplanes_at) into y + b * y_stride. The tables travel as kernel arguments (up to 64 entries),
// so a call needs no copy of its own and no synchronization.
constexpr int GEMV_BATCH_MAX = 64;
struct GemvBatch {
    int n;  // 0: not a batch
    int expert[GEMV_BATCH_MAX];
    int xrow[GEMV_BATCH_MAX];
    size_t w_stride, x_stride, y_stride;
    uint8_t* planes;
};
cudaError_t launch_gemv_batched(const WeightDev& w, const WeightDev* up, const GemvBatch& b, size_t batch, float* y, int mode, int np, int sm_count,
                                cudaStream_t st, bool pdl = false);
// Planes of `rows` vectors of K values (row r at x + r * K) into blocks `stride` bytes apart.
cudaError_t launch_xplanes_rows(const float* x, size_t rows, size_t K, uint8_t* planes, size_t stride, cudaStream_t st, bool pdl = false);
// nt (1..4) tokens in one launch, the weights read once: token i's f32 vector at x + i * x_stride (FP8 weights) or planes
// at xp + i * xp_stride bytes (the other formats), outputs at y + i * y_stride. Each token's result equals its
// single-token result bit for bit. cudaErrorInvalidValue if the tokens' vectors do not fit in shared memory together, or for
// the gated mode. `ns`: token 0's deferred norm factor (see NormScale), token i's partial sums ns_stride floats further.
cudaError_t launch_gemv_multi(const WeightDev& w, const WeightDev* up, const float* x, size_t x_stride, XPlanes xp, size_t xp_stride, float* y,
                              size_t y_stride, int nt, int mode, int sm_count, cudaStream_t st, bool pdl = false,
                              NormScale ns = NormScale{nullptr, 0, 0.0f, 0.0f}, size_t ns_stride = 0);
// Whether launch_gemv handles this format and shape.
bool gemv_supports(const WeightDev& w);

// ---- gemv_other.cu: the other GGUF block formats (dq_other.cuh), raw rows, one generic kernel ---------------------------
bool gemv_other_supports(const WeightDev& w);
cudaError_t launch_dequantize_other(const WeightDev& w, size_t r0, size_t nrows, float* out, cudaStream_t st, const int* row_dev = nullptr,
                                    bool pdl = false);
// nt (1..4) tokens: token i's f32 vector at x + i * x_stride, its outputs at y + i * y_stride; the five output modes and the pair.
cudaError_t launch_gemv_other(const WeightDev& w, const WeightDev* up, const float* x, size_t x_stride, float* y, size_t y_stride, int nt, int mode,
                              const float* gate, int sm_count, cudaStream_t st, bool pdl = false);

// ---- gemm_tc.cu: prefill dequant-GEMM on tcgen05 ------------------------------------------------
struct GemmStatus {   // written by the kernel when a bounded wait gives up
    uint32_t code;    // 0 = ok
    uint32_t where;   // which wait
    uint32_t cta;
    uint32_t iter;
    uint32_t t[8];    // cycle stamps of one CTA (diagnostics, B2_GEMM_DEBUG & 32768)
};
bool gemm_tc_supports(const WeightDev& w, size_t t);
// y[t][n_out] (f32 or bf16) = x[t][n_in] (f16, row-major, t padded by the caller to a multiple of
// 256 rows in `x16`) * W^T. `tmap_x` is the host-encoded tensor map of x16 (see make_tmap_x).
struct GemmPlan;
// a_lo_row0 > 0 (128-token tiles only): x16 holds two-term activations, the lo rows a_lo_row0 rows below the hi rows; both
// terms feed the same accumulator, so the activations enter with 22 significant bits.
// w_terms == 2 (Q4_K only; other formats ignore it): every weight enters as two f16 terms, hi + lo = the reference's f32
// value to about 22 bits; tiles are then at most 112 rows wide.
// `experts` > 1 makes a grouped plan: w.p0 holds `experts` stacked matrices of w.n_out rows, x16 / y hold the
// token rows of all experts in segments that are multiples of 128 * m_halves rows, and tile_expert[i]
// (device) names the expert of token tile i.
// Where a row-sharded product's f32 result goes when every rank is to end up with the whole y [t][ld]: this rank's columns
// of its own y (`y` of the call, already offset to them) and of n_more peers' copies (device pointers mapped from the
// peers, offset the same way). The GEMM's epilogue then issues each staging tile's bulk store once per destination, so the
// all-gather happens tile by tile from the kernel that computes the tiles.
struct GemmPeerY {
    size_t ld = 0;        // row stride of the destinations in elements (0: not a gathered product, the stride is n_out)
    int n_more = 0;       // peers' destinations
    float* more[7] = {};
};
cudaError_t gemm_tc_plan_create(const WeightDev& w, const void* x16, size_t t, void* y, int y_dtype, GemmPlan** out, char* err,
                                size_t errlen, size_t experts = 1, const int* tile_expert = nullptr, int force_m_halves = 0, size_t a_lo_row0 = 0, int w_terms = 1, const GemmPeerY* peer_y = nullptr);
void gemm_tc_plan_destroy(GemmPlan* p);
bool gemm_tc_plan_matches(const GemmPlan* p, const WeightDev& w, const void* x16, size_t t, const void* y, int y_dtype, size_t a_lo_row0 = 0,
                          int w_terms = 1, int m_halves = 0, const GemmPeerY* peer_y = nullptr);
// row_unscale (device, [t], may be null): factor the epilogue multiplies token row i's results by (launch_to_f16).
cudaError_t launch_gemm_tc(GemmPlan* p, const WeightDev& w, size_t t, void* y, int y_dtype, GemmStatus* status_dev, int sm_count,
                           cudaStream_t st, const float* row_unscale = nullptr);
// x (f32 / bf16 / f16, [t][K]) -> f16 [t][K], every row multiplied by a power of two that brings its largest magnitude
// into [2^14, 2^15) (no overflow, no subnormals, same relative rounding at every magnitude); unscale[row] = 1 / factor.
// lo_row0 > 0: two-term activations, x * factor = hi + lo; the lo rows go lo_row0 rows below the hi rows of x16.
// x_ld: elements between the rows of x (0: K, the rows are contiguous).
cudaError_t launch_to_f16(const void* x, int x_dtype, size_t t, size_t K, void* x16, float* unscale, cudaStream_t st, size_t lo_row0 = 0,
                          size_t x_ld = 0);
// Whether nt (1..4) token rows' vectors fit in shared memory together for launch_gemv_multi.
bool gemv_multi_fits(const WeightDev& w, int nt);
// Whether one launch for nt tokens beats nt one-token launches inside a chain of dependent launches: from two tokens on
// for the 4-bit formats (integer dots on the tensor cores), from three for the others (their several-token kernel does a
// token's arithmetic per token and is not the bulk-copy form).
bool gemv_multi_pays(const WeightDev& w, int nt);

// ---- gemm_f8.cu: FP8 weights x FP8 activations (tcgen05 kind::f8f6f4), 128 x 128 weight scale blocks, activations quantized
// per token and per 128 k -----------------------------------------------------------------------------------------------
bool gemm_f8_supports(const WeightDev& w, size_t t);
// Bytes of scratch for t rows of K: the e4m3 activations [t][K], then (256-byte aligned) their scales f32 [t][K / 128].
size_t gemm_f8_scratch_bytes(size_t t, size_t K);
// x (f32 / bf16 / f16, [t][K]) -> q e4m3 [t][K] and sx f32 [t][K / 128]: scale = amax / 448 per block of 128 (1 for a zero
// block), q = RNE(x / scale) saturating at +-448.
cudaError_t launch_quantize_act_e4m3(const void* x, int x_dtype, size_t t, size_t K, uint8_t* q, float* sx, cudaStream_t st);
// y[t][n_out] (f32 or bf16) = sum over 128-k blocks of sx * sw * (qx . qw).
cudaError_t launch_gemm_f8(const WeightDev& w, const uint8_t* qx, const float* sx, size_t t, void* y, int y_dtype, GemmStatus* status_dev,
                           cudaStream_t st, char* err, size_t errlen);

// ---- moe.cu: the element-wise pieces of the routed-expert layer ------------------------------------
cudaError_t launch_route_topk(const float* logits, size_t t, size_t n, size_t k, int* ids, float* w, cudaStream_t st);
// Rows to f16 operands for the grouped GEMM, each multiplied by a power of two (its largest magnitude into [2^14, 2^15));
// unscale[row] = 1 / factor is handed to the GEMM, whose epilogue multiplies the row's results by it. lo_row0 > 0: two-term
// rows, the second term lo_row0 rows below the first (see launch_to_f16).
cudaError_t launch_moe_gather(const float* x, const int* src, size_t rows, size_t h, void* xg_f16, float* unscale, size_t lo_row0, cudaStream_t st);
// kind: B2_ACT_* (0 SiLU, 1 tanh GELU, 2 SiLU with clamp `limit`).
cudaError_t launch_moe_act(const float* g, const int* src, size_t rows, size_t inter, void* a_f16, float* unscale, size_t lo_row0, cudaStream_t st,
                           int kind = 0, float limit = 0.0f);
// The same with the routes as kernel arguments (at most GEMV_BATCH_MAX pairs): slot of pair (i, j) = i k + j, no row scale.
struct SmallRoutes {
    float w[GEMV_BATCH_MAX];
};
cudaError_t launch_moe_combine_small(const float* o, const SmallRoutes& r, size_t t, size_t k, size_t h, float* y, cudaStream_t st, bool pdl = false);
cudaError_t launch_moe_combine(const float* o, const int* slots, const float* w, size_t t, size_t k, size_t h, float* y, cudaStream_t st);

// out[r][h] = x[idx[r]][h] (f32), h a multiple of 4; and an all-gather's rank-major blocks g [world][t][n_local] into the
// column blocks of y [t][world * n_local] (the tensor- and expert-parallel entry points).
cudaError_t launch_gather_rows(const float* x, const int* idx, size_t rows, size_t h, float* out, cudaStream_t st);
cudaError_t launch_scatter_blocks(const float* gathered, size_t world, size_t t, size_t n_local, float* y, cudaStream_t st);

// ---- decode_ops.cu: the non-matmul ops of one decode token -------------------------------------------
// Every kernel reads the step words `sp` on the device: sp[0] position of the token, sp[1] position of row 0
// of the RoPE table, sp[2] tokens generated so far (the argmax kernel advances [0] and [2]).
struct DecNorm {
    uint32_t n, x_stride, out_stride, add, planes;
    float pre, eps;
};
struct DecRope {
    uint32_t nh, nkv, hd, half_rot, q_stride, k_off, v_off, interleaved, v_norm, v_from_k, max_len;
    uint32_t cs_stride, cs_off;  // floats per position in the RoPE table, and where this op's cos/sin start in a row
    float eps;
};
struct DecAttn {
    uint32_t nh, nkv, hd, max_len, window, planes;
    float scale;
};
// The ranks of a tensor-parallel plan as one rank sees them: every rank's activation block and flag words, mapped
// into this process (its own entries are its local pointers).
struct PeerSet {
    uint32_t rank, world;
    float* base[8];
    uint32_t* flags[8];  // [0] epoch counter, [8 + p] "rank p arrived", [16 + p] "rank p has written"
};
// All-gather of the n-value vector at `off_floats` inside the activation block (equal contiguous parts, rank order).
// meet_first: also meet before writing (needed when a kernel since the previous exchange reads other ranks' parts).
// wait_limit_cycles: how long a rank polls for its peers before it gives up and sets the status word (0: about half a second).
cudaError_t launch_exchange(const PeerSet& ps, size_t off_floats, uint32_t n, uint32_t* lflags, uint32_t* status, cudaStream_t st,
                            bool pdl = false, bool meet_first = true, long long wait_limit_cycles = 0);
cudaError_t launch_norm(const float* x, float* out, const float* w, const DecNorm& p, uint32_t rows, XPlanes xp, cudaStream_t st, bool pdl = false);
// KV caches are [nkv][max_len][hd], f32 or (kv_f16) f16.
cudaError_t launch_qk_rope(const float* qkv, float* qo, void* kc, void* vc, int kv_f16, const float* qn, const float* kn, const float* cs_table,
                           const uint32_t* sp, const DecRope& p, cudaStream_t st, bool pdl = false);
bool attend_supports(uint32_t nh, uint32_t nkv, uint32_t hd);
size_t attend_part_floats(uint32_t nh, uint32_t hd);  // scratch for the per-split partials
// Attention that prepares its own inputs: with qkv set, the kernel applies RoPE to the token's query heads as it stages
// them (`q` is not read), and the CTA whose keys end at the token's position rotates the token's key, appends key and value
// to the caches and puts them into its tile; the arithmetic of launch_qk_rope, which is then not launched. Per-head norms
// are not taken (r.* as for launch_qk_rope; qkv == nullptr: plain attention over q and the caches).
struct FusedRope {
    const float* qkv;
    const float* cs_table;
    DecRope r;
};
// Several tokens of a step in one launch (only without FusedRope: every token's key and value must be in the caches
// already): token i's queries / outputs act_stride floats behind token 0's, its planes planes_stride bytes, its partials
// part_stride floats, its counters nkv words, its step words 4 words.
struct AttnTokens {
    int n;  // 0 or 1: one token
    size_t act_stride, planes_stride, part_stride;
};
// counters: nkv zeroed words (left zero by every launch); status: set to 1 if a bounded wait gave up.
cudaError_t launch_attend(const float* q, void* kc, void* vc, int kv_f16, float* out, float* part, uint32_t* counters,
                          const uint32_t* sp, const DecAttn& p, XPlanes xp, uint32_t* status, cudaStream_t st, bool pdl = false,
                          const FusedRope* fr = nullptr, const AttnTokens* tokens = nullptr);
// Host-order rows [n][nkv][hd] f32 <-> cache rows pos0 .. pos0 + n - 1.
cudaError_t launch_kv_rows(float* rows, void* cache, int kv_f16, bool to_cache, uint32_t nkv, uint32_t hd, uint32_t max_len, uint32_t pos0,
                           uint32_t n, cudaStream_t st);
cudaError_t launch_set_step(uint32_t* sp, uint32_t pos, uint32_t table_pos0, uint32_t count, int* token, int tok, cudaStream_t st);
cudaError_t launch_glu(const float* g, const float* u, float* out, uint32_t n, int gelu, cudaStream_t st, bool pdl = false);
// pval / pidx: 128 words each; counter: one zeroed word.
cudaError_t launch_argmax(const float* logits, uint32_t n, float* pval, int* pidx, uint32_t* counter, int* token, int* out_tokens, uint32_t* sp,
                          cudaStream_t st, bool pdl = false);

// ---- prefill_ops.cu: the same ops over many token rows (row r of an activation `stride` floats behind row r - 1) -----------
// Token row r is at position sp[0] + r; sp[1] is the position of row 0 of the RoPE table.
cudaError_t launch_qk_rope_rows(const float* qkv, float* qo, size_t stride, uint32_t rows, void* kc, void* vc, int kv_f16, const float* qn,
                                const float* kn, const float* cs_table, const uint32_t* sp, const DecRope& p, cudaStream_t st);
bool attend_rows_supports(uint32_t nh, uint32_t nkv, uint32_t hd);
// Causal attention of `rows` query tokens over the cache (which already holds their keys and values): tensor-core products
// over f16 roundings of q, k, v and the probabilities, f32 sums. `len`: positions the cache holds now (sp[0] + rows, as the
// host knows it). f32 caches: `scratch` (attend_rows_scratch_bytes) receives an f16 copy of those rows first.
size_t attend_rows_scratch_bytes(uint32_t nkv, uint32_t max_len, uint32_t hd, int kv_f16);
cudaError_t launch_attend_rows(const float* q, float* out, size_t stride, uint32_t rows, const void* kc, const void* vc, int kv_f16, void* scratch,
                               uint32_t len, const uint32_t* sp, const DecAttn& p, cudaStream_t st);
// RMS norm of `rows` rows (p.n values each, p.pre / p.eps / p.add as for launch_norm; the strides here replace p's). With
// x16 / unscale the rows also leave as the f16 operands launch_to_f16 would make of the result (rows of p.n halves).
bool norm_rows_supports(uint32_t n, const float* x, const float* out, const float* w, size_t x_stride, size_t out_stride);
cudaError_t launch_norm_rows(const float* x, size_t x_stride, float* out, size_t out_stride, const float* w, const DecNorm& p, uint32_t rows,
                             void* x16, float* unscale, cudaStream_t st);
// With x16 / unscale (glu_rows_f16_supports(n)) the rows also leave as the f16 operands launch_to_f16 would make of the result.
bool glu_rows_f16_supports(uint32_t n);
cudaError_t launch_glu_rows(const float* g, size_t g_stride, const float* u, size_t u_stride, float* out, size_t out_stride, uint32_t n,
                            uint32_t rows, int gelu, cudaStream_t st, void* x16 = nullptr, float* unscale = nullptr);
// dst[r][i] (+)= src[r][i] for i < n (a multiple of 4; 16-byte aligned rows).
cudaError_t launch_rows_op(float* dst, size_t dst_stride, const float* src, size_t src_stride, uint32_t n, uint32_t rows, bool add,
                           cudaStream_t st);

}  // namespace b2
