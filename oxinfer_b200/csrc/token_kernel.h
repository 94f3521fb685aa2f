// The persistent token kernel: one cooperative launch runs whole decode tokens. Every SM holds one CTA of 768
// threads for the length of the launch; the token's ops are a program in device memory that all CTAs walk in step,
// separated by grid barriers where one op reads what another wrote. What a kernel boundary costs in the
// one-launch-per-op form (launch, ramp-up, staging, tail: 4-5 us) becomes a barrier (about 1.5 us), and the vector a
// matrix-vector product reads is normalized and split into its integer planes by every CTA for itself in shared
// memory, so the norm and plane kernels and their round trips through global memory disappear.
#pragma once
#include "kernels.h"

namespace b2 {

enum : uint32_t {
    TK_NORM_STAGE = 1,  // RMSNorm of x (one row) -> planes in shared memory (every CTA); CTA 0 also writes the row to y
    TK_STAGE = 2,       // planes of the vector x -> shared memory (every CTA)
    TK_GEMV = 3,        // rows of w (and w2) against the staged planes, rows spread over all warps of the grid
    TK_ROPE = 4,        // heads spread over the CTAs
    TK_ATTEND = 5,      // (KV head, key split) units spread over the 256-thread groups of all CTAs
    TK_GLU = 6,
    TK_BARRIER = 7,
    TK_XPLANES = 8,     // planes of the vector x -> global memory (xp), blocks spread over all warps of the grid
    TK_COPY = 9,        // planes in global memory (xp) -> shared memory (every CTA)
};

struct TokOp {
    uint32_t kind;
    uint32_t mode;   // GEMV: B2_MODE_*
    uint32_t pair;   // GEMV: w2 is the second matrix of a pair mode
    uint32_t n;      // STAGE / GLU: length
    uint32_t gelu;
    uint32_t kv_f16;
    const float* x;
    float* y;
    const float* z;
    const float* p0;  // norm weights | q norm
    const float* p1;  // k norm
    void* kc;
    void* vc;
    WeightDev w, w2;
    DecNorm norm;
    DecRope rope;
    DecAttn attn;
    XPlanes xp;       // XPLANES / ATTEND write them, COPY reads them
};

struct TokenArgs {
    const TokOp* prog;
    uint32_t n_ops;
    uint32_t n_tokens;
    uint32_t pos0;        // position of the first token
    uint32_t table_pos0;  // position of row 0 of the RoPE table
    uint32_t with_head;   // 1: embedding lookup before and argmax after every token (greedy loop); 0: the ops once
    uint32_t n_logits;
    uint32_t max_splits;  // attention: splits per KV head at most
    uint32_t first_token;
    uint32_t ring_slots;  // slots of each warp's weight ring (2 .. 4)
    uint32_t ring_offset; // where the rings start in the work area (behind the planes)
    const float* cs_table;
    float* input;         // the token's embedding goes here
    const float* logits;
    float* part;          // attention partials
    uint32_t* att_counters;
    uint32_t* ctl;        // [0] barrier arrivals, [1] abort, [2] status (0 ok, 1 attention copy wait, 2 barrier wait)
    float* argmax_val;    // one per CTA
    int* argmax_idx;
    int* token;           // the last token chosen
    int* out_tokens;
    WeightDev embed;
    unsigned long long* prof;  // optional (diagnostics): cycles CTA 0 spent per op kind [16], and how many ops [16]
};

// Shared memory the kernel needs for planes of up to max_k values and attention with (hd, heads per KV head, cache type).
size_t token_kernel_smem(size_t max_k, uint32_t hd, uint32_t g, int kv_f16);
// The rings of the 4-bit products: where they start behind planes of max_k values, and their size for `slots` slots per warp.
size_t token_kernel_ring_offset(size_t max_k);
size_t token_kernel_ring_bytes(uint32_t slots);
size_t token_kernel_fixed_bytes();
// Whether the kernel takes this attention shape (head dim 64 / 128, 1 / 2 / 4 heads per KV head).
bool token_kernel_attend_ok(uint32_t nh, uint32_t nkv, uint32_t hd);
// The largest norm row the kernel keeps in registers.
constexpr uint32_t TOKEN_KERNEL_MAX_NORM = 768 * 8;  // two runs of four values per thread
// Cooperative launch on `st` with one CTA per SM. `ctl` must be zeroed (stream-ordered) before each launch.
cudaError_t launch_token_kernel(const TokenArgs& args, size_t smem, int sm_count, cudaStream_t st);

}  // namespace b2
