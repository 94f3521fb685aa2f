// The decode plan: a token's op list (b2_graph) resolved to device pointers, captured into a CUDA graph,
// with the KV caches it owns. The role of CudaPlan in the reference (src/cuda_decode.rs:1233-1658).
#pragma once
#include <functional>
#include <map>
#include <string>
#include <vector>

#include "../../include/b200qmm.h"
#include "kernels.h"

namespace b2 {

class DecodePlanImpl {
  public:
    // `resolve` maps a weight handle to its device description (nullptr: unknown handle).
    // Returns B2_OK, B2_DECLINED or an error code; `err` gets the reason.
    // `planes`: how many planes of the activation split the plan's products read (2: the upper two, 16 bits; otherwise all three, 21 bits).
    // `tokens` (1..4): the most tokens of a step (Backend::decode_plan_multi, src/gpu.rs:273-276). A plan of several tokens keeps
    // one activation block, planes block and block of norm sums per token.
    // `prefill`: a prefill plan (Backend::decode_plan_prefill, src/gpu.rs:283-289): steps of up to `tokens` (1..8192) tokens on
    // batched kernels (tensor-core GEMMs for the products, tensor-core causal attention), whose results differ from one-token
    // steps in rounding. Such a plan takes no logits (the reference's prefill graph ends at the final norm).
    static int create(const b2_graph* g, const std::function<const WeightDev*(uint64_t)>& resolve, int sm_count, int planes, int tokens,
                      bool prefill, DecodePlanImpl** out, std::string& err);
    ~DecodePlanImpl();

    int step(cudaStream_t st, size_t pos, const float* x, const float* rope_cs, float* hidden, float* logits, std::string& err);
    // t (1 .. tokens()) tokens at positions pos .. pos + t - 1, each attending to the ones before it: x [t][n_input],
    // hidden [t][n_hidden], logits [t][n_logits] or null; rope_cs as the reference's Step::rope_cs (src/gpu_decode.rs:546-548):
    // for each RoPE table in turn, t rows of cos then sin. Every token's results equal those of t one-token steps bit for bit.
    int step_multi(cudaStream_t st, size_t pos, size_t t, const float* x, const float* rope_cs, float* hidden, float* logits, std::string& err);
    int tokens() const { return tokens_; }
    bool is_prefill() const { return prefill_; }
    float last_step_ms() const { return last_ms_; }  // device time of the last prefill step's kernels (without the copies)
    int kv_write(cudaStream_t st, uint32_t kv, size_t pos0, size_t n, const float* k, const float* v, std::string& err);
    int kv_read(cudaStream_t st, uint32_t kv, size_t pos0, size_t n, float* k, float* v, std::string& err);
    int generate(cudaStream_t st, uint64_t embed_handle, const WeightDev& embed, int32_t first_token, size_t pos0, size_t n_tokens,
                 const float* rope_cs_table, int32_t* out_tokens, float* elapsed_ms, std::string& err);
    int export_handle(void* out128, std::string& err);
    int attach_peers(uint32_t rank, uint32_t world, const void* handles, std::string& err);
    uint64_t launches_per_step() const { return prefill_ ? prefill_launches_ : (uint64_t)ops_.size(); }
    uint64_t launches_per_step(size_t t) const { return prefill_ ? prefill_launches_ : t >= 2 && t <= 4 ? multi_launches_[t] : (uint64_t)ops_.size(); }
    bool uses_weight(uint64_t h) const;

  private:
    struct Op {
        uint32_t kind = 0;  // B2_OP_*, or OP_XPLANES
        float *x = nullptr, *y = nullptr, *z = nullptr;
        WeightDev w{}, w2{};
        bool pair = false;
        int mode = 0;
        const float *p0 = nullptr, *p1 = nullptr;  // device copies of the op's weights
        DecNorm norm{};
        uint32_t rows = 1;
        DecRope rope{};
        DecAttn attn{};
        uint32_t kv = 0;
        uint32_t n = 0;
        int gelu = 0;
        bool meet_first = true;  // EXCHANGE: meet the peers before writing too
        size_t off = 0;  // EXCHANGE: offset of the vector in the activation block, in floats
        NormScale ns{};      // LINEAR: the deferred norm factor of its vector; deferred NORM: where its partial sums go
        XPlanes xp{};  // planes this op writes (norm, attend, xplanes) or reads (linear)
        FusedRope fr{};   // ATTEND: RoPE and the cache append done by the attention kernel (the QK_ROPE op ahead of it is dropped)
        EpiPlanes epi{};  // LINEAR: the planes of its output, written by its own last warps (the split kernel behind it is dropped)
    };
    DecodePlanImpl() = default;
    int run_ops(cudaStream_t st, std::string& err, bool chained, bool first_chained);
    int run_ops_multi(cudaStream_t st, int nt, std::string& err, bool chained);
    int run_prefill(cudaStream_t st, size_t pos, size_t t, std::string& err);
    int step_prefill(cudaStream_t st, size_t pos, size_t t, const float* x, const float* rope_cs, float* hidden, std::string& err);
    int capture(cudaStream_t st, bool with_head, cudaGraphExec_t* out, std::string& err, int nt = 1);
    int check_status(std::string& err);

    std::vector<Op> ops_;
    // plans of several tokens: token i's activations, planes and norm sums sit these strides after token 0's
    int tokens_ = 1;
    size_t block_floats_ = 0, planes_block_ = 0, partial_block_ = 0;
    uint32_t* sp_multi_ = nullptr;        // [tokens][4] step words, inside words_
    std::vector<uint32_t> cs_off_;        // start of each RoPE table's values inside a row of the device table
    cudaGraphExec_t multi_exec_[5] = {};  // [nt], nt = 2 .. tokens
    uint64_t multi_launches_[5] = {};     // kernels of a step of nt tokens
    size_t part_stride_ = 0;              // floats of attention partials per token
    size_t n_counters_ = 0;               // attention counter words (KV heads x tokens)
    // prefill plans
    bool prefill_ = false;
    bool loop_attend_ = false;       // B2_PREFILL_ATTEND=loop: the one-token attention kernel token by token (for comparisons)
    void* x16_ = nullptr;            // [tokens][largest n_in] f16: a product's activations
    float* unscale_ = nullptr;       // [tokens] what the conversion to f16 multiplied each row by, inverted
    float *tmp_a_ = nullptr, *tmp_b_ = nullptr;  // [tokens][largest n_out] products that are added or paired afterwards
    GemmStatus* gemm_status_ = nullptr;
    void* kv16_ = nullptr;           // f16 copy of one f32 cache's rows for the attention kernel
    std::map<size_t, std::vector<GemmPlan*>> gemm_plans_;  // per token count: the products' tensor maps, in op order
    uint64_t prefill_launches_ = 0;
    float last_ms_ = 0.0f;
    std::vector<uint64_t> weight_handles_;
    int sm_count_ = 148;
    bool pdl_ = true;  // programmatic dependent launch between the kernels of a step (B2_PLAN_PDL=0 switches it off)
    // tensor-parallel plans
    bool has_exchange_ = false, attached_ = false;
    PeerSet peers_{};
    uint32_t* xflags_ = nullptr;  // this rank's flag words
    std::vector<void*> peer_maps_;  // what cudaIpcOpenMemHandle returned
    bool defer_norm_ = true;  // norms that feed only products: factor applied after the product (B2_PLAN_DEFER_NORM=0: off)
    float* norm_partials_ = nullptr;
    bool fuse_ = true;  // q / k / v style products of one vector as one launch over concatenated rows (B2_PLAN_FUSE=0: off)
    std::vector<void*> fused_;  // device copies made for that
    bool fuse_rope_ = true;  // RoPE inside the attention kernel where no per-head norm is asked for (B2_PLAN_FUSE_ROPE=0: separate kernels)
    bool epilogue_ = true;  // a 4-bit product writes the planes the next product reads (B2_PLAN_EPILOGUE=0: separate kernels)
    // one allocation each
    float* bufs_ = nullptr;
    std::vector<float*> buf_ptr_;
    std::vector<size_t> buf_len_;
    uint8_t* planes_ = nullptr;
    float* consts_ = nullptr;  // norm weights
    struct Kv {
        void *k = nullptr, *v = nullptr;
        uint32_t nkv = 0, hd = 0;
    };
    std::vector<Kv> kv_;
    uint32_t max_len_ = 0;
    int kv_f16_ = 0;
    float* part_ = nullptr;       // attention partials
    uint32_t* words_ = nullptr;   // sp[4] | status | argmax counter | attention counters[...]
    uint32_t* sp_ = nullptr;
    uint32_t* status_ = nullptr;
    uint32_t* argmax_counter_ = nullptr;
    uint32_t* att_counters_ = nullptr;
    float* rope_table_ = nullptr;  // [max_len][cs_stride]
    uint32_t cs_stride_ = 0;
    float* argmax_val_ = nullptr;
    int* argmax_idx_ = nullptr;
    int* token_ = nullptr;
    int* out_tokens_ = nullptr;    // [max_len]
    float* stage_ = nullptr;       // kv_write / kv_read staging on the device
    size_t stage_floats_ = 0;
    float *input_ = nullptr, *hidden_ = nullptr, *logits_ = nullptr;
    uint32_t n_input_ = 0, n_hidden_ = 0, n_logits_ = 0;
    cudaStream_t cap_stream_ = nullptr;
    cudaGraphExec_t step_exec_ = nullptr;
    cudaGraphExec_t gen_exec_ = nullptr;
    uint64_t gen_embed_ = 0;
    WeightDev gen_embed_dev_{};
    cudaEvent_t ev0_ = nullptr, ev1_ = nullptr;
};

}  // namespace b2
