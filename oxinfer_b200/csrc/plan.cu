// Decode plan: resolves a b2_graph to device pointers, decides where the activation planes of each
// matrix-vector product come from (written by the norm / attention kernel that produces the vector, or by
// a plane kernel of their own), captures the op list into CUDA graphs, and runs steps.
// What the reference does per token with ~11 cuLaunchKernel calls per layer from the host
// (src/cuda_decode.rs:1466-1658) is one cudaGraphLaunch here.
#include "plan.h"

#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <algorithm>
#include <map>
#include <memory>
#include <tuple>

namespace b2 {

namespace {

constexpr uint32_t OP_XPLANES = 100;
constexpr int ATT_THREADS_HOST = 256;  // threads of an attention unit (a thread per head dimension makes the token's key row)
static bool overlaps_f(const float* a, size_t na, const float* b, size_t nb) { return a && b && na && nb && a < b + nb && b < a + na; }
constexpr uint32_t OP_NORM_DEFERRED = 101;  // internal: planes of x * w and per-block sums of squares; the products apply the factor  // internal: planes of a vector no producer kernel could write

std::string fmt(const char* f, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, f);
    vsnprintf(buf, sizeof buf, f, ap);
    va_end(ap);
    return buf;
}

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

#define PLAN_CUDA(call, what)                                                                  \
    do {                                                                                       \
        cudaError_t e_ = (call);                                                               \
        if (e_ != cudaSuccess) {                                                               \
            err = fmt("[b200qmm: plan: %s: %s]", what, cudaGetErrorString(e_));                \
            return e_ == cudaErrorMemoryAllocation ? B2_ERR_NOMEM : B2_ERR_CUDA;               \
        }                                                                                      \
    } while (0)

// Bytes of one row in each of the (up to four) device planes of a format; 0 = plane unused.
void row_bytes(const WeightDev& w, size_t (&rb)[4]) {
    const size_t K = w.n_in;
    rb[0] = rb[1] = rb[2] = rb[3] = 0;
    switch (w.fmt) {
        case B2_FMT_MLX4:
        case B2_FMT_Q4_K: rb[0] = (K / 256) * 144; break;
        case B2_FMT_Q6_K:
            rb[0] = K / 2;
            rb[1] = K / 4;
            rb[2] = K / 16;
            rb[3] = (K / 256) * 2;
            break;
        case B2_FMT_Q8_0:
            rb[0] = K;
            rb[1] = (K / 32) * 2;
            break;
    }
}

// One matrix whose rows are the rows of `parts` in order (same format and n_in): device copies, owned by the plan.
cudaError_t fuse_rows(const std::vector<const WeightDev*>& parts, WeightDev* out, std::vector<void*>& owned) {
    *out = *parts[0];
    size_t rb[4], total = 0;
    row_bytes(*parts[0], rb);
    for (const WeightDev* w : parts) total += w->n_out;
    out->n_out = total;
    const uint8_t* WeightDev::*planes[4] = {&WeightDev::p0, &WeightDev::p1, &WeightDev::p2, &WeightDev::p3};
    for (int pl = 0; pl < 4; pl++) {
        if (!rb[pl]) continue;
        uint8_t* d = nullptr;
        cudaError_t e = cudaMalloc((void**)&d, total * rb[pl]);
        if (e != cudaSuccess) return e;
        owned.push_back(d);
        size_t at = 0;
        for (const WeightDev* w : parts) {
            e = cudaMemcpy(d + at, w->*planes[pl], w->n_out * rb[pl], cudaMemcpyDeviceToDevice);
            if (e != cudaSuccess) return e;
            at += w->n_out * rb[pl];
        }
        out->*planes[pl] = d;
    }
    return cudaSuccess;
}

}  // namespace

DecodePlanImpl::~DecodePlanImpl() {
    for (void* p : fused_) cudaFree(p);
    if (step_exec_) cudaGraphExecDestroy(step_exec_);
    for (cudaGraphExec_t e : multi_exec_)
        if (e) cudaGraphExecDestroy(e);
    if (gen_exec_) cudaGraphExecDestroy(gen_exec_);
    if (ev0_) cudaEventDestroy(ev0_);
    if (ev1_) cudaEventDestroy(ev1_);
    if (cap_stream_) cudaStreamDestroy(cap_stream_);
    for (auto& k : kv_) {
        if (k.k) cudaFree(k.k);
        if (k.v) cudaFree(k.v);
    }
    for (void* m : peer_maps_) cudaIpcCloseMemHandle(m);
    for (auto& kv : gemm_plans_)
        for (GemmPlan* gp : kv.second) gemm_tc_plan_destroy(gp);
    void* frees[] = {kv16_, x16_, unscale_, tmp_a_, tmp_b_, gemm_status_, norm_partials_, xflags_, bufs_, planes_, consts_, part_, words_, rope_table_, argmax_val_, argmax_idx_, token_, out_tokens_, stage_};
    for (void* p : frees)
        if (p) cudaFree(p);
}

bool DecodePlanImpl::uses_weight(uint64_t h) const {
    for (uint64_t w : weight_handles_)
        if (w == h) return true;
    return h != 0 && h == gen_embed_;
}

int DecodePlanImpl::create(const b2_graph* g, const std::function<const WeightDev*(uint64_t)>& resolve, int sm_count, int planes, int tokens,
                           bool prefill, DecodePlanImpl** out, std::string& err) {
    if (!g || !g->bufs || !g->ops || g->n_bufs == 0 || g->n_ops == 0 || !out) {
        err = "[b200qmm: decode_plan: empty graph]";
        return B2_ERR_ARG;
    }
    if (g->max_len == 0 || g->n_rope > 8 || (tokens > 0 && g->max_len < (uint32_t)tokens)) {
        err = "[b200qmm: decode_plan: max_len must be positive (and hold a whole step) and at most 8 RoPE tables are taken]";
        return B2_ERR_ARG;
    }
    if (tokens < 1 || tokens > (prefill ? 8192 : 4)) {
        err = prefill ? "[b200qmm: decode_plan: a prefill plan takes steps of 1 to 8192 tokens]" : "[b200qmm: decode_plan: a plan takes steps of 1 to 4 tokens]";
        return tokens >= 1 ? B2_DECLINED : B2_ERR_ARG;
    }
    if (prefill && g->n_logits) {
        err = "[b200qmm: decode_plan: a prefill plan ends at the hidden states (a graph without logits)]";
        return B2_DECLINED;
    }
    std::unique_ptr<DecodePlanImpl> p(new DecodePlanImpl());
    p->sm_count_ = sm_count;
    p->tokens_ = tokens;
    const size_t T = (size_t)tokens;
    if (const char* e = getenv("B2_PLAN_PDL")) p->pdl_ = atoi(e) != 0;
    if (const char* e = getenv("B2_PLAN_FUSE")) p->fuse_ = atoi(e) != 0;
    if (const char* e = getenv("B2_PLAN_DEFER_NORM")) p->defer_norm_ = atoi(e) != 0;
    int epi_level = 1;  // 1: products that add into the residual row (their split is a deferred norm); 2: gate / up pairs too
    if (const char* e = getenv("B2_PLAN_EPILOGUE")) {
        epi_level = atoi(e);
        p->epilogue_ = epi_level != 0;
    }
    if (const char* e = getenv("B2_PLAN_FUSE_ROPE")) p->fuse_rope_ = atoi(e) != 0;
    if (prefill) {  // the one-token kernels' fusions do not apply: the products are GEMMs
        p->prefill_ = true;
        p->defer_norm_ = p->fuse_rope_ = p->epilogue_ = false;
        const char* e = getenv("B2_PREFILL_ATTEND");
        p->loop_attend_ = e && strcmp(e, "loop") == 0;
    }
    p->max_len_ = g->max_len;
    p->kv_f16_ = g->kv_f16 ? 1 : 0;

    // ---- activation buffers: one allocation, each buffer 256-byte aligned --------------------------
    size_t total = 0;
    std::vector<size_t> off(g->n_bufs);
    for (uint32_t i = 0; i < g->n_bufs; i++) {
        off[i] = total;
        total += align_up((size_t)g->bufs[i], 64);
    }
    total = std::max<size_t>(total, 64);
    p->block_floats_ = total;
    PLAN_CUDA(cudaMalloc((void**)&p->bufs_, T * total * sizeof(float)), "cudaMalloc(buffers)");
    PLAN_CUDA(cudaMemset(p->bufs_, 0, T * total * sizeof(float)), "cudaMemset(buffers)");
    for (uint32_t i = 0; i < g->n_bufs; i++) {
        p->buf_ptr_.push_back(p->bufs_ + off[i]);
        p->buf_len_.push_back((size_t)g->bufs[i]);
    }
    bool bad_view = false;
    auto view = [&](b2_view v, size_t n) -> float* {
        if (v.buf >= g->n_bufs || (size_t)v.off + n > p->buf_len_[v.buf]) {
            bad_view = true;
            return nullptr;
        }
        return p->buf_ptr_[v.buf] + v.off;
    };

    // ---- RoPE table layout ------------------------------------------------------------------------
    std::vector<uint32_t> cs_off(g->n_rope + 1, 0);
    for (uint32_t i = 0; i < g->n_rope; i++) cs_off[i + 1] = cs_off[i] + 2 * g->rope_halves[i];
    p->cs_stride_ = cs_off[g->n_rope];
    p->cs_off_ = cs_off;

    // ---- KV caches --------------------------------------------------------------------------------
    const size_t esz = p->kv_f16_ ? 2 : 4;
    uint32_t max_nh = 0, max_hd = 0, max_nkv = 0;
    size_t max_row = 0;
    for (uint32_t i = 0; i < g->n_kv; i++) {
        Kv k;
        k.nkv = g->kv_nkv[i];
        k.hd = g->kv_hd[i];
        size_t bytes = (size_t)k.nkv * g->max_len * k.hd * esz;
        PLAN_CUDA(cudaMalloc(&k.k, bytes), "cudaMalloc(K cache)");
        p->kv_.push_back(k);  // pushed before V so that a failure below still frees K
        PLAN_CUDA(cudaMalloc(&p->kv_.back().v, bytes), "cudaMalloc(V cache)");
        PLAN_CUDA(cudaMemset(p->kv_.back().k, 0, bytes), "cudaMemset(K cache)");
        PLAN_CUDA(cudaMemset(p->kv_.back().v, 0, bytes), "cudaMemset(V cache)");
        max_nkv = std::max(max_nkv, k.nkv);
        max_row = std::max(max_row, (size_t)k.nkv * k.hd);
    }

    // ---- norm weights: one device block -----------------------------------------------------------
    size_t n_consts = 0;
    for (uint32_t i = 0; i < g->n_ops; i++) {
        const b2_op& o = g->ops[i];
        if (o.kind == B2_OP_NORM && o.p0) n_consts += align_up(o.n, 64);
        if (o.kind == B2_OP_QK_ROPE) n_consts += (o.p0 ? align_up(o.hd, 64) : 0) + (o.p1 ? align_up(o.hd, 64) : 0);
    }
    PLAN_CUDA(cudaMalloc((void**)&p->consts_, std::max<size_t>(n_consts, 64) * sizeof(float)), "cudaMalloc(norm weights)");
    size_t consts_at = 0;
    auto put_const = [&](const float* host, size_t n, const float** dev) -> cudaError_t {
        float* d = p->consts_ + consts_at;
        consts_at += align_up(n, 64);
        *dev = d;
        return cudaMemcpy(d, host, n * sizeof(float), cudaMemcpyHostToDevice);
    };

    // ---- ops -------------------------------------------------------------------------------------
    // Planes bookkeeping. key = (buffer, offset, length) of a vector; `valid` = planes of the current
    // contents exist in that region; `writer` = index (in ops_) of the norm / attention op that wrote
    // exactly this vector last and can still be told to write its planes.
    using Key = std::tuple<uint32_t, uint32_t, uint32_t>;
    std::map<Key, size_t> valid;    // -> region index
    std::map<Key, size_t> writer;   // -> op index
    std::vector<size_t> region_k;   // K of each planes region
    auto touch = [&](uint32_t buf) {  // a write into `buf`: planes and writers of its vectors are stale
        for (auto it = valid.begin(); it != valid.end();) it = std::get<0>(it->first) == buf ? valid.erase(it) : std::next(it);
        for (auto it = writer.begin(); it != writer.end();) it = std::get<0>(it->first) == buf ? writer.erase(it) : std::next(it);
    };
    std::vector<std::pair<size_t, size_t>> region_of_op;  // (op index, region): xp filled in once regions are allocated

    for (uint32_t i = 0; i < g->n_ops; i++) {
        const b2_op& o = g->ops[i];
        Op op;
        op.kind = o.kind;
        switch (o.kind) {
            case B2_OP_NORM: {
                if (o.n == 0 || o.rows == 0) {
                    err = "[b200qmm: decode_plan: norm of nothing]";
                    return B2_ERR_ARG;
                }
                size_t xs = o.x_stride ? o.x_stride : o.n, os = o.out_stride ? o.out_stride : o.n;
                op.x = view(o.x, (size_t)(o.rows - 1) * xs + o.n);
                op.y = view(o.y, (size_t)(o.rows - 1) * os + o.n);
                op.norm = DecNorm{o.n, (uint32_t)xs, (uint32_t)os, o.add ? 1u : 0u, 0u, o.pre == 0.0f ? 1.0f : o.pre, o.eps};
                op.rows = o.rows;
                if (o.p0) PLAN_CUDA(put_const(o.p0, o.n, &op.p0), "cudaMemcpy(norm weights)");
                touch(o.y.buf);
                if (o.rows == 1 && o.n % 32 == 0) writer[Key{o.y.buf, o.y.off, o.n}] = p->ops_.size();
                break;
            }
            case B2_OP_LINEAR: {
                const WeightDev* w = resolve(o.w);
                if (!w) {
                    err = "[b200qmm: decode_plan: unknown weight handle]";
                    return B2_ERR_ARG;
                }
                if (w->n_out != o.n_out || w->n_in != o.n_in) {
                    err = fmt("[b200qmm: decode_plan: linear %u x %u does not match its weight %zu x %zu]", o.n_out, o.n_in, w->n_out, w->n_in);
                    return B2_ERR_ARG;
                }
                if (!prefill && !gemv_supports(*w)) {
                    err = "[b200qmm: decode_plan: a weight's shape is outside the matrix-vector kernels]";
                    return B2_DECLINED;
                }
                if (prefill && (!gemm_tc_supports(*w, (size_t)tokens) || o.mode == B2_MODE_ADD_GATED || o.n_out % 4)) {
                    err = "[b200qmm: decode_plan: a prefill plan takes products with a tensor-core kernel (Q4_K, MLX-4, Q6_K, Q8_0, FP8), rows in multiples of 4, "
                          "and no gated mode]";
                    return B2_DECLINED;
                }
                op.w = *w;
                p->weight_handles_.push_back(o.w);
                op.mode = (int)o.mode;
                if (o.mode > B2_MODE_ADD_GATED) {
                    err = "[b200qmm: decode_plan: bad linear mode]";
                    return B2_ERR_ARG;
                }
                op.pair = o.mode == B2_MODE_SILU_PAIR || o.mode == B2_MODE_GELU_PAIR;
                if (op.pair) {
                    const WeightDev* u = resolve(o.w2);
                    if (!u) {
                        err = "[b200qmm: decode_plan: a pair needs its second matrix]";
                        return B2_ERR_ARG;
                    }
                    if (u->fmt != w->fmt || u->n_in != w->n_in || u->n_out != w->n_out) {
                        err = "[b200qmm: decode_plan: the pair's matrices differ in shape or format]";
                        return B2_DECLINED;
                    }
                    op.w2 = *u;
                    p->weight_handles_.push_back(o.w2);
                }
                op.x = view(o.x, o.n_in);
                op.y = view(o.y, o.n_out);
                if (o.mode == B2_MODE_ADD_GATED) op.z = view(o.z, 1);
                // Products of the same vector that store into consecutive ranges (q, k, v) run as one launch over
                // a row-wise concatenation of their matrices (a device copy the plan owns).
                if (p->fuse_ && o.mode == B2_MODE_STORE && w->fmt != B2_FMT_F8E4M3) {
                    std::vector<const WeightDev*> parts{w};
                    uint32_t end = o.y.off + o.n_out, j = i + 1;
                    for (; j < g->n_ops; j++) {
                        const b2_op& n = g->ops[j];
                        if (n.kind != B2_OP_LINEAR || n.mode != B2_MODE_STORE || n.x.buf != o.x.buf || n.x.off != o.x.off || n.n_in != o.n_in ||
                            n.y.buf != o.y.buf || n.y.off != end || n.y.buf == n.x.buf)
                            break;
                        const WeightDev* nw = resolve(n.w);
                        if (!nw || nw->fmt != w->fmt || nw->n_in != w->n_in || nw->n_out != n.n_out || nw->group != w->group) break;
                        parts.push_back(nw);
                        p->weight_handles_.push_back(n.w);
                        end += n.n_out;
                    }
                    if (parts.size() > 1) {
                        PLAN_CUDA(fuse_rows(parts, &op.w, p->fused_), "fusing matrices of one vector");
                        op.y = view(o.y, end - o.y.off);
                        i = j - 1;  // the fused ops are done
                    }
                }
                if (w->fmt != B2_FMT_F8E4M3 && !prefill) {
                    Key key{o.x.buf, o.x.off, o.n_in};
                    size_t region;
                    auto v = valid.find(key);
                    if (v != valid.end()) {
                        region = v->second;
                    } else {
                        region = region_k.size();
                        region_k.push_back(o.n_in);
                        auto wr = writer.find(key);
                        if (wr != writer.end()) {
                            Op& prod = p->ops_[wr->second];
                            if (prod.kind == B2_OP_NORM) prod.norm.planes = 1;
                            else prod.attn.planes = 1;
                            region_of_op.push_back({wr->second, region});
                        } else {
                            Op xp;
                            xp.kind = OP_XPLANES;
                            xp.x = op.x;
                            xp.n = o.n_in;
                            region_of_op.push_back({p->ops_.size(), region});
                            p->ops_.push_back(xp);
                        }
                        valid[key] = region;
                    }
                    region_of_op.push_back({p->ops_.size(), region});
                }
                if (o.y.buf == o.x.buf && !(o.y.off + o.n_out <= o.x.off || o.x.off + o.n_in <= o.y.off)) {
                    err = "[b200qmm: decode_plan: a linear op writes over its own input]";
                    return B2_ERR_ARG;
                }
                touch(o.y.buf);
                break;
            }
            case B2_OP_QK_ROPE: {
                if (o.kv >= g->n_kv || o.rope >= g->n_rope || g->kv_nkv[o.kv] != o.nkv || g->kv_hd[o.kv] != o.hd || o.hd > 256 || o.hd % 32 ||
                    g->rope_halves[o.rope] != o.half_rot || 2 * o.half_rot > o.hd) {
                    err = "[b200qmm: decode_plan: qk_rope does not match its KV cache or RoPE table]";
                    return B2_ERR_ARG;
                }
                size_t q_stride = o.q_stride ? o.q_stride : o.hd;
                size_t need = std::max({(size_t)(o.nh - 1) * q_stride + o.hd, (size_t)o.k_off + (size_t)o.nkv * o.hd,
                                        o.v_from_k ? (size_t)0 : (size_t)o.v_off + (size_t)o.nkv * o.hd});
                op.x = view(o.x, need);
                op.y = view(o.y, (size_t)o.nh * o.hd);
                op.kv = o.kv;
                op.rope = DecRope{o.nh, o.nkv, o.hd, o.half_rot, (uint32_t)q_stride, o.k_off, o.v_off, o.interleaved, o.v_norm, o.v_from_k,
                                  g->max_len, p->cs_stride_, cs_off[o.rope], o.eps};
                if (o.p0) PLAN_CUDA(put_const(o.p0, o.hd, &op.p0), "cudaMemcpy(q norm)");
                if (o.p1) PLAN_CUDA(put_const(o.p1, o.hd, &op.p1), "cudaMemcpy(k norm)");
                touch(o.y.buf);
                break;
            }
            case B2_OP_ATTEND: {
                if (o.kv >= g->n_kv || g->kv_nkv[o.kv] != o.nkv || g->kv_hd[o.kv] != o.hd) {
                    err = "[b200qmm: decode_plan: attend does not match its KV cache]";
                    return B2_ERR_ARG;
                }
                if (prefill && !attend_rows_supports(o.nh, o.nkv, o.hd)) {
                    err = "[b200qmm: decode_plan: prefill attention takes head dimensions 64 and 128]";
                    return B2_DECLINED;
                }
                if ((!prefill || p->loop_attend_) && !attend_supports(o.nh, o.nkv, o.hd)) {
                    err = fmt("[b200qmm: decode_plan: attention with %u heads over %u KV heads of %u is outside the kernel (head dim 64 / 128, "
                              "1 / 2 / 4 / 8 heads per KV head)]", o.nh, o.nkv, o.hd);
                    return B2_DECLINED;
                }
                op.x = view(o.x, (size_t)o.nh * o.hd);
                op.y = view(o.y, (size_t)o.nh * o.hd);
                op.kv = o.kv;
                op.attn = DecAttn{o.nh, o.nkv, o.hd, g->max_len, o.window, 0u, o.scale};
                max_nh = std::max(max_nh, o.nh);
                max_hd = std::max(max_hd, o.hd);
                touch(o.y.buf);
                writer[Key{o.y.buf, o.y.off, o.nh * o.hd}] = p->ops_.size();
                break;
            }
            case B2_OP_GLU: {
                op.x = view(o.x, o.n);
                op.z = view(o.z, o.n);
                op.y = view(o.y, o.n);
                op.n = o.n;
                op.gelu = o.gelu ? 1 : 0;
                touch(o.y.buf);
                break;
            }
            case B2_OP_EXCHANGE: {
                if (tokens > 1) {
                    err = "[b200qmm: decode_plan: a tensor-parallel graph runs one token per step]";
                    return B2_DECLINED;
                }
                if (o.n == 0 || o.n % 32) {
                    err = "[b200qmm: decode_plan: an exchanged vector must be a positive multiple of 32 values]";
                    return B2_ERR_ARG;
                }
                op.x = view(o.x, o.n);
                op.n = o.n;
                if (op.x) op.off = (size_t)(op.x - p->bufs_);
                p->has_exchange_ = true;
                touch(o.x.buf);
                break;
            }
            default:
                err = fmt("[b200qmm: decode_plan: op kind %u is not taken by this backend]", o.kind);
                return B2_DECLINED;
        }
        if (bad_view) {
            err = fmt("[b200qmm: decode_plan: op %u reaches outside its buffer]", i);
            return B2_ERR_ARG;
        }
        p->ops_.push_back(op);
    }
    p->n_input_ = g->n_input;
    p->n_hidden_ = g->n_hidden;
    p->n_logits_ = g->n_logits;
    p->input_ = view(g->input, g->n_input);
    p->hidden_ = view(g->hidden, g->n_hidden);
    if (g->n_logits) p->logits_ = view(g->logits, g->n_logits);
    if (bad_view) {
        err = "[b200qmm: decode_plan: input / hidden / logits reach outside their buffers]";
        return B2_ERR_ARG;
    }

    // ---- norms whose output only products read: the factor moves behind the product -----------------------------
    // The one-CTA norm spends most of its time splitting the row into planes on a single SM; when nothing reads the
    // normalized row itself (every reader is a product over its planes), a grid of independent warps splits x * w and
    // leaves the blocks' sums of squares, and the products multiply by the factor (NormScale).
    size_t norm_floats = 0;
    if (p->defer_norm_) {
        auto overlaps = [](const float* a, size_t na, const float* b, size_t nb) { return a && b && a < b + nb && b < a + na; };
        for (size_t a = 0; a < p->ops_.size(); a++) {
            Op& nrm = p->ops_[a];
            if (nrm.kind != B2_OP_NORM || !nrm.norm.planes || nrm.rows != 1 || nrm.norm.add) continue;
            const float* y = nrm.y;
            const size_t n = nrm.norm.n;
            if (overlaps(y, n, p->hidden_, p->n_hidden_) || overlaps(y, n, p->logits_, p->n_logits_) || overlaps(y, n, p->input_, p->n_input_)) continue;
            bool ok = true;
            std::vector<size_t> users;
            for (size_t b = a + 1; b < p->ops_.size() && ok; b++) {
                const Op& o = p->ops_[b];
                bool writes = false;
                switch (o.kind) {
                    case B2_OP_LINEAR:
                        if (o.x == y && o.w.n_in == n && o.w.fmt != B2_FMT_F8E4M3) users.push_back(b);
                        else if (overlaps(y, n, o.x, o.w.n_in)) ok = false;
                        if (overlaps(y, n, o.y, o.w.n_out)) {
                            if (o.mode != B2_MODE_STORE && !o.pair) ok = false;  // reads what it adds to
                            writes = true;
                        }
                        break;
                    case B2_OP_NORM:
                    case OP_NORM_DEFERRED:
                        if (overlaps(y, n, o.x, (size_t)(o.rows - 1) * o.norm.x_stride + o.norm.n)) ok = false;
                        writes = overlaps(y, n, o.y, (size_t)(o.rows - 1) * o.norm.out_stride + o.norm.n);
                        break;
                    case OP_XPLANES: ok = ok && !overlaps(y, n, o.x, o.n); break;
                    case B2_OP_EXCHANGE:
                        if (overlaps(y, n, o.x, o.n)) ok = false;
                        break;
                    case B2_OP_GLU:
                        if (overlaps(y, n, o.x, o.n) || overlaps(y, n, o.z, o.n)) ok = false;
                        writes = overlaps(y, n, o.y, o.n);
                        break;
                    default:  // RoPE, attention: any overlap of their views with the row disqualifies it
                        if (overlaps(y, n, o.x, n) || overlaps(y, n, o.y, n)) ok = false;
                        break;
                }
                if (writes) break;
            }
            if (!ok || users.empty()) continue;
            nrm.kind = OP_NORM_DEFERRED;
            nrm.ns = NormScale{(const float*)(uintptr_t)norm_floats, (uint32_t)(n / 32), 1.0f / (float)n, nrm.norm.eps};  // offset now, pointer below
            for (size_t b : users) p->ops_[b].ns = nrm.ns;
            norm_floats += (n / 32 + 63) / 64 * 64;
        }
    }
    p->partial_block_ = norm_floats;
    if (norm_floats) {
        PLAN_CUDA(cudaMalloc((void**)&p->norm_partials_, T * norm_floats * sizeof(float)), "cudaMalloc(norm partial sums)");
        PLAN_CUDA(cudaMemset(p->norm_partials_, 0, T * norm_floats * sizeof(float)), "cudaMemset(norm partial sums)");
        for (Op& o : p->ops_)
            if ((o.kind == OP_NORM_DEFERRED || o.kind == B2_OP_LINEAR) && o.ns.count)
                o.ns.partial = p->norm_partials_ + (size_t)(uintptr_t)o.ns.partial;
    }

    // ---- planes regions ---------------------------------------------------------------------------
    size_t planes_total = 0;
    std::vector<size_t> region_at(region_k.size());
    for (size_t r = 0; r < region_k.size(); r++) {
        region_at[r] = planes_total;
        planes_total += align_up(xplanes_bytes(region_k[r]), 256);
    }
    planes_total = std::max<size_t>(planes_total, 256);
    p->planes_block_ = planes_total;
    PLAN_CUDA(cudaMalloc((void**)&p->planes_, T * planes_total), "cudaMalloc(planes)");
    for (auto& [oi, r] : region_of_op) {
        p->ops_[oi].xp = xplanes_at(p->planes_ + region_at[r], region_k[r]);
        p->ops_[oi].xp.np = planes;
    }

    // ---- RoPE inside the attention kernel ----------------------------------------------------------------------
    // A QK_ROPE op without per-head norms whose rotated queries only the ATTEND op right behind it reads: the attention
    // kernel rotates the queries as it stages them and the unit that holds the newest keys appends the token's key and
    // value (FusedRope); one launch fewer per layer.
    if (p->fuse_rope_) {
        std::vector<Op> kept;
        kept.reserve(p->ops_.size());
        for (size_t b = 0; b < p->ops_.size(); b++) {
            Op& at = p->ops_[b];
            Op* rp = kept.empty() ? nullptr : &kept.back();
            if (at.kind == B2_OP_ATTEND && rp && rp->kind == B2_OP_QK_ROPE && !rp->p0 && !rp->p1 && !rp->rope.v_norm && !rp->rope.v_from_k &&
                rp->kv == at.kv && rp->y == at.x && rp->rope.nh == at.attn.nh && rp->rope.nkv == at.attn.nkv && rp->rope.hd == at.attn.hd &&
                rp->rope.hd <= (uint32_t)ATT_THREADS_HOST) {
                // nobody else may read the rotated queries: they are not written any more
                bool other_reader = overlaps_f(rp->y, (size_t)rp->rope.nh * rp->rope.hd, p->hidden_, p->n_hidden_) ||
                                    overlaps_f(rp->y, (size_t)rp->rope.nh * rp->rope.hd, p->logits_, p->n_logits_);
                for (size_t c = 0; c < p->ops_.size() && !other_reader; c++) {
                    if (c == b || &p->ops_[c] == &at) continue;
                    const Op& o = p->ops_[c];
                    if (o.kind == B2_OP_QK_ROPE) continue;  // writes it
                    const float* q0 = rp->y;
                    const size_t qn = (size_t)rp->rope.nh * rp->rope.hd;
                    const size_t xn = o.kind == B2_OP_LINEAR ? o.w.n_in : o.kind == B2_OP_ATTEND ? (size_t)o.attn.nh * o.attn.hd
                                      : (o.kind == B2_OP_NORM || o.kind == OP_NORM_DEFERRED) ? (size_t)(o.rows - 1) * o.norm.x_stride + o.norm.n : o.n;
                    if (o.kind == B2_OP_ATTEND && o.x == q0) continue;  // another layer's attention over its own fused queries
                    if (overlaps_f(q0, qn, o.x, xn) || overlaps_f(q0, qn, o.z, o.n ? o.n : 1)) other_reader = true;
                }
                if (!other_reader) {
                    at.fr = FusedRope{rp->x, nullptr, rp->rope};  // the table's address is known at launch
                    kept.back() = at;
                    continue;
                }
            }
            kept.push_back(at);
        }
        p->ops_ = std::move(kept);
    }

    // ---- planes written by the product ahead ---------------------------------------------------------------------
    // A split kernel (deferred norm, or the planes of an MLP activation) that directly follows the 4-bit product which
    // wrote its whole input is dropped: that product's CTAs then own whole blocks of 32 rows and split each block once
    // its rows are done (EpiPlanes). Saves a launch per product whose output feeds another product.
    if (p->epilogue_ && p->pdl_) {
        std::vector<Op> kept;
        kept.reserve(p->ops_.size());
        for (size_t b = 0; b < p->ops_.size(); b++) {
            const Op& nx = p->ops_[b];
            Op* lin = kept.empty() ? nullptr : &kept.back();
            if (lin && lin->kind == B2_OP_LINEAR && !lin->epi.out.planes && gemv_takes_epilogue(lin->w)) {
                const size_t n = lin->w.n_out;
                const bool norm = nx.kind == OP_NORM_DEFERRED && nx.x == lin->y && nx.norm.n == n && nx.rows == 1;
                const bool split = nx.kind == OP_XPLANES && nx.x == lin->y && nx.n == n && (epi_level >= 2 || !lin->pair);
                if (norm || split) {
                    lin->epi = EpiPlanes{nx.xp, norm ? nx.p0 : nullptr, norm ? const_cast<float*>(nx.ns.partial) : nullptr, norm ? nx.norm.pre : 1.0f};
                    continue;
                }
            }
            kept.push_back(nx);
        }
        p->ops_ = std::move(kept);
    }

    // ---- scratch ------------------------------------------------------------------------------------
    p->part_stride_ = max_nh ? attend_part_floats(max_nh, max_hd) : 0;
    if (max_nh) PLAN_CUDA(cudaMalloc((void**)&p->part_, (prefill ? 1 : T) * p->part_stride_ * sizeof(float)), "cudaMalloc(attention partials)");
    size_t n_words = 8 + T * std::max<uint32_t>(max_nkv, 1) + 4 * T;  // (a prefill plan's T counters are unused: a few KB)
    PLAN_CUDA(cudaMalloc((void**)&p->words_, n_words * 4), "cudaMalloc(step words)");
    PLAN_CUDA(cudaMemset(p->words_, 0, n_words * 4), "cudaMemset(step words)");
    if (p->has_exchange_) {
        PLAN_CUDA(cudaMalloc((void**)&p->xflags_, 32 * 4), "cudaMalloc(exchange flags)");
        PLAN_CUDA(cudaMemset(p->xflags_, 0, 32 * 4), "cudaMemset(exchange flags)");
    }
    p->sp_ = p->words_;
    p->status_ = p->words_ + 4;
    p->argmax_counter_ = p->words_ + 5;
    p->att_counters_ = p->words_ + 8;
    p->n_counters_ = T * std::max<uint32_t>(max_nkv, 1);
    p->sp_multi_ = p->words_ + 8 + p->n_counters_;
    size_t table = (size_t)std::max<uint32_t>(p->cs_stride_, 1) * g->max_len;
    PLAN_CUDA(cudaMalloc((void**)&p->rope_table_, table * sizeof(float)), "cudaMalloc(rope table)");
    PLAN_CUDA(cudaMemset(p->rope_table_, 0, table * sizeof(float)), "cudaMemset(rope table)");
    const size_t n_partials = std::max(128, sm_count);  // one per CTA of the argmax kernel
    PLAN_CUDA(cudaMalloc((void**)&p->argmax_val_, n_partials * sizeof(float)), "cudaMalloc(argmax)");
    PLAN_CUDA(cudaMalloc((void**)&p->argmax_idx_, n_partials * sizeof(int)), "cudaMalloc(argmax)");
    PLAN_CUDA(cudaMalloc((void**)&p->token_, sizeof(int)), "cudaMalloc(token)");
    PLAN_CUDA(cudaMalloc((void**)&p->out_tokens_, (size_t)g->max_len * sizeof(int)), "cudaMalloc(tokens)");
    p->stage_floats_ = std::max<size_t>(max_row, 1) * 256;
    PLAN_CUDA(cudaMalloc((void**)&p->stage_, 2 * p->stage_floats_ * sizeof(float)), "cudaMalloc(KV staging)");
    PLAN_CUDA(cudaStreamCreateWithFlags(&p->cap_stream_, cudaStreamNonBlocking), "cudaStreamCreate");
    PLAN_CUDA(cudaEventCreate(&p->ev0_), "cudaEventCreate");
    PLAN_CUDA(cudaEventCreate(&p->ev1_), "cudaEventCreate");

    if (prefill) {
        size_t max_k = 64, max_n = 64;
        for (const Op& o : p->ops_)
            if (o.kind == B2_OP_LINEAR) {
                max_k = std::max(max_k, o.w.n_in);
                max_n = std::max(max_n, o.w.n_out);
            }
        PLAN_CUDA(cudaMalloc(&p->x16_, T * max_k * 2), "cudaMalloc(f16 activations)");
        PLAN_CUDA(cudaMalloc((void**)&p->unscale_, T * sizeof(float)), "cudaMalloc(row factors)");
        PLAN_CUDA(cudaMalloc((void**)&p->tmp_a_, T * max_n * sizeof(float)), "cudaMalloc(products)");
        PLAN_CUDA(cudaMalloc((void**)&p->tmp_b_, T * max_n * sizeof(float)), "cudaMalloc(products)");
        size_t kv16 = 0;
        for (const Kv& k : p->kv_) kv16 = std::max(kv16, attend_rows_scratch_bytes(k.nkv, g->max_len, k.hd, p->kv_f16_));
        if (kv16) PLAN_CUDA(cudaMalloc(&p->kv16_, kv16), "cudaMalloc(f16 cache rows)");
        PLAN_CUDA(cudaMalloc((void**)&p->gemm_status_, sizeof(GemmStatus)), "cudaMalloc(GEMM status)");
        PLAN_CUDA(cudaMemset(p->gemm_status_, 0, sizeof(GemmStatus)), "cudaMemset(GEMM status)");
        *out = p.release();  // nothing is captured: a step launches its kernels (a few per op, whatever the token count)
        return B2_OK;
    }
    // One eager pass (loads every kernel outside a capture, and surfaces launch errors with their op),
    // then the step graph.
    PLAN_CUDA(launch_set_step(p->sp_, 0, 0, 0, nullptr, 0, p->cap_stream_), "set_step");
    int rc = p->run_ops(p->cap_stream_, err, false, false);
    if (rc) return rc;
    PLAN_CUDA(cudaStreamSynchronize(p->cap_stream_), "first pass");
    rc = p->check_status(err);
    if (rc) return rc;
    rc = p->capture(p->cap_stream_, false, &p->step_exec_, err);
    if (rc) return rc;
    // Steps of several tokens: the same eager pass and a graph per token count.
    for (int nt = 2; nt <= tokens; nt++) {
        uint32_t words[16] = {};
        for (int tk = 0; tk < nt; tk++) words[4 * tk] = (uint32_t)tk;
        PLAN_CUDA(cudaMemcpyAsync(p->sp_multi_, words, 16 * nt, cudaMemcpyHostToDevice, p->cap_stream_), "cudaMemcpy(step words)");
        rc = p->run_ops_multi(p->cap_stream_, nt, err, false);
        if (rc) return rc;
        PLAN_CUDA(cudaStreamSynchronize(p->cap_stream_), "first pass (several tokens)");
        rc = p->check_status(err);
        if (rc) return rc;
        rc = p->capture(p->cap_stream_, false, &p->multi_exec_[nt], err, nt);
        if (rc) return rc;
    }
    *out = p.release();
    return B2_OK;
}

// `chained`: every launch but the first (`first_chained`: the first too) carries the programmatic-dependent-launch
// attribute, so each kernel starts (and fetches its first weights) while the one before it drains.
int DecodePlanImpl::run_ops(cudaStream_t st, std::string& err, bool chained, bool first_chained) {
    for (size_t i = 0; i < ops_.size(); i++) {
        const Op& o = ops_[i];
        const bool pdl = chained && (i > 0 || first_chained);
        cudaError_t e = cudaSuccess;
        switch (o.kind) {
            case B2_OP_NORM: e = launch_norm(o.x, o.y, o.p0, o.norm, o.rows, o.xp, st, pdl); break;
            case OP_XPLANES: e = launch_xplanes(o.x, o.n, o.xp, st, pdl); break;
            case OP_NORM_DEFERRED: e = launch_norm_planes(o.x, o.p0, o.norm.pre, o.norm.n, o.xp, const_cast<float*>(o.ns.partial), st, pdl); break;
            case B2_OP_LINEAR: e = launch_gemv(o.w, o.pair ? &o.w2 : nullptr, o.x, o.xp, o.y, o.mode, o.z, sm_count_, st, pdl, o.ns, o.epi); break;
            case B2_OP_QK_ROPE:
                e = launch_qk_rope(o.x, o.y, kv_[o.kv].k, kv_[o.kv].v, kv_f16_, o.p0, o.p1, rope_table_, sp_, o.rope, st, pdl);
                break;
            case B2_OP_ATTEND:
                if (o.fr.qkv) {
                    FusedRope fr = o.fr;
                    fr.cs_table = rope_table_;
                    e = launch_attend(o.x, kv_[o.kv].k, kv_[o.kv].v, kv_f16_, o.y, part_, att_counters_, sp_, o.attn, o.xp, status_, st, pdl, &fr);
                } else {
                    e = launch_attend(o.x, kv_[o.kv].k, kv_[o.kv].v, kv_f16_, o.y, part_, att_counters_, sp_, o.attn, o.xp, status_, st, pdl);
                }
                break;
            case B2_OP_GLU: e = launch_glu(o.x, o.z, o.y, o.n, o.gelu, st, pdl); break;
            case B2_OP_EXCHANGE:
                if (attached_) e = launch_exchange(peers_, o.off, o.n, xflags_, status_, st, pdl, o.meet_first);  // the first pass of a lone rank has nobody to meet
                break;
            default: e = cudaErrorInvalidValue;
        }
        if (e != cudaSuccess) {
            err = fmt("[b200qmm: plan: op %zu (kind %u): %s]", i, o.kind, cudaGetErrorString(e));
            return B2_ERR_CUDA;
        }
    }
    return B2_OK;
}

// The ops for nt tokens at once, op by op: a product reads its weights once for all tokens where the tokens' vectors fit in
// shared memory together (launch_gemv_multi: each token's sums are its one-token sums), every other op runs once per token
// on that token's blocks (activations, planes, norm sums, step words). Attention and RoPE are ordinary launches, not
// dependent ones: token i's attention reads the keys the launches just ahead of it appended, and its first key tile is
// fetched before the dependency wait.
int DecodePlanImpl::run_ops_multi(cudaStream_t st, int nt, std::string& err, bool chained) {
    auto A = [&](const float* p, int tk) -> float* { return p ? const_cast<float*>(p) + (size_t)tk * block_floats_ : nullptr; };
    auto P = [&](XPlanes xp, int tk) {
        if (!xp.planes) return xp;
        const size_t off = (size_t)tk * planes_block_;
        xp.planes = (int8_t*)((uint8_t*)xp.planes + off);
        xp.sx = (float2*)((uint8_t*)xp.sx + off);
        xp.v16 = (int32_t*)((uint8_t*)xp.v16 + off);
        return xp;
    };
    auto N = [&](NormScale ns, int tk) {
        if (ns.partial) ns.partial += (size_t)tk * partial_block_;
        return ns;
    };
    bool first = true;
    uint64_t count = 0;
    auto pdl = [&]() {
        const bool v = chained && !first;
        first = false;
        count++;
        return v;
    };
    for (size_t i = 0; i < ops_.size(); i++) {
        const Op& o = ops_[i];
        cudaError_t e = cudaSuccess;
        switch (o.kind) {
            case B2_OP_NORM:
                for (int tk = 0; tk < nt && e == cudaSuccess; tk++)
                    e = launch_norm(A(o.x, tk), A(o.y, tk), o.p0, o.norm, o.rows, P(o.xp, tk), st, pdl());
                break;
            case OP_XPLANES:  // one launch for all tokens (a block of a token's planes is made by one warp either way: the same bits)
                e = launch_xplanes(o.x, o.n, o.xp, st, pdl(), nt, block_floats_, planes_block_);
                break;
            case OP_NORM_DEFERRED:
                e = launch_norm_planes(o.x, o.p0, o.norm.pre, o.norm.n, o.xp, const_cast<float*>(o.ns.partial), st, pdl(), nt, block_floats_, planes_block_,
                                       partial_block_);
                break;
            case B2_OP_LINEAR: {
                // FP8 products go token by token: their one-token kernel is the tensor-core one, and the tokens must match it.
                // So do two tokens of a Q6_K / Q8_0 product: their several-token kernel does a token's arithmetic per token, and the
                // one-token launches are the faster form inside a chain of dependent launches (gemv_multi_pays).
                const bool together = o.mode != B2_MODE_ADD_GATED && o.w.fmt != B2_FMT_F8E4M3 && gemv_multi_pays(o.w, nt);
                if (together) {
                    e = launch_gemv_multi(o.w, o.pair ? &o.w2 : nullptr, o.x, block_floats_, o.xp, planes_block_, o.y, block_floats_, nt, o.mode,
                                          sm_count_, st, pdl(), o.ns, partial_block_);
                    // the split the one-token product does in its epilogue (the same bits as the kernels of their own)
                    if (e == cudaSuccess && o.epi.out.planes) {
                        if (o.epi.partial)
                            e = launch_norm_planes(o.y, o.epi.w, o.epi.pre, o.w.n_out, o.epi.out, o.epi.partial, st, pdl(), nt, block_floats_, planes_block_,
                                                   partial_block_);
                        else
                            e = launch_xplanes(o.y, o.w.n_out, o.epi.out, st, pdl(), nt, block_floats_, planes_block_);
                    }
                    break;
                }
                for (int tk = 0; tk < nt && e == cudaSuccess; tk++) {
                    EpiPlanes epi = o.epi;
                    if (epi.out.planes) {
                        epi.out = P(epi.out, tk);
                        if (epi.partial) epi.partial += (size_t)tk * partial_block_;
                    }
                    e = launch_gemv(o.w, o.pair ? &o.w2 : nullptr, A(o.x, tk), P(o.xp, tk), A(o.y, tk), o.mode, A(o.z, tk), sm_count_, st, pdl(),
                                    N(o.ns, tk), epi);
                }
                break;
            }
            case B2_OP_QK_ROPE:  // all tokens in one launch (the one-token arithmetic per head)
                e = launch_qk_rope_rows(o.x, o.y, block_floats_, (uint32_t)nt, kv_[o.kv].k, kv_[o.kv].v, kv_f16_, o.p0, o.p1, rope_table_, sp_multi_, o.rope,
                                        st);
                first = false;
                count++;
                break;
            case B2_OP_ATTEND: {
                // Where the one-token plan rotates and appends inside the attention kernel, the tokens' keys and values go into
                // the caches first (the same arithmetic in a kernel of its own); then one launch attends for all tokens.
                if (o.fr.qkv) {
                    e = launch_qk_rope_rows(o.fr.qkv, o.x, block_floats_, (uint32_t)nt, kv_[o.kv].k, kv_[o.kv].v, kv_f16_, nullptr, nullptr, rope_table_,
                                            sp_multi_, o.fr.r, st);
                    count++;
                }
                const AttnTokens at{nt, block_floats_, planes_block_, part_stride_};
                if (e == cudaSuccess)
                    e = launch_attend(o.x, kv_[o.kv].k, kv_[o.kv].v, kv_f16_, o.y, part_, att_counters_, sp_multi_, o.attn, o.xp, status_, st, false, nullptr,
                                      &at);
                first = false;
                count++;
                break;
            }
            case B2_OP_GLU:
                for (int tk = 0; tk < nt && e == cudaSuccess; tk++) e = launch_glu(A(o.x, tk), A(o.z, tk), A(o.y, tk), o.n, o.gelu, st, pdl());
                break;
            default: e = cudaErrorInvalidValue;
        }
        if (e != cudaSuccess) {
            err = fmt("[b200qmm: plan: op %zu (kind %u) for %d tokens: %s]", i, o.kind, nt, cudaGetErrorString(e));
            return B2_ERR_CUDA;
        }
    }
    multi_launches_[nt] = count;
    return B2_OK;
}

// Captures [embedding lookup,] ops [, argmax + advance] on `st` (not the legacy stream) into an executable graph.
int DecodePlanImpl::capture(cudaStream_t st, bool with_head, cudaGraphExec_t* out, std::string& err, int nt) {
    PLAN_CUDA(cudaStreamBeginCapture(st, cudaStreamCaptureModeThreadLocal), "cudaStreamBeginCapture");
    int rc = B2_OK;
    cudaError_t e = cudaSuccess;
    if (with_head) e = launch_dequantize(gen_embed_dev_, 0, 1, input_, st, token_);
    if (e == cudaSuccess) rc = nt > 1 ? run_ops_multi(st, nt, err, pdl_) : run_ops(st, err, pdl_, with_head);
    if (e == cudaSuccess && rc == B2_OK && with_head)
        e = launch_argmax(logits_, n_logits_, argmax_val_, argmax_idx_, argmax_counter_, token_, out_tokens_, sp_, st, pdl_);
    cudaGraph_t graph = nullptr;
    cudaError_t e2 = cudaStreamEndCapture(st, &graph);
    if (rc) {
        if (graph) cudaGraphDestroy(graph);
        return rc;
    }
    if (e != cudaSuccess || e2 != cudaSuccess) {
        if (graph) cudaGraphDestroy(graph);
        err = fmt("[b200qmm: plan: capture: %s]", cudaGetErrorString(e != cudaSuccess ? e : e2));
        return B2_ERR_CUDA;
    }
    e = cudaGraphInstantiate(out, graph, 0);
    cudaGraphDestroy(graph);
    PLAN_CUDA(e, "cudaGraphInstantiate");
    return B2_OK;
}

int DecodePlanImpl::check_status(std::string& err) {
    uint32_t s = 0;
    PLAN_CUDA(cudaMemcpy(&s, status_, 4, cudaMemcpyDeviceToHost), "cudaMemcpy(status)");
    if (s) {
        cudaMemset(status_, 0, 4);
        cudaMemset(att_counters_, 0, 4 * n_counters_);  // a CTA that gave up never counted itself
        err = s == 4 ? "[b200qmm: plan: a peer did not arrive at an exchange within the time limit]"
                     : "[b200qmm: plan: an attention kernel's wait on its copy ran into the time limit]";
        return B2_ERR_TIMEOUT;
    }
    return B2_OK;
}

int DecodePlanImpl::step(cudaStream_t st, size_t pos, const float* x, const float* rope_cs, float* hidden, float* logits, std::string& err) {
    if (prefill_) return step_multi(st, pos, 1, x, rope_cs, hidden, logits, err);
    if (!x || (cs_stride_ && !rope_cs) || !hidden) {
        err = "[b200qmm: plan step: x, rope_cs and hidden are required]";
        return B2_ERR_ARG;
    }
    if (pos >= max_len_) {
        err = fmt("[b200qmm: plan step: position %zu is past the %u the caches hold]", pos, max_len_);
        return B2_ERR_ARG;
    }
    if (logits && !n_logits_) {
        err = "[b200qmm: plan step: the graph has no logits]";
        return B2_ERR_ARG;
    }
    if (has_exchange_ && !attached_) {
        err = "[b200qmm: plan step: a tensor-parallel plan needs its peers first (b2_plan_attach_peers)]";
        return B2_ERR_ARG;
    }
    PLAN_CUDA(launch_set_step(sp_, (uint32_t)pos, (uint32_t)pos, 0, nullptr, 0, st), "set_step");
    PLAN_CUDA(cudaMemcpyAsync(input_, x, n_input_ * sizeof(float), cudaMemcpyHostToDevice, st), "cudaMemcpy(x)");
    if (cs_stride_) PLAN_CUDA(cudaMemcpyAsync(rope_table_, rope_cs, cs_stride_ * sizeof(float), cudaMemcpyHostToDevice, st), "cudaMemcpy(rope)");
    PLAN_CUDA(cudaGraphLaunch(step_exec_, st), "cudaGraphLaunch");
    PLAN_CUDA(cudaMemcpyAsync(hidden, hidden_, n_hidden_ * sizeof(float), cudaMemcpyDeviceToHost, st), "cudaMemcpy(hidden)");
    if (logits) PLAN_CUDA(cudaMemcpyAsync(logits, logits_, n_logits_ * sizeof(float), cudaMemcpyDeviceToHost, st), "cudaMemcpy(logits)");
    PLAN_CUDA(cudaStreamSynchronize(st), "step");
    return check_status(err);
}

int DecodePlanImpl::step_multi(cudaStream_t st, size_t pos, size_t t, const float* x, const float* rope_cs, float* hidden, float* logits,
                               std::string& err) {
    if (prefill_) {
        if (logits) {
            err = "[b200qmm: plan step: a prefill plan has no logits]";
            return B2_ERR_ARG;
        }
        return step_prefill(st, pos, t, x, rope_cs, hidden, err);
    }
    if (t == 0 || t > (size_t)tokens_) {
        err = fmt("[b200qmm: plan step: %zu tokens in a step of a plan made for %d]", t, tokens_);
        return B2_ERR_ARG;
    }
    if (t == 1) return step(st, pos, x, rope_cs, hidden, logits, err);  // one row per table: the one-token layout
    if (!x || (cs_stride_ && !rope_cs) || !hidden) {
        err = "[b200qmm: plan step: x, rope_cs and hidden are required]";
        return B2_ERR_ARG;
    }
    if (pos + t > max_len_) {
        err = fmt("[b200qmm: plan step: positions %zu .. %zu are past the %u the caches hold]", pos, pos + t - 1, max_len_);
        return B2_ERR_ARG;
    }
    if (logits && !n_logits_) {
        err = "[b200qmm: plan step: the graph has no logits]";
        return B2_ERR_ARG;
    }
    uint32_t words[16] = {};
    for (size_t tk = 0; tk < t; tk++) {
        words[4 * tk] = (uint32_t)(pos + tk);  // the token's position
        words[4 * tk + 1] = (uint32_t)pos;     // the position of row 0 of the RoPE table
    }
    PLAN_CUDA(cudaMemcpyAsync(sp_multi_, words, 16 * t, cudaMemcpyHostToDevice, st), "cudaMemcpy(step words)");
    PLAN_CUDA(cudaMemcpy2DAsync(input_, block_floats_ * 4, x, (size_t)n_input_ * 4, (size_t)n_input_ * 4, t, cudaMemcpyHostToDevice, st),
              "cudaMemcpy(x)");
    for (size_t i = 0; i + 1 < cs_off_.size(); i++) {  // table i: t rows of cos | sin, behind the rows of the tables ahead of it
        const size_t row = (size_t)(cs_off_[i + 1] - cs_off_[i]) * 4;
        if (row == 0) continue;
        PLAN_CUDA(cudaMemcpy2DAsync(rope_table_ + cs_off_[i], (size_t)cs_stride_ * 4, rope_cs + t * cs_off_[i], row, row, t, cudaMemcpyHostToDevice, st),
                  "cudaMemcpy(rope)");
    }
    PLAN_CUDA(cudaGraphLaunch(multi_exec_[t], st), "cudaGraphLaunch");
    PLAN_CUDA(cudaMemcpy2DAsync(hidden, (size_t)n_hidden_ * 4, hidden_, block_floats_ * 4, (size_t)n_hidden_ * 4, t, cudaMemcpyDeviceToHost, st),
              "cudaMemcpy(hidden)");
    if (logits)
        PLAN_CUDA(cudaMemcpy2DAsync(logits, (size_t)n_logits_ * 4, logits_, block_floats_ * 4, (size_t)n_logits_ * 4, t, cudaMemcpyDeviceToHost, st),
                  "cudaMemcpy(logits)");
    PLAN_CUDA(cudaStreamSynchronize(st), "step");
    return check_status(err);
}

// A prefill step's kernels for t token rows. A product = the rows to f16 (each multiplied by a power of two, taken out again
// by the GEMM's epilogue), then the tensor-core GEMM: straight into the activation rows where it stores, into a scratch
// matrix where it adds to the rows (a row-wise add follows) or is one of a gate / up pair (the activation kernel follows).
int DecodePlanImpl::run_prefill(cudaStream_t st, size_t pos, size_t t, std::string& err) {
    std::vector<GemmPlan*>& plans = gemm_plans_[t];
    const bool build = plans.empty();
    size_t slot = 0;
    uint64_t count = 0;
    const size_t ld = block_floats_;
    const uint32_t rows = (uint32_t)t;
    const float* x16_src = nullptr;  // the vector whose f16 rows the scratch holds
    size_t x16_k = 0;
    auto gemm = [&](const WeightDev& w, float* y, size_t y_ld) -> cudaError_t {
        GemmPlan* gp = nullptr;
        if (build) {
            char msg[256] = {0};
            GemmPeerY py;
            py.ld = y_ld;
            cudaError_t e = gemm_tc_plan_create(w, x16_, t, y, B2_F32, &gp, msg, sizeof msg, 1, nullptr, 0, 0, 1, y_ld != w.n_out ? &py : nullptr);
            if (e != cudaSuccess) {
                err = fmt("[b200qmm: prefill: %s]", msg);
                return e;
            }
            plans.push_back(gp);
        } else {
            gp = plans[slot];
        }
        slot++;
        count++;
        return launch_gemm_tc(gp, w, t, y, B2_F32, gemm_status_, sm_count_, st, unscale_);
    };
    int rc = B2_OK;
    for (size_t i = 0; i < ops_.size() && rc == B2_OK; i++) {
        const Op& o = ops_[i];
        cudaError_t e = cudaSuccess;
        switch (o.kind) {
            case B2_OP_NORM:
                if (o.rows == 1 && norm_rows_supports(o.norm.n, o.x, o.y, o.p0, ld, ld)) {
                    // a product right behind it that reads exactly this vector gets its f16 rows from the norm kernel
                    const Op* nx = i + 1 < ops_.size() ? &ops_[i + 1] : nullptr;
                    const bool feeds = nx && nx->kind == B2_OP_LINEAR && nx->x == o.y && nx->w.n_in == o.norm.n && o.norm.n % 8 == 0;
                    e = launch_norm_rows(o.x, ld, o.y, ld, o.p0, o.norm, rows, feeds ? x16_ : nullptr, unscale_, st);
                    count++;
                    if (feeds) {
                        x16_src = o.y;
                        x16_k = o.norm.n;
                        break;  // (the overlap check below would forget the rows just made)
                    }
                } else if (o.rows == 1) {
                    DecNorm n = o.norm;
                    n.x_stride = n.out_stride = (uint32_t)ld;
                    e = launch_norm(o.x, o.y, o.p0, n, rows, XPlanes{}, st, false);
                    count++;
                } else {
                    for (size_t tk = 0; tk < t && e == cudaSuccess; tk++, count++)
                        e = launch_norm(o.x + tk * ld, o.y + tk * ld, o.p0, o.norm, o.rows, XPlanes{}, st, false);
                }
                if (overlaps_f(o.y, (size_t)(o.rows - 1) * o.norm.out_stride + o.norm.n, x16_src, x16_k)) x16_src = nullptr;
                break;
            case B2_OP_LINEAR: {
                const size_t K = o.w.n_in, n_out = o.w.n_out;
                if (!(x16_src == o.x && x16_k == K)) {
                    e = launch_to_f16(o.x, B2_F32, t, K, x16_, unscale_, st, 0, ld);
                    count++;
                    x16_src = o.x;
                    x16_k = K;
                }
                if (e != cudaSuccess) break;
                if (o.pair) {
                    e = gemm(o.w, tmp_a_, n_out);
                    if (e == cudaSuccess) e = gemm(o.w2, tmp_b_, n_out);
                    // a product right behind the pair that reads exactly its output gets its f16 rows from the activation kernel
                    // (both GEMMs above have read the scratch rows by then: the kernel is an ordinary launch behind them)
                    const Op* nx = i + 1 < ops_.size() ? &ops_[i + 1] : nullptr;
                    const bool feeds = nx && nx->kind == B2_OP_LINEAR && nx->x == o.y && nx->w.n_in == n_out && glu_rows_f16_supports((uint32_t)n_out);
                    if (e == cudaSuccess)
                        e = launch_glu_rows(tmp_a_, n_out, tmp_b_, n_out, o.y, ld, (uint32_t)n_out, rows, o.mode == B2_MODE_GELU_PAIR, st,
                                            feeds ? x16_ : nullptr, unscale_);
                    count++;
                    if (feeds && e == cudaSuccess) {
                        x16_src = o.y;
                        x16_k = n_out;
                        break;  // (the overlap check below would forget the rows just made)
                    }
                } else if (o.mode == B2_MODE_STORE && ((uintptr_t)o.y & 15) == 0) {
                    e = gemm(o.w, o.y, ld);
                } else {
                    // (a product that adds goes through the scratch matrix: its dense rows let the GEMM pick its widest tiles, which
                    // the strided destination's copy-engine stores cannot take; measured 63 + 13 us against 95 us at 4096 x 4096)
                    e = gemm(o.w, tmp_a_, n_out);
                    if (e == cudaSuccess) e = launch_rows_op(o.y, ld, tmp_a_, n_out, (uint32_t)n_out, rows, o.mode == B2_MODE_ADD, st);
                    count++;
                }
                if (overlaps_f(o.y, n_out, x16_src, x16_k)) x16_src = nullptr;
                break;
            }
            case B2_OP_QK_ROPE:
                e = launch_qk_rope_rows(o.x, o.y, ld, rows, kv_[o.kv].k, kv_[o.kv].v, kv_f16_, o.p0, o.p1, rope_table_, sp_, o.rope, st);
                count++;
                if (overlaps_f(o.y, (size_t)o.rope.nh * o.rope.hd, x16_src, x16_k)) x16_src = nullptr;
                break;
            case B2_OP_ATTEND:
                if (loop_attend_) {
                    for (size_t tk = 0; tk < t && e == cudaSuccess; tk++, count++)
                        e = launch_attend(o.x + tk * ld, kv_[o.kv].k, kv_[o.kv].v, kv_f16_, o.y + tk * ld, part_, att_counters_, sp_multi_ + 4 * tk, o.attn,
                                          XPlanes{}, status_, st, false, nullptr);
                } else {
                    e = launch_attend_rows(o.x, o.y, ld, rows, kv_[o.kv].k, kv_[o.kv].v, kv_f16_, kv16_, (uint32_t)(pos + t), sp_, o.attn, st);
                    count += kv_f16_ ? 1 : 3;
                }
                if (overlaps_f(o.y, (size_t)o.attn.nh * o.attn.hd, x16_src, x16_k)) x16_src = nullptr;
                break;
            case B2_OP_GLU:
                if (o.n % 4 == 0 && (((uintptr_t)o.x | (uintptr_t)o.y | (uintptr_t)o.z) & 15) == 0) {
                    e = launch_glu_rows(o.x, ld, o.z, ld, o.y, ld, o.n, rows, o.gelu, st);
                    count++;
                } else {
                    for (size_t tk = 0; tk < t && e == cudaSuccess; tk++, count++)
                        e = launch_glu(o.x + tk * ld, o.z + tk * ld, o.y + tk * ld, o.n, o.gelu, st, false);
                }
                if (overlaps_f(o.y, o.n, x16_src, x16_k)) x16_src = nullptr;
                break;
            default: e = cudaErrorInvalidValue;
        }
        if (e != cudaSuccess) {
            if (err.empty()) err = fmt("[b200qmm: prefill: op %zu (kind %u) for %zu tokens: %s]", i, o.kind, t, cudaGetErrorString(e));
            rc = B2_ERR_CUDA;
        }
    }
    if (rc != B2_OK && build) {  // a half-made list must not be found again
        for (GemmPlan* gp : plans) gemm_tc_plan_destroy(gp);
        gemm_plans_.erase(t);
    }
    prefill_launches_ = count;
    return rc;
}

int DecodePlanImpl::step_prefill(cudaStream_t st, size_t pos, size_t t, const float* x, const float* rope_cs, float* hidden, std::string& err) {
    if (!x || (cs_stride_ && !rope_cs) || !hidden) {
        err = "[b200qmm: plan step: x, rope_cs and hidden are required]";
        return B2_ERR_ARG;
    }
    if (t == 0 || t > (size_t)tokens_ || pos + t > max_len_) {
        err = fmt("[b200qmm: plan step: %zu tokens from position %zu: the plan takes %d per step and its caches hold %u positions]", t, pos, tokens_,
                  max_len_);
        return B2_ERR_ARG;
    }
    err.clear();
    PLAN_CUDA(launch_set_step(sp_, (uint32_t)pos, (uint32_t)pos, 0, nullptr, 0, st), "set_step");
    if (loop_attend_) {
        std::vector<uint32_t> words(4 * t, 0u);
        for (size_t tk = 0; tk < t; tk++) {
            words[4 * tk] = (uint32_t)(pos + tk);
            words[4 * tk + 1] = (uint32_t)pos;
        }
        PLAN_CUDA(cudaMemcpyAsync(sp_multi_, words.data(), 16 * t, cudaMemcpyHostToDevice, st), "cudaMemcpy(step words)");
        PLAN_CUDA(cudaStreamSynchronize(st), "step words");
    }
    PLAN_CUDA(cudaMemcpy2DAsync(input_, block_floats_ * 4, x, (size_t)n_input_ * 4, (size_t)n_input_ * 4, t, cudaMemcpyHostToDevice, st),
              "cudaMemcpy(x)");
    for (size_t i = 0; i + 1 < cs_off_.size(); i++) {
        const size_t row = (size_t)(cs_off_[i + 1] - cs_off_[i]) * 4;
        if (row == 0) continue;
        PLAN_CUDA(cudaMemcpy2DAsync(rope_table_ + cs_off_[i], (size_t)cs_stride_ * 4, rope_cs + t * cs_off_[i], row, row, t, cudaMemcpyHostToDevice, st),
                  "cudaMemcpy(rope)");
    }
    PLAN_CUDA(cudaEventRecord(ev0_, st), "cudaEventRecord");
    int rc = run_prefill(st, pos, t, err);
    if (rc) {
        cudaStreamSynchronize(st);
        return rc;
    }
    PLAN_CUDA(cudaEventRecord(ev1_, st), "cudaEventRecord");
    PLAN_CUDA(cudaMemcpy2DAsync(hidden, (size_t)n_hidden_ * 4, hidden_, block_floats_ * 4, (size_t)n_hidden_ * 4, t, cudaMemcpyDeviceToHost, st),
              "cudaMemcpy(hidden)");
    PLAN_CUDA(cudaStreamSynchronize(st), "step");
    PLAN_CUDA(cudaEventElapsedTime(&last_ms_, ev0_, ev1_), "cudaEventElapsedTime");
    GemmStatus gs{};
    PLAN_CUDA(cudaMemcpy(&gs, gemm_status_, sizeof gs, cudaMemcpyDeviceToHost), "cudaMemcpy(GEMM status)");
    if (gs.code) {
        cudaMemset(gemm_status_, 0, sizeof gs);
        err = fmt("[b200qmm: prefill: a GEMM's bounded wait %u gave up in CTA %u]", gs.where, gs.cta);
        return B2_ERR_TIMEOUT;
    }
    return check_status(err);
}

int DecodePlanImpl::kv_write(cudaStream_t st, uint32_t kv, size_t pos0, size_t n, const float* k, const float* v, std::string& err) {
    if (kv >= kv_.size() || !k || !v || pos0 + n > max_len_) {
        err = "[b200qmm: plan kv_write: bad cache index, pointers or range]";
        return B2_ERR_ARG;
    }
    const Kv& c = kv_[kv];
    const size_t row = (size_t)c.nkv * c.hd, chunk = stage_floats_ / row;
    for (size_t at = 0; at < n; at += chunk) {
        size_t m = std::min(chunk, n - at);
        PLAN_CUDA(cudaMemcpyAsync(stage_, k + at * row, m * row * 4, cudaMemcpyHostToDevice, st), "cudaMemcpy(K rows)");
        PLAN_CUDA(cudaMemcpyAsync(stage_ + stage_floats_, v + at * row, m * row * 4, cudaMemcpyHostToDevice, st), "cudaMemcpy(V rows)");
        PLAN_CUDA(launch_kv_rows(stage_, c.k, kv_f16_, true, c.nkv, c.hd, max_len_, (uint32_t)(pos0 + at), (uint32_t)m, st), "kv_rows");
        PLAN_CUDA(launch_kv_rows(stage_ + stage_floats_, c.v, kv_f16_, true, c.nkv, c.hd, max_len_, (uint32_t)(pos0 + at), (uint32_t)m, st),
                  "kv_rows");
        PLAN_CUDA(cudaStreamSynchronize(st), "kv_write");  // the host rows may be pageable: the staging buffer is reused next round
    }
    return B2_OK;
}

int DecodePlanImpl::kv_read(cudaStream_t st, uint32_t kv, size_t pos0, size_t n, float* k, float* v, std::string& err) {
    if (kv >= kv_.size() || !k || !v || pos0 + n > max_len_) {
        err = "[b200qmm: plan kv_read: bad cache index, pointers or range]";
        return B2_ERR_ARG;
    }
    const Kv& c = kv_[kv];
    const size_t row = (size_t)c.nkv * c.hd, chunk = stage_floats_ / row;
    for (size_t at = 0; at < n; at += chunk) {
        size_t m = std::min(chunk, n - at);
        PLAN_CUDA(launch_kv_rows(stage_, c.k, kv_f16_, false, c.nkv, c.hd, max_len_, (uint32_t)(pos0 + at), (uint32_t)m, st), "kv_rows");
        PLAN_CUDA(launch_kv_rows(stage_ + stage_floats_, c.v, kv_f16_, false, c.nkv, c.hd, max_len_, (uint32_t)(pos0 + at), (uint32_t)m, st),
                  "kv_rows");
        PLAN_CUDA(cudaMemcpyAsync(k + at * row, stage_, m * row * 4, cudaMemcpyDeviceToHost, st), "cudaMemcpy(K rows)");
        PLAN_CUDA(cudaMemcpyAsync(v + at * row, stage_ + stage_floats_, m * row * 4, cudaMemcpyDeviceToHost, st), "cudaMemcpy(V rows)");
        PLAN_CUDA(cudaStreamSynchronize(st), "kv_read");
    }
    return B2_OK;
}

int DecodePlanImpl::generate(cudaStream_t st, uint64_t embed_handle, const WeightDev& embed, int32_t first_token, size_t pos0, size_t n_tokens,
                             const float* rope_cs_table, int32_t* out_tokens, float* elapsed_ms, std::string& err) {
    if (!n_logits_ || !logits_) {
        err = "[b200qmm: plan generate: the graph has no logits]";
        return B2_ERR_ARG;
    }
    if (!out_tokens || (cs_stride_ && !rope_cs_table) || n_tokens == 0 || pos0 + n_tokens > max_len_) {
        err = fmt("[b200qmm: plan generate: %zu tokens from position %zu do not fit the %u positions of the caches, or a pointer is missing]",
                  n_tokens, pos0, max_len_);
        return B2_ERR_ARG;
    }
    if (has_exchange_ && !attached_) {
        err = "[b200qmm: plan generate: a tensor-parallel plan needs its peers first (b2_plan_attach_peers)]";
        return B2_ERR_ARG;
    }
    if (embed.n_in != n_input_ || first_token < 0 || (size_t)first_token >= embed.n_out) {
        err = "[b200qmm: plan generate: the embedding matrix does not match the graph's input, or the token is outside it]";
        return B2_ERR_ARG;
    }
    if (!gen_exec_ || gen_embed_ != embed_handle || gen_embed_dev_.p0 != embed.p0) {
        if (gen_exec_) cudaGraphExecDestroy(gen_exec_);
        gen_exec_ = nullptr;
        gen_embed_ = embed_handle;
        gen_embed_dev_ = embed;
        // the two kernels the step graph does not have, once outside a capture
        PLAN_CUDA(launch_set_step(sp_, 0, 0, 0, token_, first_token, cap_stream_), "set_step");
        PLAN_CUDA(launch_dequantize(embed, 0, 1, input_, cap_stream_, token_), "embedding lookup");
        PLAN_CUDA(launch_argmax(logits_, n_logits_, argmax_val_, argmax_idx_, argmax_counter_, token_, out_tokens_, sp_, cap_stream_), "argmax");
        PLAN_CUDA(cudaStreamSynchronize(cap_stream_), "generate warm-up");
        int rc = capture(cap_stream_, true, &gen_exec_, err);
        if (rc) return rc;
    }
    PLAN_CUDA(launch_set_step(sp_, (uint32_t)pos0, (uint32_t)pos0, 0, token_, first_token, st), "set_step");
    if (cs_stride_)
        PLAN_CUDA(cudaMemcpyAsync(rope_table_, rope_cs_table, n_tokens * cs_stride_ * sizeof(float), cudaMemcpyHostToDevice, st), "cudaMemcpy(rope)");
    PLAN_CUDA(cudaEventRecord(ev0_, st), "cudaEventRecord");
    for (size_t i = 0; i < n_tokens; i++) PLAN_CUDA(cudaGraphLaunch(gen_exec_, st), "cudaGraphLaunch");
    PLAN_CUDA(cudaEventRecord(ev1_, st), "cudaEventRecord");
    PLAN_CUDA(cudaMemcpyAsync(out_tokens, out_tokens_, n_tokens * sizeof(int), cudaMemcpyDeviceToHost, st), "cudaMemcpy(tokens)");
    PLAN_CUDA(cudaStreamSynchronize(st), "generate");
    if (elapsed_ms) PLAN_CUDA(cudaEventElapsedTime(elapsed_ms, ev0_, ev1_), "cudaEventElapsedTime");
    return check_status(err);
}


// ---- tensor-parallel plans: peers ------------------------------------------------------------------------------------
int DecodePlanImpl::export_handle(void* out128, std::string& err) {
    if (!has_exchange_) {
        err = "[b200qmm: plan export: the graph has no exchange op]";
        return B2_ERR_ARG;
    }
    cudaIpcMemHandle_t h[2];
    static_assert(sizeof h == B2_PLAN_HANDLE_BYTES, "handle size");
    PLAN_CUDA(cudaIpcGetMemHandle(&h[0], bufs_), "cudaIpcGetMemHandle(buffers)");
    PLAN_CUDA(cudaIpcGetMemHandle(&h[1], xflags_), "cudaIpcGetMemHandle(flags)");
    memcpy(out128, h, sizeof h);
    return B2_OK;
}

int DecodePlanImpl::attach_peers(uint32_t rank, uint32_t world, const void* handles, std::string& err) {
    if (!has_exchange_ || attached_ || world < 2 || world > 8 || rank >= world || !handles) {
        err = "[b200qmm: plan attach: needs a graph with exchange ops, 2 to 8 ranks, and is done once]";
        return B2_ERR_ARG;
    }
    peers_.rank = rank;
    peers_.world = world;
    for (uint32_t p = 0; p < world; p++) {
        if (p == rank) {
            peers_.base[p] = bufs_;
            peers_.flags[p] = xflags_;
            continue;
        }
        cudaIpcMemHandle_t h[2];
        memcpy(h, (const char*)handles + (size_t)p * B2_PLAN_HANDLE_BYTES, sizeof h);
        void *b = nullptr, *f = nullptr;
        PLAN_CUDA(cudaIpcOpenMemHandle(&b, h[0], cudaIpcMemLazyEnablePeerAccess), "cudaIpcOpenMemHandle(buffers)");
        peer_maps_.push_back(b);
        PLAN_CUDA(cudaIpcOpenMemHandle(&f, h[1], cudaIpcMemLazyEnablePeerAccess), "cudaIpcOpenMemHandle(flags)");
        peer_maps_.push_back(f);
        peers_.base[p] = (float*)b;
        peers_.flags[p] = (uint32_t*)f;
    }
    attached_ = true;
    // Which exchanges need the meeting before the writes: those with a kernel, since the previous exchange, that reads
    // the vector outside this rank's own part (the first exchange of the list always meets: its predecessors are the
    // previous step's kernels).
    {
        auto reads_outside = [&](const float* a, size_t na, const Op& ex) {
            if (!a || na == 0) return false;
            const float* v = ex.x;
            const size_t part = ex.n / world;
            const float* own = v + (size_t)rank * part;
            if (!(a < v + ex.n && v < a + na)) return false;  // does not touch the vector
            return !(a >= own && a + na <= own + part);        // touches it outside the own part
        };
        bool first = true;
        for (size_t i = 0; i < ops_.size(); i++) {
            if (ops_[i].kind != B2_OP_EXCHANGE) continue;
            Op& ex = ops_[i];
            bool need = first;
            first = false;
            for (size_t b = i; b-- > 0 && !need;) {
                const Op& o = ops_[b];
                if (o.kind == B2_OP_EXCHANGE) break;
                switch (o.kind) {
                    case B2_OP_LINEAR:
                        if (o.w.fmt == B2_FMT_F8E4M3) need = reads_outside(o.x, o.w.n_in, ex);
                        if (o.mode != B2_MODE_STORE && !o.pair) need = need || reads_outside(o.y, o.w.n_out, ex);
                        need = need || reads_outside(o.z, 1, ex);
                        break;
                    case B2_OP_NORM:
                    case OP_NORM_DEFERRED: need = reads_outside(o.x, (size_t)(o.rows - 1) * o.norm.x_stride + o.norm.n, ex); break;
                    case OP_XPLANES: need = reads_outside(o.x, o.n, ex); break;
                    case B2_OP_GLU: need = reads_outside(o.x, o.n, ex) || reads_outside(o.z, o.n, ex); break;
                    case B2_OP_QK_ROPE: need = reads_outside(o.x, (size_t)o.rope.v_off + (size_t)o.rope.nkv * o.rope.hd + (size_t)o.rope.nh * o.rope.q_stride, ex); break;
                    case B2_OP_ATTEND: need = reads_outside(o.x, (size_t)o.attn.nh * o.attn.hd, ex); break;
                    default: need = true;
                }
            }
            ex.meet_first = need;
        }
    }
    // the step graph captured at creation has no exchange nodes: capture it again
    if (step_exec_) cudaGraphExecDestroy(step_exec_);
    step_exec_ = nullptr;
    return capture(cap_stream_, false, &step_exec_, err);
}

}  // namespace b2
