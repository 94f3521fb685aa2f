// Host side of the engine: a C++ mirror of oxinfer's `gpu::Backend` trait for CUDA
// (src/gpu.rs:151-294, implemented by CudaBackend in src/cuda.rs) and the C ABI over it
// (include/b200qmm.h). Same method names, argument meaning and error behaviour: a call either does
// all of its work or none of it, and reports "declined" so that the caller can run the batch on the
// CPU (src/gpu.rs:158-160, src/model.rs:875-886).
#include <chrono>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <string>
#include <unordered_map>
#include <vector>

#include "dq_other.cuh"
#include "kernels.h"
#include "nccl_dyn.h"
#include "plan.h"

namespace b2 {

struct Weight {
    WeightDev dev{};
    std::vector<void*> owned;  // device allocations freed with the weight (empty for row shards)
    size_t bytes = 0;
};

// A device buffer that only grows.
// Device state of the routed experts of one MoE layer (Backend::upload_moe, src/gpu.rs:200-215): the
// experts' fused gate/up matrices stacked into one buffer, and their down matrices into another.
struct Moe {
    int fmt = 0;
    size_t experts = 0, h = 0, inter = 0;
    int act = B2_ACT_SILU;   // MoeAct
    float act_limit = 0.0f;  // SiluClamp's limit
    void* gate_up = nullptr;  // [experts][2 inter][h / 256][144]
    void* down = nullptr;     // [experts][h][inter / 256][144]
    size_t bytes = 0;
};

struct Scratch {
    void* p = nullptr;
    size_t cap = 0;
    cudaError_t reserve(size_t n) {
        if (n <= cap) return cudaSuccess;
        if (p) cudaFree(p);
        p = nullptr;
        cap = 0;
        size_t want = (n + (1u << 20) - 1) & ~(size_t)((1u << 20) - 1);
        cudaError_t e = cudaMalloc(&p, want);
        if (e == cudaSuccess) cap = want;
        return e;
    }
    void release() {
        if (p) cudaFree(p);
        p = nullptr;
        cap = 0;
    }
};

class Backend {
  public:
    int device = 0;
    int sm_count = 148;
    cudaStream_t stream = nullptr;
    bool chained = false;  // b2_set_chained
    bool exact = false;    // b2_set_exact
    bool fast_planes = false;  // b2_set_fast_planes
    bool fp8_act = false;  // b2_set_fp8_activations
    std::mutex mu;  // calls serialize, like the staging lock of src/cuda.rs:430,1443
    std::string err;
    std::string stats_text;
    std::unordered_map<uint64_t, Weight> weights;
    std::unordered_map<uint64_t, Moe> moes;
    std::unordered_map<uint64_t, DecodePlanImpl*> decode_plans;
    Scratch moe_idx, moe_xg, moe_g, moe_a, moe_o;
    // tensor / expert parallel (b2_comm_init): this process's rank in a group of `world` processes, one GPU each
    NcclComm comm = nullptr;
    int world = 1, rank = 0;
    Scratch tp_stage, tp_gather, ep_idx, ep_send, ep_recv, ep_out, ep_back;
    uint64_t next_handle = 1;
    uint64_t launches = 0;
    // staging for the host-buffer entry points
    Scratch x_dev, y_dev, x16, x8, xplanes, pair_tmp;
    GemmStatus* gemm_status = nullptr;  // device
    // cached tensor maps of the tensor-core GEMM (see matmul_dev)
    std::vector<GemmPlan*> plans;
    // cumulative times, like Backend::stats (src/cuda.rs:403-409)
    double ns_in = 0, ns_gpu = 0, ns_out = 0;
    uint64_t calls = 0;

    int fail(int code, const char* fmt, ...) {
        char buf[512];
        va_list ap;
        va_start(ap, fmt);
        vsnprintf(buf, sizeof buf, fmt, ap);
        va_end(ap);
        err = buf;
        return code;
    }
    int cuda_fail(cudaError_t e, const char* what) {
        return fail(e == cudaErrorMemoryAllocation ? B2_ERR_NOMEM : B2_ERR_CUDA, "[b200qmm: %s: %s]", what, cudaGetErrorString(e));
    }
    bool bind() { return cudaSetDevice(device) == cudaSuccess; }

    Weight* find(uint64_t h) {
        auto it = weights.find(h);
        return it == weights.end() ? nullptr : &it->second;
    }

    // ---- Backend::wants (src/cuda.rs:1134-1136): the reference offers a matmul to CUDA from 32 tokens
    // and 1 GFLOP up, n_out % 64 == 0, n_in % 32 == 0. Here every supported shape is worth it (the
    // weights are resident and a B200 GEMV outruns the host cores by two orders of magnitude), so the
    // only conditions are the kernels' shape rules.
    bool wants(size_t n_out, size_t n_in, size_t t) const { return t >= 1 && n_out >= 1 && n_in % 32 == 0; }

    // The planes record at `base` as the products of this context read it: all three planes, or the upper two under
    // b2_set_fast_planes (never under the exactness switch).
    int planes_read() const { return fast_planes && !exact ? 2 : 3; }
    XPlanes planes_at(void* base, size_t K) const {
        XPlanes p = xplanes_at(base, K);
        p.np = planes_read();
        return p;
    }
    int alloc_copy(const void* host, size_t bytes, void** out, std::vector<void*>& owned) {
        void* p = nullptr;
        cudaError_t e = cudaMalloc(&p, bytes ? bytes : 16);
        if (e != cudaSuccess) return cuda_fail(e, "cudaMalloc(weight)");
        owned.push_back(p);
        if (host && bytes) {
            e = cudaMemcpyAsync(p, host, bytes, cudaMemcpyHostToDevice, stream);
            if (e != cudaSuccess) return cuda_fail(e, "cudaMemcpy(weight)");
        }
        *out = p;
        return B2_OK;
    }
    void drop(std::vector<void*>& owned) {
        for (void* p : owned) cudaFree(p);
        owned.clear();
    }

    // ---- Backend::upload (src/cuda.rs:640-699)
    int upload_mlx4(const uint32_t* w, const uint16_t* scales, const uint16_t* biases, size_t n_out, size_t n_in, size_t group,
                    uint64_t* out) {
        if (!w || !scales || !biases || !out) return fail(B2_ERR_ARG, "[b200qmm: upload_mlx4: null argument]");
        if (group != 64 || n_in % 256 != 0 || n_out == 0)
            return fail(B2_DECLINED, "[b200qmm: upload_mlx4: group must be 64 and n_in a multiple of 256]");
        // The triple is repacked on the device into Q4_K-shaped blocks (formats.cuh): same bytes per weight,
        // and every 4-bit kernel then serves both formats. The reference repacks too (from_mlx_q4).
        Weight wt;
        std::vector<void*> tmp;
        void *p0, *p1, *p2, *blocks;
        int rc;
        size_t nb = n_out * (n_in / 256);
        if ((rc = alloc_copy(w, n_out * n_in / 2, &p0, tmp)) || (rc = alloc_copy(scales, n_out * (n_in / 64) * 2, &p1, tmp)) ||
            (rc = alloc_copy(biases, n_out * (n_in / 64) * 2, &p2, tmp)) || (rc = alloc_copy(nullptr, nb * 144, &blocks, wt.owned))) {
            drop(tmp);
            drop(wt.owned);
            return rc;
        }
        cudaError_t e = launch_repack_mlx4((const uint32_t*)p0, (const uint16_t*)p1, (const uint16_t*)p2, n_out, n_in, (uint8_t*)blocks, stream);
        launches++;
        if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
        drop(tmp);
        if (e != cudaSuccess) {
            drop(wt.owned);
            return cuda_fail(e, "repack_mlx4");
        }
        wt.dev.fmt = B2_FMT_MLX4;
        wt.dev.n_out = n_out;
        wt.dev.n_in = n_in;
        wt.dev.group = group;
        wt.dev.p0 = (const uint8_t*)blocks;
        wt.bytes = nb * 144;
        *out = next_handle++;
        weights[*out] = std::move(wt);
        return B2_OK;
    }

    // ---- Backend::upload for WeightRef::Q4(&Q4Matrix) with offsets (src/gpu.rs:15-21, src/cuda.rs:640-699): the layout the
    // reference's loader hands a backend (src/quant.rs:427-440), i.e. what from_mlx_q4 made of an MLX checkpoint. Produces the
    // same device blocks as upload_mlx4 does from the on-disk triple.
    int upload_q4(const uint8_t* q, const uint16_t* scales, const uint16_t* offsets, size_t group, size_t n_out, size_t n_in, uint64_t* out) {
        if (!q || !scales || !out) return fail(B2_ERR_ARG, "[b200qmm: upload_q4: null argument]");
        if (!offsets) {
            // A plain Q4 matrix (--quant q4: one f16 scale per 32 weights, w = (nibble - 8) * scale, src/quant.rs:427-440) holds
            // what GGUF Q4_0 blocks hold, in two arrays: interleaved into 18-byte blocks it runs through the generic kernels.
            if (n_in % 32 != 0 || n_out == 0) return fail(B2_DECLINED, "[b200qmm: upload_q4: n_in must be a multiple of 32]");
            const size_t nb32 = n_out * (n_in / 32);
            std::vector<uint8_t> blocks(nb32 * 18);
            for (size_t b = 0; b < nb32; b++) {
                blocks[b * 18] = (uint8_t)(scales[b] & 0xff);
                blocks[b * 18 + 1] = (uint8_t)(scales[b] >> 8);
                std::memcpy(&blocks[b * 18 + 2], q + b * 16, 16);
            }
            return upload_gguf(B2_FMT_Q4_0, blocks.data(), n_out, n_in, nullptr, 0, 0, out);
        }
        if (group == 0 || group % 64 != 0 || n_in % 256 != 0 || n_in % group != 0 || n_out == 0)
            return fail(B2_DECLINED, "[b200qmm: upload_q4: the offsets' group must be a multiple of 64 dividing n_in, and n_in a multiple of 256]");
        Weight wt;
        std::vector<void*> tmp;
        void *p0, *p1, *p2, *flag, *blocks;
        int rc;
        const size_t nb = n_out * (n_in / 256);
        if ((rc = alloc_copy(q, n_out * n_in / 2, &p0, tmp)) || (rc = alloc_copy(scales, n_out * (n_in / 32) * 2, &p1, tmp)) ||
            (rc = alloc_copy(offsets, n_out * (n_in / group) * 2, &p2, tmp)) || (rc = alloc_copy(nullptr, 4, &flag, tmp)) ||
            (rc = alloc_copy(nullptr, nb * 144, &blocks, wt.owned))) {
            drop(tmp);
            drop(wt.owned);
            return rc;
        }
        int mismatch = 0;
        cudaError_t e = cudaMemsetAsync(flag, 0, 4, stream);
        if (e == cudaSuccess) e = launch_repack_q4a((const uint8_t*)p0, (const uint16_t*)p1, (const uint16_t*)p2, n_out, n_in, group, (uint8_t*)blocks, (int*)flag, stream);
        launches++;
        if (e == cudaSuccess) e = cudaMemcpyAsync(&mismatch, flag, 4, cudaMemcpyDeviceToHost, stream);
        if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
        drop(tmp);
        if (e != cudaSuccess || mismatch) {
            drop(wt.owned);
            if (e != cudaSuccess) return cuda_fail(e, "repack_q4a");
            return fail(B2_DECLINED, "[b200qmm: upload_q4: the two 32-blocks of a 64-group differ in scale (not a matrix from_mlx_q4 made)]");
        }
        wt.dev.fmt = B2_FMT_MLX4;
        wt.dev.n_out = n_out;
        wt.dev.n_in = n_in;
        wt.dev.group = 64;
        wt.dev.p0 = (const uint8_t*)blocks;
        wt.bytes = nb * 144;
        *out = next_handle++;
        weights[*out] = std::move(wt);
        return B2_OK;
    }

    int upload_gguf(int fmt, const uint8_t* data, size_t n_out, size_t n_in, const float* bscales, size_t bs_rows, size_t bs_cols,
                    uint64_t* out) {
        if (!data || !out || n_out == 0) return fail(B2_ERR_ARG, "[b200qmm: upload_gguf: null argument]");
        Weight wt;
        wt.dev.fmt = fmt;
        wt.dev.n_out = n_out;
        wt.dev.n_in = n_in;
        int rc = B2_OK;
        cudaError_t e = cudaSuccess;
        if (fmt == B2_FMT_Q4_K) {
            if (n_in % 256) return fail(B2_DECLINED, "[b200qmm: Q4_K needs n_in %% 256 == 0]");
            void* p;
            wt.bytes = n_out * (n_in / 256) * 144;
            if ((rc = alloc_copy(data, wt.bytes, &p, wt.owned))) return rc;
            wt.dev.p0 = (const uint8_t*)p;
        } else if (fmt == B2_FMT_Q6_K) {
            if (n_in % 256) return fail(B2_DECLINED, "[b200qmm: Q6_K needs n_in %% 256 == 0]");
            size_t nb = n_out * (n_in / 256);
            wt.bytes = nb * 210;
            std::vector<void*> tmp;
            void *raw, *ql, *qh, *sc, *d;
            if ((rc = alloc_copy(data, nb * 210, &raw, tmp)) || (rc = alloc_copy(nullptr, nb * 128, &ql, wt.owned)) ||
                (rc = alloc_copy(nullptr, nb * 64, &qh, wt.owned)) || (rc = alloc_copy(nullptr, nb * 16, &sc, wt.owned)) ||
                (rc = alloc_copy(nullptr, nb * 2, &d, wt.owned))) {
                drop(tmp);
                drop(wt.owned);
                return rc;
            }
            e = launch_repack_q6k((const uint8_t*)raw, n_out, n_in, (uint8_t*)ql, (uint8_t*)qh, (int8_t*)sc, (uint16_t*)d, stream);
            launches++;
            if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
            drop(tmp);
            if (e != cudaSuccess) {
                drop(wt.owned);
                return cuda_fail(e, "repack_q6k");
            }
            wt.dev.p0 = (const uint8_t*)ql;
            wt.dev.p1 = (const uint8_t*)qh;
            wt.dev.p2 = (const uint8_t*)sc;
            wt.dev.p3 = (const uint8_t*)d;
        } else if (fmt == B2_FMT_Q8_0) {
            if (n_in % 32) return fail(B2_DECLINED, "[b200qmm: Q8_0 needs n_in %% 32 == 0]");
            size_t nb = n_out * (n_in / 32);
            wt.bytes = nb * 34;
            std::vector<void*> tmp;
            void *raw, *qs, *d;
            if ((rc = alloc_copy(data, nb * 34, &raw, tmp)) || (rc = alloc_copy(nullptr, nb * 32, &qs, wt.owned)) ||
                (rc = alloc_copy(nullptr, nb * 2, &d, wt.owned))) {
                drop(tmp);
                drop(wt.owned);
                return rc;
            }
            e = launch_repack_q8_0((const uint8_t*)raw, n_out, n_in, (int8_t*)qs, (uint16_t*)d, stream);
            launches++;
            if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
            drop(tmp);
            if (e != cudaSuccess) {
                drop(wt.owned);
                return cuda_fail(e, "repack_q8_0");
            }
            wt.dev.p0 = (const uint8_t*)qs;
            wt.dev.p1 = (const uint8_t*)d;
        } else if (fmt == B2_FMT_F8E4M3) {
            if (n_in % 16) return fail(B2_DECLINED, "[b200qmm: F8E4M3 needs n_in %% 16 == 0]");
            void* p;
            wt.bytes = n_out * n_in;
            if ((rc = alloc_copy(data, n_out * n_in, &p, wt.owned))) return rc;
            wt.dev.p0 = (const uint8_t*)p;
            if (bscales) {
                if (!bs_rows || !bs_cols) {
                    drop(wt.owned);
                    return fail(B2_ERR_ARG, "[b200qmm: F8E4M3 block scales need bs_rows, bs_cols > 0]");
                }
                size_t ncb = (n_in + bs_cols - 1) / bs_cols, nrb = (n_out + bs_rows - 1) / bs_rows;
                void* s;
                if ((rc = alloc_copy(bscales, ncb * nrb * 4, &s, wt.owned))) {
                    drop(wt.owned);
                    return rc;
                }
                wt.dev.p1 = (const uint8_t*)s;
                wt.dev.bs_rows = bs_rows;
                wt.dev.bs_cols = bs_cols;
                wt.dev.bs_ncb = ncb;
                wt.bytes += ncb * nrb * 4;
            }
        } else if (fmt_is_other(fmt)) {
            // the other GGUF block formats stay as they are in the file (raw rows) and run through the generic kernels
            if (n_in % other_block_size(fmt) || n_in % 32) return fail(B2_DECLINED, "[b200qmm: format %d needs n_in to be a multiple of its block size]", fmt);
            void* p;
            wt.bytes = n_out * other_row_bytes(fmt, n_in);
            // 16 bytes of room after the last row: the matrix-vector kernel reads whole aligned 16-byte words
            if ((rc = alloc_copy(nullptr, wt.bytes + 16, &p, wt.owned))) return rc;
            if ((e = cudaMemcpyAsync(p, data, wt.bytes, cudaMemcpyHostToDevice, stream)) != cudaSuccess || (e = cudaStreamSynchronize(stream)) != cudaSuccess) {
                drop(wt.owned);
                return cuda_fail(e, "upload copy");
            }
            if (bscales) {  // NVFP4's global scale: one value for the whole matrix
                if (fmt != B2_FMT_NVFP4 || bs_rows < n_out || bs_cols < n_in) {
                    drop(wt.owned);
                    return fail(B2_DECLINED, "[b200qmm: upload_gguf: block scales on this format must be one scale for the whole NVFP4 matrix]");
                }
                void* gs;
                if ((rc = alloc_copy(bscales, 4, &gs, wt.owned))) {
                    drop(wt.owned);
                    return rc;
                }
                if ((e = cudaStreamSynchronize(stream)) != cudaSuccess) {
                    drop(wt.owned);
                    return cuda_fail(e, "upload copy");
                }
                wt.dev.p1 = (const uint8_t*)gs;
            }
            wt.dev.p0 = (const uint8_t*)p;
        } else {
            return fail(B2_DECLINED, "[b200qmm: format %d has no device kernels]", fmt);
        }
        cudaStreamSynchronize(stream);
        *out = next_handle++;
        weights[*out] = std::move(wt);
        return B2_OK;
    }

    int shard_rows(uint64_t h, size_t r0, size_t r1, uint64_t* out) {
        Weight* w = find(h);
        if (!w || !out) return fail(B2_ERR_ARG, "[b200qmm: shard_rows: unknown weight]");
        if (r0 >= r1 || r1 > w->dev.n_out) return fail(B2_ERR_ARG, "[b200qmm: shard_rows: bad row range]");
        Weight s;
        s.dev = w->dev;
        s.dev.n_out = r1 - r0;
        size_t K = w->dev.n_in;
        switch (w->dev.fmt) {
            case B2_FMT_MLX4:
            case B2_FMT_Q4_K: s.dev.p0 += r0 * (K / 256) * 144; break;
            case B2_FMT_Q6_K:
                s.dev.p0 += r0 * (K / 2);
                s.dev.p1 += r0 * (K / 4);
                s.dev.p2 += r0 * (K / 16);
                s.dev.p3 += r0 * (K / 256) * 2;
                break;
            case B2_FMT_Q8_0:
                s.dev.p0 += r0 * K;
                s.dev.p1 += r0 * (K / 32) * 2;
                break;
            case B2_FMT_F8E4M3:
                s.dev.p0 += r0 * K;
                s.dev.bs_row0 += r0;
                break;
            default:
                if (fmt_is_other(w->dev.fmt)) s.dev.p0 += r0 * other_row_bytes(w->dev.fmt, K);
                break;
        }
        s.bytes = w->bytes / w->dev.n_out * (r1 - r0);
        *out = next_handle++;
        weights[*out] = std::move(s);
        return B2_OK;
    }

    int free_weight(uint64_t h) {
        auto it = weights.find(h);
        if (it == weights.end()) return fail(B2_ERR_ARG, "[b200qmm: free_weight: unknown weight]");
        for (auto& dp : decode_plans)
            if (dp.second->uses_weight(h)) return fail(B2_ERR_ARG, "[b200qmm: free_weight: a decode plan still uses this weight (b2_plan_free first)]");
        cudaStreamSynchronize(stream);
        for (GemmPlan* p : plans) gemm_tc_plan_destroy(p);  // tensor maps may point into this weight
        plans.clear();
        drop(it->second.owned);
        weights.erase(it);
        return B2_OK;
    }

    int dequantize_rows_dev(uint64_t h, size_t r0, size_t r1, float* out_dev) {
        Weight* w = find(h);
        if (!w) return fail(B2_ERR_ARG, "[b200qmm: dequantize_rows: unknown weight]");
        if (r0 > r1 || r1 > w->dev.n_out) return fail(B2_ERR_ARG, "[b200qmm: dequantize_rows: bad row range]");
        cudaError_t e = fmt_is_other(w->dev.fmt) ? launch_dequantize_other(w->dev, r0, r1 - r0, out_dev, stream) : launch_dequantize(w->dev, r0, r1 - r0, out_dev, stream);
        launches++;
        if (e != cudaSuccess) return cuda_fail(e, "dequantize");
        return B2_OK;
    }

    int dequantize_rows(uint64_t h, size_t r0, size_t r1, float* out) {
        Weight* w = find(h);
        if (!w || !out) return fail(B2_ERR_ARG, "[b200qmm: dequantize_rows: unknown weight]");
        if (r0 > r1 || r1 > w->dev.n_out) return fail(B2_ERR_ARG, "[b200qmm: dequantize_rows: bad row range]");
        size_t bytes = (r1 - r0) * w->dev.n_in * 4;
        if (bytes == 0) return B2_OK;
        cudaError_t e = y_dev.reserve(bytes);
        if (e != cudaSuccess) return cuda_fail(e, "cudaMalloc(staging)");
        int rc = dequantize_rows_dev(h, r0, r1, (float*)y_dev.p);
        if (rc) return rc;
        e = cudaMemcpyAsync(out, y_dev.p, bytes, cudaMemcpyDeviceToHost, stream);
        if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
        if (e != cudaSuccess) return cuda_fail(e, "dequantize copy-out");
        return B2_OK;
    }

    // The activation planes of one vector (kernels.h, XPlanes), computed once and read by every
    // matrix-vector product over that vector: the role of quantize_act, which the reference's CPU
    // driver also runs once per batch of jobs (src/kernels.rs:1731-1879, `xa`).
    size_t prepared_k = 0;
    int prepare_x(const float* x_dev_, size_t n_in) {
        if (!x_dev_ || n_in == 0 || n_in % 32) return fail(B2_ERR_ARG, "[b200qmm: prepare_x: n_in must be a positive multiple of 32]");
        cudaError_t e = xplanes.reserve(xplanes_bytes(n_in));
        if (e != cudaSuccess) return cuda_fail(e, "cudaMalloc(planes)");
        e = launch_xplanes(x_dev_, n_in, planes_at(xplanes.p, n_in), stream, chained);
        launches++;
        if (e != cudaSuccess) return cuda_fail(e, "xplanes");
        prepared_k = n_in;
        return B2_OK;
    }

    // One token on the device over the prepared planes (FP8 weights read x itself).
    // `after_planes`: the product directly follows the plane kernel of its own vector in the stream, so it is launched as
    // that kernel's dependent (it fetches its first weights while the planes are written, and waits for them on the device).
    int matvec_prepared(uint64_t h, uint64_t up, const float* x_dev_, float* y_dev_, int mode, const float* gate, bool after_planes = false) {
        Weight* w = find(h);
        if (!w) return fail(B2_ERR_ARG, "[b200qmm: matvec: unknown weight]");
        bool pair = mode == B2_MODE_SILU_PAIR || mode == B2_MODE_GELU_PAIR;
        Weight* u = nullptr;
        if (pair) {
            u = find(up);
            if (!u) return fail(B2_ERR_ARG, "[b200qmm: matvec: pair mode needs the second matrix]");
            if (u->dev.fmt != w->dev.fmt || u->dev.n_in != w->dev.n_in || u->dev.n_out != w->dev.n_out)
                return fail(B2_DECLINED, "[b200qmm: matvec: the pair's matrices differ in shape or format]");
        }
        if (mode < 0 || mode > 4 || (mode == B2_MODE_ADD_GATED && !gate)) return fail(B2_ERR_ARG, "[b200qmm: matvec: bad mode]");
        if (fmt_is_other(w->dev.fmt)) {  // the generic kernel reads x itself
            if (!gemv_other_supports(w->dev)) return fail(B2_DECLINED, "[b200qmm: matvec: shape not supported for this format]");
            cudaError_t eo = launch_gemv_other(w->dev, u ? &u->dev : nullptr, x_dev_, 0, y_dev_, 0, 1, mode, gate, sm_count, stream, chained);
            launches++;
            if (eo != cudaSuccess) return cuda_fail(eo, "gemv (generic)");
            return B2_OK;
        }
        if (!gemv_supports(w->dev)) return fail(B2_DECLINED, "[b200qmm: matvec: shape not supported by the GEMV kernels]");
        XPlanes xp{};
        if (w->dev.fmt != B2_FMT_F8E4M3) {
            if (prepared_k != w->dev.n_in) return fail(B2_ERR_ARG, "[b200qmm: matvec: no planes prepared for n_in = %zu (b2_prepare_x_dev)]", w->dev.n_in);
            xp = planes_at(xplanes.p, w->dev.n_in);
        }
        cudaError_t e = launch_gemv(w->dev, u ? &u->dev : nullptr, x_dev_, xp, y_dev_, mode, gate, sm_count, stream, chained || after_planes,
                                    NormScale{nullptr, 0, 0.0f, 0.0f}, EpiPlanes{XPlanes{nullptr, nullptr, nullptr}, nullptr, nullptr, 1.0f}, after_planes && !chained);
        launches++;
        if (e != cudaSuccess) return cuda_fail(e, "gemv");
        return B2_OK;
    }

    int matvec_dev(uint64_t h, uint64_t up, const float* x_dev_, float* y_dev_, int mode, const float* gate) {
        Weight* w = find(h);
        if (!w) return fail(B2_ERR_ARG, "[b200qmm: matvec: unknown weight]");
        bool planes = false;
        if (w->dev.fmt != B2_FMT_F8E4M3 && !fmt_is_other(w->dev.fmt) && gemv_supports(w->dev)) {
            int rc = prepare_x(x_dev_, w->dev.n_in);
            if (rc) return rc;
            // the product is launched as the plane kernel's dependent, in its register-load form (the 4-bit ring form loses when
            // launched alone): its first weights travel while the planes are made
            planes = true;
        }
        return matvec_prepared(h, up, x_dev_, y_dev_, mode, gate, planes);
    }

    int ensure_status() {
        if (gemm_status) return B2_OK;
        cudaError_t e = cudaMalloc((void**)&gemm_status, sizeof(GemmStatus));
        if (e == cudaSuccess) e = cudaMemset(gemm_status, 0, sizeof(GemmStatus));
        if (e != cudaSuccess) return cuda_fail(e, "cudaMalloc(status)");
        return B2_OK;
    }

    // Formats whose many-token products run through the multi-row matrix-vector kernel (no tensor-core kernel for them).
    static bool rows_path(const WeightDev& w) { return (w.fmt == B2_FMT_Q6_K || w.fmt == B2_FMT_Q8_0) && gemv_supports(w); }

    // t tokens on the device through the tensor-core GEMM (or token by token through the GEMV).
    // peer_y (matmul_sharded_peer): the result goes, tile by tile from the GEMM's epilogue, to this rank's columns of its own y and
    // of the peers' copies; only the tensor-core GEMM takes it, every other route declines.
    int matmul_dev(uint64_t h, const void* x, int x_dtype, size_t t, void* y, int y_dtype, const GemmPeerY* peer_y = nullptr) {
        Weight* w = find(h);
        if (!w) return fail(B2_ERR_ARG, "[b200qmm: matmul: unknown weight]");
        if (t == 0) return B2_OK;
        if (y_dtype != B2_F32 && y_dtype != B2_BF16) return fail(B2_ERR_ARG, "[b200qmm: matmul: y must be f32 or bf16]");
        size_t K = w->dev.n_in;
        if (peer_y && (t <= 8 || y_dtype != B2_F32 || !gemm_tc_supports(w->dev, t) || (fp8_act && !exact && w->dev.fmt == B2_FMT_F8E4M3)))
            return fail(B2_DECLINED, "[b200qmm: matmul_sharded_peer: only the tensor-core GEMM with f32 results stores to peers (more than 8 tokens)]");
        if (fmt_is_other(w->dev.fmt)) {
            // no tensor-core kernel for these formats: four tokens at a time through the generic matrix-vector kernel (the weights
            // are read once per four tokens; every row equals its one-token row bit for bit)
            if (x_dtype != B2_F32 || y_dtype != B2_F32 || !gemv_other_supports(w->dev)) return fail(B2_DECLINED, "[b200qmm: matmul: this format takes f32 activations and results]");
            for (size_t i = 0; i < t; i += 4) {
                const int nt = (int)std::min<size_t>(4, t - i);
                cudaError_t eo = launch_gemv_other(w->dev, nullptr, (const float*)x + i * K, K, (float*)y + i * w->dev.n_out, w->dev.n_out, nt, B2_MODE_STORE, nullptr,
                                                   sm_count, stream);
                launches++;
                if (eo != cudaSuccess) return cuda_fail(eo, "gemv (generic, several rows)");
            }
            return B2_OK;
        }
        // Two to eight tokens of a 4-bit format: four at a time through the several-token matrix-vector kernel (its integer
        // dots on the tensor cores), every row equal to its one-token row bit for bit.
        const bool few_4bit = t >= 2 && t <= 8 && x_dtype == B2_F32 && y_dtype == B2_F32 && (w->dev.fmt == B2_FMT_Q4_K || w->dev.fmt == B2_FMT_MLX4) &&
                              gemv_supports(w->dev) && gemv_multi_pays(w->dev, (int)std::min<size_t>(t, 4));
        if (!few_4bit && t <= 8 && x_dtype == B2_F32 && y_dtype == B2_F32 && gemv_supports(w->dev) && !(fp8_act && w->dev.fmt == B2_FMT_F8E4M3)) {
            for (size_t i = 0; i < t; i++) {
                int rc = matvec_dev(h, 0, (const float*)x + i * K, (float*)y + i * w->dev.n_out, B2_MODE_STORE, nullptr);
                if (rc) return rc;
            }
            return B2_OK;
        }
        if (few_4bit || (rows_path(w->dev) && x_dtype == B2_F32 && y_dtype == B2_F32 && (exact || !gemm_tc_supports(w->dev, t)))) {
            // Q6_K / Q8_0 under the exact switch (or at a shape the tensor-core kernel does not take): the tokens go four at a
            // time through the multi-row matrix-vector kernel (the weights are read once per four tokens; every row equals its
            // one-token result bit for bit).
            const size_t stride = (xplanes_bytes(K) + 255) / 256 * 256;
            cudaError_t e = xplanes.reserve(t * stride);
            if (e != cudaSuccess) return cuda_fail(e, "cudaMalloc(planes)");
            e = launch_xplanes_rows((const float*)x, t, K, (uint8_t*)xplanes.p, stride, stream);
            launches++;
            prepared_k = 0;  // the scratch holds many rows' planes now
            if (e != cudaSuccess) return cuda_fail(e, "xplanes (rows)");
            const size_t n_out = w->dev.n_out;
            for (size_t i = 0; i < t; i += 4) {
                const size_t nt = std::min<size_t>(4, t - i);
                const float* xi = (const float*)x + i * K;
                float* yi = (float*)y + i * n_out;
                uint8_t* pi = (uint8_t*)xplanes.p + i * stride;
                if (nt > 1 && gemv_multi_fits(w->dev, (int)nt)) {
                    e = launch_gemv_multi(w->dev, nullptr, xi, K, planes_at(pi, K), stride, yi, n_out, (int)nt, B2_MODE_STORE, sm_count, stream);
                    launches++;
                    if (e != cudaSuccess) return cuda_fail(e, "gemv (several rows)");
                    continue;
                }
                for (size_t r = 0; r < nt; r++) {  // one row, or the rows' planes do not fit in shared memory together
                    e = launch_gemv(w->dev, nullptr, xi + r * K, planes_at(pi + r * stride, K), yi + r * n_out, B2_MODE_STORE, nullptr, sm_count, stream);
                    launches++;
                    if (e != cudaSuccess) return cuda_fail(e, "gemv");
                }
            }
            return B2_OK;
        }
        if (fp8_act && !exact && gemm_f8_supports(w->dev, t)) {
            // FP8 on both sides: the activations are quantized per token and per 128 k to e4m3, and the tensor cores multiply
            // e4m3 by e4m3 (kind::f8f6f4); partial sums of every 128 k are scaled by both scales and added in f32
            int rc8 = ensure_status();
            if (rc8) return rc8;
            cudaError_t e8 = x8.reserve(gemm_f8_scratch_bytes(t, K));
            if (e8 != cudaSuccess) return cuda_fail(e8, "cudaMalloc(x8)");
            uint8_t* q = (uint8_t*)x8.p;
            float* sx = (float*)(q + (t * K + 255) / 256 * 256);
            e8 = launch_quantize_act_e4m3(x, x_dtype, t, K, q, sx, stream);
            launches++;
            if (e8 != cudaSuccess) return cuda_fail(e8, "quantize_act_e4m3");
            char msg[256] = {0};
            e8 = launch_gemm_f8(w->dev, q, sx, t, y, y_dtype, gemm_status, stream, msg, sizeof msg);
            launches++;
            if (e8 != cudaSuccess) return msg[0] ? fail(B2_ERR_CUDA, "[b200qmm: %s]", msg) : cuda_fail(e8, "gemm_f8");
            return B2_OK;
        }
        if (!gemm_tc_supports(w->dev, t)) return fail(B2_DECLINED, "[b200qmm: matmul: no tensor-core kernel for this format / shape]");
        int rc = ensure_status();
        if (rc) return rc;
        cudaError_t e;
        const void* xh = x;  // f16 activations are used where they lie (16-byte aligned rows): in f16's range by definition
        const float* unscale = nullptr;
        size_t lo_row0 = 0;
        // exact: 128-token tiles for any t, so that the activations go in as two f16 terms, and two-term weights where the
        // format's values do not fit f16 (Q4_K): f32-like results, several times the tensor-core work
        const int w_terms = exact ? 2 : 1;
        if (x_dtype != B2_F16 || ((uintptr_t)x & 15)) {
            // f32 / bf16 rows -> f16 with a power-of-two factor per token row that the GEMM's epilogue takes out again
            // (up to 128 tokens, where a CTA's tile has room for it, as two f16 terms: 22 bits of every activation)
            lo_row0 = exact ? (t + 127) / 128 * 128 : (t <= 128 ? 128 : 0);
            if (rows_path(w->dev)) lo_row0 = 0;  // the Q6_K / Q8_0 arms of the kernel take one-term operands
            const size_t x16_bytes = ((lo_row0 + t) * K * 2 + 255) / 256 * 256;
            e = x16.reserve(x16_bytes + t * 4);
            if (e != cudaSuccess) return cuda_fail(e, "cudaMalloc(x16)");
            float* us = (float*)((uint8_t*)x16.p + x16_bytes);
            e = launch_to_f16(x, x_dtype, t, K, x16.p, us, stream, lo_row0);
            launches++;
            if (e != cudaSuccess) return cuda_fail(e, "to_f16");
            xh = x16.p;
            unscale = us;
        }
        // Tensor maps (activations + packed weights) are cached per (weights, activations, t).
        GemmPlan* plan = nullptr;
        for (GemmPlan* p : plans)
            if (gemm_tc_plan_matches(p, w->dev, xh, t, y, y_dtype, lo_row0, w_terms, lo_row0 ? 1 : 0, peer_y)) {
                plan = p;
                break;
            }
        if (!plan) {
            if (plans.size() >= 256) {
                for (GemmPlan* p : plans) gemm_tc_plan_destroy(p);
                plans.clear();
            }
            char msg[256] = {0};
            e = gemm_tc_plan_create(w->dev, xh, t, y, y_dtype, &plan, msg, sizeof msg, 1, nullptr, lo_row0 ? 1 : 0, lo_row0, w_terms, peer_y);
            if (e != cudaSuccess) return fail(B2_ERR_CUDA, "[b200qmm: %s]", msg);
            plans.push_back(plan);
        }
        e = launch_gemm_tc(plan, w->dev, t, y, y_dtype, gemm_status, sm_count, stream, unscale);
        launches++;
        if (e != cudaSuccess) return cuda_fail(e, "gemm_tc");
        return B2_OK;
    }

    // Reads the status word the GEMM writes when a bounded wait gives up (after a synchronize).
    int check_gemm_status() {
        if (!gemm_status) return B2_OK;
        GemmStatus s{};
        cudaError_t e = cudaMemcpy(&s, gemm_status, sizeof s, cudaMemcpyDeviceToHost);
        if (e != cudaSuccess) return cuda_fail(e, "status read");
#ifdef B2_DEBUG
        if (getenv("B2_GEMM_DEBUG") && (atoi(getenv("B2_GEMM_DEBUG")) & 32768)) fprintf(stderr, "[gemm debug] mma loop cycles %u over %u stages; stamps: loop start %u, loop end %u, acc seen %u, epilogue done %u, all done %u; mma thread waited %u on activations, %u on weights\n", s.where, s.iter, s.t[0], s.t[1], s.t[2], s.t[3], s.t[4], s.t[5], s.t[6]);
#endif
        if (s.code) {
            cudaMemset(gemm_status, 0, sizeof s);
            return fail(B2_ERR_TIMEOUT, "[b200qmm: gemm: a device wait gave up (wait %u, cta %u, k-stage %u)]", s.where, s.cta, s.iter);
        }
        return B2_OK;
    }

    using clk = std::chrono::steady_clock;
    static double since(clk::time_point t0) { return std::chrono::duration<double, std::nano>(clk::now() - t0).count(); }

    // ---- Backend::matmul (src/cuda.rs:1428-1493)
    int matmul(const float* x, size_t t, size_t n_in, b2_job* jobs, size_t n_jobs) {
        if (t == 0 || n_jobs == 0) return B2_OK;
        if (!x || !jobs) return fail(B2_ERR_ARG, "[b200qmm: matmul: null argument]");
        for (size_t j = 0; j < n_jobs; j++) {
            Weight* w = find(jobs[j].w);
            if (!w) return fail(B2_ERR_ARG, "[b200qmm: matmul: unknown weight in job %zu]", j);
            if (w->dev.n_in != n_in || w->dev.n_out != jobs[j].n_out || !jobs[j].y)
                return fail(B2_ERR_ARG, "[b200qmm: matmul: job %zu does not match its weight's shape]", j);
            bool small = (t <= 8 && gemv_supports(w->dev)) || gemv_other_supports(w->dev);
            if (!small && !gemm_tc_supports(w->dev, t) && !rows_path(w->dev)) return fail(B2_DECLINED, "[b200qmm: matmul: job %zu has no kernel at t = %zu]", j, t);
        }
        auto t0 = clk::now();
        // every job's result is staged on the device and all jobs run before any result goes back: a job that fails leaves
        // every y untouched ("nothing written unless 0")
        std::vector<size_t> y_off(n_jobs);
        size_t y_total = 0;
        for (size_t j = 0; j < n_jobs; j++) {
            y_off[j] = y_total;
            y_total += (t * jobs[j].n_out * 4 + 255) / 256 * 256;
        }
        cudaError_t e = x_dev.reserve(t * n_in * 4);
        if (e == cudaSuccess) e = y_dev.reserve(y_total);
        if (e != cudaSuccess) return cuda_fail(e, "cudaMalloc(staging)");
        e = cudaMemcpyAsync(x_dev.p, x, t * n_in * 4, cudaMemcpyHostToDevice, stream);
        if (e != cudaSuccess) return cuda_fail(e, "copy-in");
        ns_in += since(t0);
        auto t1 = clk::now();
        for (size_t j = 0; j < n_jobs; j++) {
            int rc = matmul_dev(jobs[j].w, x_dev.p, B2_F32, t, (uint8_t*)y_dev.p + y_off[j], B2_F32);
            if (rc) {
                cudaStreamSynchronize(stream);
                return rc;
            }
        }
        e = cudaStreamSynchronize(stream);
        if (e != cudaSuccess) return cuda_fail(e, "matmul kernels");
        if (int rc = check_gemm_status()) return rc;
        ns_gpu += since(t1);
        auto t2 = clk::now();
        for (size_t j = 0; j < n_jobs && e == cudaSuccess; j++)
            e = cudaMemcpyAsync(jobs[j].y, (uint8_t*)y_dev.p + y_off[j], t * jobs[j].n_out * 4, cudaMemcpyDeviceToHost, stream);
        if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
        if (e != cudaSuccess) return cuda_fail(e, "copy-out");
        ns_out += since(t2);
        calls++;
        return B2_OK;
    }

    // ---- Backend::matvec_rows (src/gpu.rs:165-167)
    int matvec_rows(const float* x, size_t t, size_t n_in, b2_rows_job* jobs, size_t n_jobs) {
        if (t == 0 || n_jobs == 0) return B2_OK;
        if (t > 4) return fail(B2_DECLINED, "[b200qmm: matvec_rows: at most 4 rows]");
        if (!x || !jobs) return fail(B2_ERR_ARG, "[b200qmm: matvec_rows: null argument]");
        std::vector<size_t> y_off(n_jobs);
        size_t y_total = 0;
        for (size_t j = 0; j < n_jobs; j++) {
            Weight* w = find(jobs[j].w);
            if (!w || w->dev.n_in != n_in || w->dev.n_out != jobs[j].n_out || !jobs[j].y)
                return fail(B2_ERR_ARG, "[b200qmm: matvec_rows: job %zu does not match its weight]", j);
            if (!gemv_supports(w->dev) && !gemv_other_supports(w->dev)) return fail(B2_DECLINED, "[b200qmm: matvec_rows: job %zu has no kernel]", j);
            if (jobs[j].up) {
                Weight* u = find(jobs[j].up);
                if (!u || u->dev.fmt != w->dev.fmt || u->dev.n_in != w->dev.n_in || u->dev.n_out != w->dev.n_out)
                    return fail(B2_DECLINED, "[b200qmm: matvec_rows: the pair's matrices differ in shape or format]");
            }
            y_off[j] = y_total;
            y_total += (t * jobs[j].n_out * 4 + 255) / 256 * 256;
        }
        auto t0 = clk::now();
        cudaError_t e = x_dev.reserve(t * n_in * 4);
        if (e == cudaSuccess) e = y_dev.reserve(y_total);  // all jobs run before any result goes back to the host
        if (e != cudaSuccess) return cuda_fail(e, "cudaMalloc(staging)");
        e = cudaMemcpyAsync(x_dev.p, x, t * n_in * 4, cudaMemcpyHostToDevice, stream);
        if (e != cudaSuccess) return cuda_fail(e, "copy-in");
        ns_in += since(t0);
        auto t1 = clk::now();
        // The planes of this call's rows are computed at most once, by the first job that reads them; a job that takes the
        // row-by-row route writes one vector's planes into the same scratch, after which they must be computed again.
        bool planes_ready = false;
        const size_t stride = (xplanes_bytes(n_in) + 255) / 256 * 256;
        for (size_t j = 0; j < n_jobs; j++) {
            Weight* w = find(jobs[j].w);
            Weight* u = jobs[j].up ? find(jobs[j].up) : nullptr;
            float* yj = (float*)((uint8_t*)y_dev.p + y_off[j]);
            const int mode = jobs[j].up ? B2_MODE_SILU_PAIR : B2_MODE_STORE;
            if (fmt_is_other(w->dev.fmt)) {
                e = launch_gemv_other(w->dev, u ? &u->dev : nullptr, (const float*)x_dev.p, n_in, yj, jobs[j].n_out, (int)t, mode, nullptr, sm_count, stream);
                launches++;
                if (e != cudaSuccess) return cuda_fail(e, "gemv (generic)");
                continue;
            }
            // Two to four rows: one launch that reads the weights once (each row's result is the one-row result bit for bit),
            // when the rows' vectors fit in shared memory together. FP8 rows go one by one: their single-row kernel is the
            // tensor-core one, and the rows must match it bit for bit.
            if (t > 1 && w->dev.fmt != B2_FMT_F8E4M3 && gemv_multi_fits(w->dev, (int)t)) {
                if (!planes_ready) {
                    e = xplanes.reserve(t * stride);
                    if (e != cudaSuccess) return cuda_fail(e, "cudaMalloc(planes)");
                    e = launch_xplanes_rows((const float*)x_dev.p, t, n_in, (uint8_t*)xplanes.p, stride, stream);
                    launches++;
                    if (e != cudaSuccess) return cuda_fail(e, "xplanes (rows)");
                    prepared_k = 0;  // the scratch now holds several rows' planes, not one prepared vector
                    planes_ready = true;
                }
                e = launch_gemv_multi(w->dev, u ? &u->dev : nullptr, (const float*)x_dev.p, n_in, planes_at(xplanes.p, n_in), stride, yj, jobs[j].n_out,
                                      (int)t, mode, sm_count, stream);
                launches++;
                if (e != cudaSuccess) return cuda_fail(e, "gemv (several rows)");
                continue;
            }
            for (size_t i = 0; i < t; i++) {
                if (w->dev.fmt != B2_FMT_F8E4M3) planes_ready = false;  // matvec_dev overwrites the planes scratch
                int rc = matvec_dev(jobs[j].w, jobs[j].up, (const float*)x_dev.p + i * n_in, yj + i * jobs[j].n_out, mode, nullptr);
                if (rc) {
                    cudaStreamSynchronize(stream);
                    return rc;
                }
            }
        }
        // Every launch was accepted (a refused one returned above, before any y is touched): the results follow the kernels on
        // the stream and the call synchronizes once. (The matrix-vector kernels have no status word to consult in between; a
        // product of a few microseconds would otherwise pay two host round trips.) The kernels' and the copies' time are
        // booked together as kernel time.
        for (size_t j = 0; j < n_jobs && e == cudaSuccess; j++)
            e = cudaMemcpyAsync(jobs[j].y, (uint8_t*)y_dev.p + y_off[j], t * jobs[j].n_out * 4, cudaMemcpyDeviceToHost, stream);
        if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
        if (e != cudaSuccess) return cuda_fail(e, "matvec_rows kernels / copy-out");
        ns_gpu += since(t1);
        calls++;
        return B2_OK;
    }

    // ---- Backend::upload_moe (src/gpu.rs:200-215, src/cuda.rs:777-796): the experts were uploaded one by
    // one with b2_upload_*; their blocks are copied into two stacked buffers the grouped GEMM indexes by
    // expert, after which the caller may free the per-expert handles.
    // `up` == nullptr: gate_up[e] is the fused projection [2 inter][h]; else gate_up[e] is the gate projection [inter][h] and up[e]
    // the up projection [inter][h] (GGUF files store them apart, src/gpu.rs:200-215): they are stacked into the fused layout here.
    int upload_moe(const uint64_t* gate_up, const uint64_t* up, const uint64_t* down, size_t experts, size_t h, size_t inter, int act, float limit,
                   uint64_t* out) {
        if (!gate_up || !down || !out || experts == 0) return fail(B2_ERR_ARG, "[b200qmm: upload_moe: null argument]");
        if (h % 256 || inter % 256) return fail(B2_DECLINED, "[b200qmm: upload_moe: h and inter must be multiples of 256]");
        if (act != B2_ACT_SILU && act != B2_ACT_GELU_TANH && act != B2_ACT_SILU_CLAMP)
            return fail(B2_DECLINED, "[b200qmm: upload_moe: activation %d is not run on the device (SwigluOai and SiTU stay on the CPU, as in the reference)]", act);
        Moe m;
        m.act = act;
        m.act_limit = limit;
        m.experts = experts;
        m.h = h;
        m.inter = inter;
        const size_t gu_bytes = 2 * inter * (h / 256) * 144, dn_bytes = h * (inter / 256) * 144;
        for (size_t e = 0; e < experts; e++) {
            Weight *g = find(gate_up[e]), *d = find(down[e]), *u = up ? find(up[e]) : nullptr;
            if (!g || !d || (up && !u)) return fail(B2_ERR_ARG, "[b200qmm: upload_moe: unknown weight for expert %zu]", e);
            if (e == 0) m.fmt = g->dev.fmt;
            if ((m.fmt != B2_FMT_MLX4 && m.fmt != B2_FMT_Q4_K) || g->dev.fmt != m.fmt || d->dev.fmt != m.fmt || (u && u->dev.fmt != m.fmt))
                return fail(B2_DECLINED, "[b200qmm: upload_moe: experts must all be MLX-4 or all Q4_K]");
            if (g->dev.n_out != (up ? inter : 2 * inter) || g->dev.n_in != h || d->dev.n_out != h || d->dev.n_in != inter ||
                (u && (u->dev.n_out != inter || u->dev.n_in != h)))
                return fail(B2_ERR_ARG, "[b200qmm: upload_moe: expert %zu has the wrong shape]", e);
        }
        cudaError_t e1 = cudaMalloc(&m.gate_up, gu_bytes * experts), e2 = cudaSuccess;
        if (e1 == cudaSuccess) e2 = cudaMalloc(&m.down, dn_bytes * experts);
        if (e1 != cudaSuccess || e2 != cudaSuccess) {
            if (m.gate_up) cudaFree(m.gate_up);
            return cuda_fail(e1 != cudaSuccess ? e1 : e2, "cudaMalloc(moe)");
        }
        for (size_t e = 0; e < experts; e++) {
            if (up) {  // gate rows, then up rows
                cudaMemcpyAsync((uint8_t*)m.gate_up + e * gu_bytes, find(gate_up[e])->dev.p0, gu_bytes / 2, cudaMemcpyDeviceToDevice, stream);
                cudaMemcpyAsync((uint8_t*)m.gate_up + e * gu_bytes + gu_bytes / 2, find(up[e])->dev.p0, gu_bytes / 2, cudaMemcpyDeviceToDevice, stream);
            } else {
                cudaMemcpyAsync((uint8_t*)m.gate_up + e * gu_bytes, find(gate_up[e])->dev.p0, gu_bytes, cudaMemcpyDeviceToDevice, stream);
            }
            cudaMemcpyAsync((uint8_t*)m.down + e * dn_bytes, find(down[e])->dev.p0, dn_bytes, cudaMemcpyDeviceToDevice, stream);
        }
        cudaError_t e = cudaStreamSynchronize(stream);
        if (e != cudaSuccess) {
            cudaFree(m.gate_up);
            cudaFree(m.down);
            return cuda_fail(e, "upload_moe copies");
        }
        m.bytes = (gu_bytes + dn_bytes) * experts;
        *out = next_handle++;
        moes[*out] = m;
        return B2_OK;
    }

    int free_moe(uint64_t h) {
        auto it = moes.find(h);
        if (it == moes.end()) return fail(B2_ERR_ARG, "[b200qmm: free_moe: unknown handle]");
        cudaStreamSynchronize(stream);
        cudaFree(it->second.gate_up);
        cudaFree(it->second.down);
        moes.erase(it);
        return B2_OK;
    }

    // One grouped GEMM: rows of xg (f16, segments of whole 128-row tiles per expert) times the stacked matrices.
    int grouped_gemm(int fmt, const void* stacked, size_t experts, size_t n_out, size_t n_in, const void* xg, size_t rows, const int* tile_expert,
                     float* out_dev, int m_halves, const float* row_unscale, size_t a_lo_row0) {
        WeightDev w{};
        w.fmt = fmt;
        w.n_out = n_out;
        w.n_in = n_in;
        w.p0 = (const uint8_t*)stacked;
        GemmPlan* plan = nullptr;
        char msg[256] = {0};
        cudaError_t e = gemm_tc_plan_create(w, xg, rows, out_dev, B2_F32, &plan, msg, sizeof msg, experts, tile_expert, m_halves, a_lo_row0, a_lo_row0 ? 2 : 1);
        if (e != cudaSuccess) return fail(B2_ERR_CUDA, "[b200qmm: %s]", msg);
        e = launch_gemm_tc(plan, w, rows, out_dev, B2_F32, gemm_status, sm_count, stream, row_unscale);
        launches++;
        gemm_tc_plan_destroy(plan);  // the tensor maps were copied into the launch's parameters
        if (e != cudaSuccess) return cuda_fail(e, "grouped gemm");
        return B2_OK;
    }

    // ---- Backend::moe (src/gpu.rs:232-248, src/cuda.rs:798-966): y[i] += sum_j w_ij down_e(act(gate_e x_i) * up_e x_i).
    // The host builds the per-expert segments as the reference does (src/cuda.rs:810-857), padded to the
    // GEMM's 128-row token tile; x_dev / y_dev are device f32 [t][h].
    // A few (token, route) pairs (decode): every pair is its own matrix-vector product, so the tensor-core GEMM's 128-row
    // tiles would be almost empty. Five launches instead: planes of the tokens, one batched GEMV over the pairs' fused
    // gate / up matrices (SiLU pair), planes of the activations, one batched GEMV over the down matrices, and the ordered
    // combine (src/moe.rs:625-828 does the same per expert on the CPU; exact f32 / integer arithmetic, no f16 operands).
    int moe_small(const Moe& m, const float* x_dev_, size_t t, const int32_t* ids, const float* rw, size_t k, float* y_dev_) {
        const size_t R = t * k;
        const size_t sx = (xplanes_bytes(m.h) + 255) / 256 * 256, sa = (xplanes_bytes(m.inter) + 255) / 256 * 256;
        cudaError_t e = moe_xg.reserve(t * sx);
        if (e == cudaSuccess) e = moe_g.reserve(R * m.inter * 4);
        if (e == cudaSuccess) e = moe_a.reserve(R * sa);
        if (e == cudaSuccess) e = moe_o.reserve(R * m.h * 4);
        if (e != cudaSuccess) return cuda_fail(e, "cudaMalloc(moe scratch)");
        // the routes travel as kernel arguments: no copy, no synchronization
        GemvBatch b1{}, b2{};
        SmallRoutes routes{};
        b1.n = b2.n = (int)R;
        for (size_t i = 0; i < R; i++) {
            b1.expert[i] = b2.expert[i] = ids[i];
            b1.xrow[i] = (int)(i / k);  // the pair's token
            b2.xrow[i] = (int)i;        // the pair's own activations
            routes.w[i] = rw[i];
        }
        const size_t rb_h = m.h / 256 * 144, rb_i = m.inter / 256 * 144;
        WeightDev gate{};
        gate.fmt = m.fmt;
        gate.n_out = m.inter;
        gate.n_in = m.h;
        gate.group = 64;
        gate.p0 = (const uint8_t*)m.gate_up;
        WeightDev up = gate;
        up.p0 = gate.p0 + m.inter * rb_h;
        WeightDev down = gate;
        down.n_out = m.h;
        down.n_in = m.inter;
        down.p0 = (const uint8_t*)m.down;
        e = launch_xplanes_rows(x_dev_, t, m.h, (uint8_t*)moe_xg.p, sx, stream);
        b1.w_stride = 2 * m.inter * rb_h;
        b1.x_stride = sx;
        b1.y_stride = m.inter;
        b1.planes = (uint8_t*)moe_xg.p;
        b2.w_stride = m.h * rb_i;
        b2.x_stride = sa;
        b2.y_stride = m.h;
        b2.planes = (uint8_t*)moe_a.p;
        if (e == cudaSuccess)
            e = launch_gemv_batched(gate, &up, b1, R, (float*)moe_g.p, m.act == B2_ACT_GELU_TANH ? B2_MODE_GELU_PAIR : B2_MODE_SILU_PAIR, planes_read(), sm_count, stream,
                                    true);
        // (the five kernels are a chain of dependent launches: each may start while the one ahead drains and waits for it
        // before it reads what that one wrote)
        if (e == cudaSuccess) e = launch_xplanes_rows((const float*)moe_g.p, R, m.inter, (uint8_t*)moe_a.p, sa, stream, true);
        if (e == cudaSuccess) e = launch_gemv_batched(down, nullptr, b2, R, (float*)moe_o.p, B2_MODE_STORE, planes_read(), sm_count, stream, true);
        if (e == cudaSuccess) e = launch_moe_combine_small((const float*)moe_o.p, routes, t, k, m.h, y_dev_, stream, true);
        launches += 5;
        if (e != cudaSuccess) return cuda_fail(e, "moe (batched matrix-vector path)");
        return B2_OK;
    }

    static size_t rows_for(const std::vector<size_t>& count, size_t tile) {
        size_t rows = 0;
        for (size_t c : count) rows += (c + tile - 1) / tile * tile;
        return rows;
    }

    int moe_dev(uint64_t handle, const float* x_dev_, size_t t, const int32_t* ids, const float* rw, size_t k, float* y_dev_) {
        auto it = moes.find(handle);
        if (it == moes.end()) return fail(B2_ERR_ARG, "[b200qmm: moe: unknown handle]");
        const Moe& m = it->second;
        if (t == 0 || k == 0) return B2_OK;
        if (((uintptr_t)x_dev_ | (uintptr_t)y_dev_) & 15) return fail(B2_ERR_ARG, "[b200qmm: moe: x and y must be 16-byte aligned]");
        int rc = ensure_status();
        if (rc) return rc;
        std::vector<size_t> count(m.experts, 0);
        for (size_t i = 0; i < t * k; i++) {
            if (ids[i] < 0 || (size_t)ids[i] >= m.experts) return fail(B2_ERR_ARG, "[b200qmm: moe: expert index out of range]");
            count[(size_t)ids[i]]++;
        }
        // (the clamped SiLU has no fused pair mode in the matrix-vector kernels: those layers take the GEMM path at any batch)
        if (t * k <= 64 && m.act != B2_ACT_SILU_CLAMP && !getenv("B2_MOE_NO_GEMV")) return moe_small(m, x_dev_, t, ids, rw, k, y_dev_);
        // Token tiles of 128 or 256 rows. A tile costs about the same either way (the kernel is bound by the expansion of
        // the tile's weights, which both heights share), so the taller tile wins as soon as it needs clearly fewer tiles:
        // large batches, where the experts hold more than a tile's worth of tokens each.
        size_t tiles128 = 0, tiles256 = 0;
        for (size_t e = 0; e < m.experts; e++) {
            tiles128 += (count[e] + 127) / 128;
            tiles256 += (count[e] + 255) / 256;
        }
        static const int force_tile = [] {
            const char* e = getenv("B2_MOE_TILE");
            return e ? atoi(e) : 0;
        }();
        // Two-term operands (activations of both projections as two f16 terms, Q4_K weights as two f16 terms) need the
        // 128-row tile. Q4_K experts always take them: Q4_K values round harder to f16 than MLX-4's, and one-term operands
        // through two chained projections leave that layer above 1e-3 per output row (MLX-4 stays near 3e-4 with one term).
        const bool two_term = m.fmt == B2_FMT_Q4_K || exact;
        const size_t TILE = two_term ? 128
                            : force_tile == 128 || force_tile == 256 ? (size_t)force_tile
                            : tiles256 * 10 <= tiles128 * 8 ? 256 : 128;
        const int m_halves = (int)(TILE / 128);
        const size_t lo_row0 = two_term ? rows_for(count, 128) : 0;
        std::vector<size_t> off(m.experts, 0);
        std::vector<int32_t> tile_expert;
        size_t rows = 0;
        const size_t terms = lo_row0 ? 2 : 1;
        for (size_t e = 0; e < m.experts; e++) {
            off[e] = rows;
            size_t tiles = (count[e] + TILE - 1) / TILE;
            for (size_t i = 0; i < tiles; i++) tile_expert.push_back((int32_t)e);
            rows += tiles * TILE;
        }
        std::vector<int32_t> src(rows, -1), slots(t * k);
        std::vector<size_t> fill(m.experts, 0);
        for (size_t i = 0; i < t; i++)
            for (size_t j = 0; j < k; j++) {
                size_t e = (size_t)ids[i * k + j];
                size_t r = off[e] + fill[e]++;
                src[r] = (int32_t)i;
                slots[i * k + j] = (int32_t)r;
            }
        // index block on the device: src | slots | tile_expert | route weights
        const size_t n_idx = rows + t * k + tile_expert.size();
        cudaError_t e = moe_idx.reserve(n_idx * 4 + t * k * 4);
        if (e == cudaSuccess) e = moe_xg.reserve(terms * rows * m.h * 2 + rows * 4);
        if (e == cudaSuccess) e = moe_g.reserve(rows * 2 * m.inter * 4);
        if (e == cudaSuccess) e = moe_a.reserve(terms * rows * m.inter * 2 + rows * 4);
        if (e == cudaSuccess) e = moe_o.reserve(rows * m.h * 4);
        if (e != cudaSuccess) return cuda_fail(e, "cudaMalloc(moe scratch)");
        int32_t* d_src = (int32_t*)moe_idx.p;
        int32_t* d_slots = d_src + rows;
        int32_t* d_tiles = d_slots + t * k;
        float* d_w = (float*)(d_tiles + tile_expert.size());
        std::vector<int32_t> host(n_idx);
        std::memcpy(host.data(), src.data(), rows * 4);
        std::memcpy(host.data() + rows, slots.data(), t * k * 4);
        std::memcpy(host.data() + rows + t * k, tile_expert.data(), tile_expert.size() * 4);
        e = cudaMemcpyAsync(d_src, host.data(), n_idx * 4, cudaMemcpyHostToDevice, stream);
        if (e == cudaSuccess) e = cudaMemcpyAsync(d_w, rw, t * k * 4, cudaMemcpyHostToDevice, stream);
        if (e == cudaSuccess) e = cudaStreamSynchronize(stream);  // the host vectors go out of scope
        if (e != cudaSuccess) return cuda_fail(e, "moe index upload");
        float* x_unscale = (float*)((uint8_t*)moe_xg.p + terms * rows * m.h * 2);
        float* a_unscale = (float*)((uint8_t*)moe_a.p + terms * rows * m.inter * 2);
        e = launch_moe_gather(x_dev_, d_src, rows, m.h, moe_xg.p, x_unscale, lo_row0, stream);
        launches++;
        if (e != cudaSuccess) return cuda_fail(e, "moe_gather");
        if ((rc = grouped_gemm(m.fmt, m.gate_up, m.experts, 2 * m.inter, m.h, moe_xg.p, rows, d_tiles, (float*)moe_g.p, m_halves, x_unscale, lo_row0))) return rc;
        e = launch_moe_act((const float*)moe_g.p, d_src, rows, m.inter, moe_a.p, a_unscale, lo_row0, stream, m.act, m.act_limit);
        launches++;
        if (e != cudaSuccess) return cuda_fail(e, "moe_act");
        if ((rc = grouped_gemm(m.fmt, m.down, m.experts, m.h, m.inter, moe_a.p, rows, d_tiles, (float*)moe_o.p, m_halves, a_unscale, lo_row0))) return rc;
        e = launch_moe_combine((const float*)moe_o.p, d_slots, d_w, t, k, m.h, y_dev_, stream);
        launches++;
        if (e != cudaSuccess) return cuda_fail(e, "moe_combine");
        return B2_OK;
    }

    int moe(uint64_t handle, const float* x, size_t t, const int32_t* ids, const float* rw, size_t k, float* y) {
        auto it = moes.find(handle);
        if (it == moes.end()) return fail(B2_ERR_ARG, "[b200qmm: moe: unknown handle]");
        if (!x || !y || !ids || !rw) return fail(B2_ERR_ARG, "[b200qmm: moe: null argument]");
        const size_t h = it->second.h;
        cudaError_t e = x_dev.reserve(t * h * 4);
        if (e == cudaSuccess) e = y_dev.reserve(t * h * 4);
        if (e != cudaSuccess) return cuda_fail(e, "cudaMalloc(staging)");
        e = cudaMemcpyAsync(x_dev.p, x, t * h * 4, cudaMemcpyHostToDevice, stream);
        if (e == cudaSuccess) e = cudaMemcpyAsync(y_dev.p, y, t * h * 4, cudaMemcpyHostToDevice, stream);
        if (e != cudaSuccess) return cuda_fail(e, "copy-in");
        int rc = moe_dev(handle, (const float*)x_dev.p, t, ids, rw, k, (float*)y_dev.p);
        if (rc) return rc;
        e = cudaStreamSynchronize(stream);
        if (e != cudaSuccess) return cuda_fail(e, "moe kernels");
        if ((rc = check_gemm_status())) return rc;
        e = cudaMemcpyAsync(y, y_dev.p, t * h * 4, cudaMemcpyDeviceToHost, stream);
        if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
        if (e != cudaSuccess) return cuda_fail(e, "copy-out");
        calls++;
        return B2_OK;
    }

    int route_topk(const float* logits_dev, size_t t, size_t n, size_t k, int32_t* ids_dev, float* w_dev) {
        cudaError_t e = launch_route_topk(logits_dev, t, n, k, ids_dev, w_dev, stream);
        launches++;
        if (e != cudaSuccess) return cuda_fail(e, "route_topk");
        return B2_OK;
    }

    // ---- tensor parallel / expert parallel over NCCL (no counterpart in the reference, which has one device) ----
    int nccl_fail(int rc, const char* what) { return fail(B2_ERR_CUDA, "[b200qmm: %s: %s]", what, nccl_api().GetErrorString ? nccl_api().GetErrorString(rc) : "NCCL error"); }

    int comm_init(int world_, int rank_, const void* id) {
        const NcclApi& n = nccl_api();
        if (!n.ok) return fail(B2_DECLINED, "[b200qmm: comm_init: libnccl.so.2 was not found]");
        if (!id || world_ < 1 || rank_ < 0 || rank_ >= world_) return fail(B2_ERR_ARG, "[b200qmm: comm_init: bad world / rank / id]");
        if (comm) return fail(B2_ERR_ARG, "[b200qmm: comm_init: this context already has a communicator]");
        NcclId uid;
        std::memcpy(&uid, id, sizeof uid);
        int rc = n.CommInitRank(&comm, world_, uid, rank_);
        if (rc) {
            comm = nullptr;
            return nccl_fail(rc, "ncclCommInitRank");
        }
        world = world_;
        rank = rank_;
        return B2_OK;
    }
    int comm_free() {
        if (comm) {
            cudaStreamSynchronize(stream);
            tp_sym_release();
            nccl_api().CommDestroy(comm);
        }
        comm = nullptr;
        world = 1;
        rank = 0;
        return B2_OK;
    }

    // y[t][world * n_local] (f32, on every rank) = x[t][n_in] W^T for a W whose rows are sharded in equal contiguous parts over the
    // ranks (w = this rank's shard): the shard's product into a staging buffer, one all-gather of the ranks' [t][n_local]
    // blocks, and a copy that puts each block into its columns. Every column is computed by the kernel that computes it on one
    // GPU, so the result equals the unsharded product bit for bit.
    int matmul_sharded(uint64_t h, const void* x, int x_dtype, size_t t, float* y) {
        Weight* w = find(h);
        if (!w) return fail(B2_ERR_ARG, "[b200qmm: matmul_sharded: unknown weight]");
        if (!comm) return fail(B2_ERR_ARG, "[b200qmm: matmul_sharded: no communicator (b2_comm_init)]");
        if (t == 0) return B2_OK;
        const size_t nl = w->dev.n_out, block = t * nl;
        cudaError_t e = tp_stage.reserve(block * 4);
        if (e == cudaSuccess) e = tp_gather.reserve(block * 4 * (size_t)world);
        if (e != cudaSuccess) return cuda_fail(e, "cudaMalloc(gather staging)");
        int rc = matmul_dev(h, x, x_dtype, t, tp_stage.p, B2_F32);
        if (rc) return rc;
        int nrc = nccl_api().AllGather(tp_stage.p, tp_gather.p, block, NCCL_FLOAT32, comm, stream);
        if (nrc) return nccl_fail(nrc, "ncclAllGather");
        e = launch_scatter_blocks((const float*)tp_gather.p, (size_t)world, t, nl, y, stream);
        launches++;
        if (e != cudaSuccess) return cuda_fail(e, "scatter_blocks");
        return B2_OK;
    }

    // ---- the same product with the all-gather done by the GEMM's own epilogue -------------------------------------------------
    // Every rank keeps a buffer of the same size, mapped into the other ranks (CUDA IPC): 1 KB of flag words, then two result
    // areas used in turn. A rank's GEMM stores each finished tile into its columns of ITS OWN area and of EVERY PEER's area
    // (bulk tensor stores through NVLink), then the ranks meet (flags written into the peers' buffers with system-scope
    // release, bounded polling of the own ones): past that point on the stream, the area holds the whole y. The areas
    // alternate so that a call never writes what a peer may still be reading from the call before.
    struct TpSym {
        uint8_t* local = nullptr;
        size_t half = 0;  // bytes of one result area
        uint8_t* peer[8] = {};
        uint32_t calls = 0;
    } tp_sym;
    static constexpr size_t TP_SYM_HEADER = 1024;

    void tp_sym_release() {
        for (int p = 0; p < 8; p++)
            if (tp_sym.peer[p]) cudaIpcCloseMemHandle(tp_sym.peer[p]);
        if (tp_sym.local) cudaFree(tp_sym.local);
        tp_sym = TpSym{};
    }
    // Collective (every rank calls it with the same size): makes the buffers at least `bytes` per area.
    int tp_sym_reserve(size_t bytes) {
        if (tp_sym.half >= bytes) return B2_OK;
        const NcclApi& n = nccl_api();
        cudaError_t e = tp_stage.reserve(64 + 64 * (size_t)world);
        if (e != cudaSuccess) return cuda_fail(e, "cudaMalloc(handle exchange)");
        // 1. nobody maps an old buffer any more before anybody frees one
        for (int p = 0; p < 8; p++)
            if (tp_sym.peer[p]) {
                cudaIpcCloseMemHandle(tp_sym.peer[p]);
                tp_sym.peer[p] = nullptr;
            }
        int nrc = n.AllGather(tp_stage.p, (uint8_t*)tp_stage.p + 64, 16, NCCL_FLOAT32, comm, stream);
        if (nrc) return nccl_fail(nrc, "ncclAllGather(barrier)");
        if ((e = cudaStreamSynchronize(stream)) != cudaSuccess) return cuda_fail(e, "synchronize");
        if (tp_sym.local) cudaFree(tp_sym.local);
        tp_sym = TpSym{};
        // 2. the new buffer, its flags cleared, and its handle to everybody
        const size_t half = (bytes + ((size_t)1 << 20) - 1) >> 20 << 20;
        if ((e = cudaMalloc((void**)&tp_sym.local, TP_SYM_HEADER + 2 * half)) != cudaSuccess) return cuda_fail(e, "cudaMalloc(result buffer)");
        cudaIpcMemHandle_t mine;
        static_assert(sizeof mine == 64, "handle size");
        if ((e = cudaMemsetAsync(tp_sym.local, 0, TP_SYM_HEADER, stream)) != cudaSuccess || (e = cudaIpcGetMemHandle(&mine, tp_sym.local)) != cudaSuccess ||
            (e = cudaMemcpyAsync(tp_stage.p, &mine, 64, cudaMemcpyHostToDevice, stream)) != cudaSuccess)
            return cuda_fail(e, "cudaIpcGetMemHandle");
        nrc = n.AllGather(tp_stage.p, (uint8_t*)tp_stage.p + 64, 16, NCCL_FLOAT32, comm, stream);
        if (nrc) return nccl_fail(nrc, "ncclAllGather(handles)");
        std::vector<cudaIpcMemHandle_t> all((size_t)world);
        if ((e = cudaMemcpyAsync(all.data(), (uint8_t*)tp_stage.p + 64, 64 * (size_t)world, cudaMemcpyDeviceToHost, stream)) != cudaSuccess ||
            (e = cudaStreamSynchronize(stream)) != cudaSuccess)
            return cuda_fail(e, "handle exchange");
        for (int p = 0; p < world; p++) {
            if (p == rank) continue;
            void* m = nullptr;
            if ((e = cudaIpcOpenMemHandle(&m, all[(size_t)p], cudaIpcMemLazyEnablePeerAccess)) != cudaSuccess) return cuda_fail(e, "cudaIpcOpenMemHandle(peer result buffer)");
            tp_sym.peer[p] = (uint8_t*)m;
        }
        tp_sym.half = half;
        return B2_OK;
    }

    // y_out: this rank's copy of y [t][world * n_local] (f32), inside the library's buffer, complete once the stream reaches the
    // end of this call and valid until the call after the next one. Bit-identical to matmul_sharded.
    int matmul_sharded_peer(uint64_t h, const void* x, int x_dtype, size_t t, float** y_out) {
        Weight* w = find(h);
        if (!w || !y_out) return fail(B2_ERR_ARG, "[b200qmm: matmul_sharded_peer: unknown weight or null result pointer]");
        if (!comm || world < 2 || world > 8) return fail(B2_DECLINED, "[b200qmm: matmul_sharded_peer: needs a communicator of 2 to 8 ranks (b2_comm_init)]");
        const size_t nl = w->dev.n_out, N = nl * (size_t)world;
        if (t <= 8 || nl % 4 || !gemm_tc_supports(w->dev, t) || (fp8_act && !exact && w->dev.fmt == B2_FMT_F8E4M3))
            return fail(B2_DECLINED, "[b200qmm: matmul_sharded_peer: only the tensor-core GEMM with f32 results stores to peers (more than 8 tokens, n_out %% 4 == 0)]");
        int rc = tp_sym_reserve(t * N * 4);
        if (rc) return rc;
        if ((rc = ensure_status())) return rc;
        const size_t area = TP_SYM_HEADER + (size_t)(tp_sym.calls & 1) * tp_sym.half;
        float* mine = (float*)(tp_sym.local + area);
        GemmPeerY py;
        py.ld = N;
        PeerSet ps{};
        ps.rank = (uint32_t)rank;
        ps.world = (uint32_t)world;
        for (int p = 0; p < world; p++) {
            uint8_t* base = p == rank ? tp_sym.local : tp_sym.peer[p];
            ps.base[p] = (float*)(base + area);
            ps.flags[p] = (uint32_t*)base;
            if (p != rank) py.more[py.n_more++] = (float*)(base + area) + (size_t)rank * nl;
        }
        rc = matmul_dev(h, x, x_dtype, t, mine + (size_t)rank * nl, B2_F32, &py);
        if (rc) return rc;
        // the ranks meet: every rank's tiles have landed in every buffer (the kernel waited for its stores before it ended)
        // (the ranks' hosts are not in lockstep: a peer may be a few launches behind; four seconds of polling before giving up)
        cudaError_t e = launch_exchange(ps, 0, 0, (uint32_t*)tp_sym.local, &gemm_status->code, stream, true, false, 8000000000ll);
        launches++;
        if (e != cudaSuccess) return cuda_fail(e, "peer barrier");
        tp_sym.calls++;
        *y_out = mine;
        return B2_OK;
    }

    // Expert-parallel routed experts: the layer's experts are sharded in equal contiguous parts over the ranks (`handle` holds
    // this rank's, n_experts_global / world of them), the tokens x [t][h] are this rank's own, route_ids are GLOBAL expert
    // numbers. Every (token, route) pair travels to the rank that owns its expert and its result travels back:
    //   1. all-gather of every rank's per-expert pair counts (one small copy back to the host: the only synchronization);
    //   2. the pairs' token rows, grouped by destination rank, then by expert, token order kept, sent with one grouped
    //      send / receive (a receiver knows each row's expert from the counts alone, so no ids travel);
    //   3. the local experts over the received rows (moe_dev with one route of weight 1 per row);
    //   4. the results back the same way, and the combine y[i] += sum_j w_ij o_ij in route order.
    // Each pair runs the kernels it runs on one GPU with the same inputs, and the combine keeps the route order: bit-identical
    // to the single-GPU layer.
    int moe_ep(uint64_t handle, size_t n_experts_global, const float* x_dev_, size_t t, const int32_t* ids, const float* rw, size_t k, float* y_dev_) {
        auto it = moes.find(handle);
        if (it == moes.end()) return fail(B2_ERR_ARG, "[b200qmm: moe_ep: unknown handle]");
        if (!comm) return fail(B2_ERR_ARG, "[b200qmm: moe_ep: no communicator (b2_comm_init)]");
        const size_t E = n_experts_global, W = (size_t)world, per = it->second.experts, hdim = it->second.h;
        if (E != per * W) return fail(B2_ERR_ARG, "[b200qmm: moe_ep: this rank must hold n_experts_global / world experts]");
        const NcclApi& n = nccl_api();
        const size_t P = t * k;
        for (size_t i = 0; i < P; i++)
            if (ids[i] < 0 || (size_t)ids[i] >= E) return fail(B2_ERR_ARG, "[b200qmm: moe_ep: expert index out of range]");
        // 1. counts
        std::vector<int32_t> mine(E, 0), all(E * W, 0);
        for (size_t i = 0; i < P; i++) mine[(size_t)ids[i]]++;
        cudaError_t e = ep_idx.reserve((E + E * W) * 4 + (2 * P + 16) * 4);
        if (e != cudaSuccess) return cuda_fail(e, "cudaMalloc(ep index)");
        int32_t* d_mine = (int32_t*)ep_idx.p;
        int32_t* d_all = d_mine + E;
        int32_t* d_order = d_all + E * W;   // [P] token of the i-th sent row
        int32_t* d_slots = d_order + P;     // [P] position of pair (i, j) in the returned rows
        e = cudaMemcpyAsync(d_mine, mine.data(), E * 4, cudaMemcpyHostToDevice, stream);
        if (e != cudaSuccess) return cuda_fail(e, "ep counts upload");
        int nrc = n.AllGather(d_mine, d_all, E, NCCL_INT32, comm, stream);
        if (nrc) return nccl_fail(nrc, "ncclAllGather(counts)");
        e = cudaMemcpyAsync(all.data(), d_all, E * W * 4, cudaMemcpyDeviceToHost, stream);
        if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
        if (e != cudaSuccess) return cuda_fail(e, "ep counts");
        // 2. send order: by expert (hence by owner rank), token order kept
        std::vector<size_t> start(E + 1, 0);
        for (size_t x = 0; x < E; x++) start[x + 1] = start[x] + (size_t)mine[x];
        std::vector<int32_t> order(P), slots(P);
        {
            std::vector<size_t> fill(start.begin(), start.end() - 1);
            for (size_t i = 0; i < t; i++)
                for (size_t j = 0; j < k; j++) {
                    const size_t pos = fill[(size_t)ids[i * k + j]]++;
                    order[pos] = (int32_t)i;
                    slots[i * k + j] = (int32_t)pos;
                }
        }
        std::vector<size_t> send_rows(W, 0), recv_rows(W, 0);
        size_t n_recv = 0;
        for (size_t r = 0; r < W; r++) {
            for (size_t x = r * per; x < (r + 1) * per; x++) send_rows[r] += (size_t)mine[x];
            for (size_t x = (size_t)rank * per; x < ((size_t)rank + 1) * per; x++) recv_rows[r] += (size_t)all[r * E + x];
            n_recv += recv_rows[r];
        }
        e = ep_send.reserve(std::max<size_t>(P, 1) * hdim * 4);
        if (e == cudaSuccess) e = ep_recv.reserve(std::max<size_t>(n_recv, 1) * hdim * 4);
        if (e == cudaSuccess) e = ep_out.reserve(std::max<size_t>(n_recv, 1) * hdim * 4);
        if (e == cudaSuccess) e = ep_back.reserve(std::max<size_t>(P, 1) * hdim * 4);
        if (e != cudaSuccess) return cuda_fail(e, "cudaMalloc(ep rows)");
        if (P) {
            e = cudaMemcpyAsync(d_order, order.data(), P * 4, cudaMemcpyHostToDevice, stream);
            if (e == cudaSuccess) e = cudaMemcpyAsync(d_slots, slots.data(), P * 4, cudaMemcpyHostToDevice, stream);
            if (e == cudaSuccess) e = launch_gather_rows(x_dev_, d_order, P, hdim, (float*)ep_send.p, stream);
            launches++;
            if (e != cudaSuccess) return cuda_fail(e, "ep gather");
        }
        auto exchange = [&](const float* sendbuf, const std::vector<size_t>& srows, float* recvbuf, const std::vector<size_t>& rrows) -> int {
            int rc = n.GroupStart();
            size_t so = 0, ro = 0;
            for (size_t r = 0; r < W && !rc; r++) {
                if (srows[r]) rc = n.Send(sendbuf + so * hdim, srows[r] * hdim, NCCL_FLOAT32, (int)r, comm, stream);
                if (!rc && rrows[r]) rc = n.Recv(recvbuf + ro * hdim, rrows[r] * hdim, NCCL_FLOAT32, (int)r, comm, stream);
                so += srows[r];
                ro += rrows[r];
            }
            int rc2 = n.GroupEnd();
            return rc ? rc : rc2;
        };
        nrc = exchange((const float*)ep_send.p, send_rows, (float*)ep_recv.p, recv_rows);
        if (nrc) return nccl_fail(nrc, "dispatch (ncclSend / ncclRecv)");
        // 3. the local experts: rows from rank r arrive sorted by expert with the counts every rank now knows
        if (n_recv) {
            std::vector<int32_t> lid(n_recv);
            std::vector<float> one(n_recv, 1.0f);
            size_t at = 0;
            for (size_t r = 0; r < W; r++)
                for (size_t x = 0; x < per; x++)
                    for (int32_t c = 0; c < all[r * E + (size_t)rank * per + x]; c++) lid[at++] = (int32_t)x;
            e = cudaMemsetAsync(ep_out.p, 0, n_recv * hdim * 4, stream);
            if (e != cudaSuccess) return cuda_fail(e, "ep memset");
            int rc = moe_dev(handle, (const float*)ep_recv.p, n_recv, lid.data(), one.data(), 1, (float*)ep_out.p);
            if (rc) return rc;
        }
        // 4. back, and the combine in route order
        nrc = exchange((const float*)ep_out.p, recv_rows, (float*)ep_back.p, send_rows);
        if (nrc) return nccl_fail(nrc, "combine (ncclSend / ncclRecv)");
        if (P) {
            float* d_w = (float*)(d_slots + P);
            e = cudaMemcpyAsync(d_w, rw, P * 4, cudaMemcpyHostToDevice, stream);
            if (e == cudaSuccess) e = launch_moe_combine((const float*)ep_back.p, d_slots, d_w, t, k, hdim, y_dev_, stream);
            launches++;
            if (e == cudaSuccess) e = cudaStreamSynchronize(stream);  // the host vectors above go out of scope
            if (e != cudaSuccess) return cuda_fail(e, "ep combine");
        }
        return B2_OK;
    }

    const char* stats() {
        char buf[256];
        snprintf(buf, sizeof buf, "b200qmm: %llu calls, %llu launches, copy-in %.3f ms, gpu %.3f ms, copy-out %.3f ms",
                 (unsigned long long)calls, (unsigned long long)launches, ns_in * 1e-6, ns_gpu * 1e-6, ns_out * 1e-6);
        stats_text = buf;
        return stats_text.c_str();
    }

    // ---- Backend::decode_plan (src/gpu.rs:262-289) and DecodePlan::step (src/gpu_decode.rs:538-587) ----
    int decode_plan(const b2_graph* g, uint64_t* out, int tokens = 1, bool prefill = false) {
        if (!out) return fail(B2_ERR_ARG, "[b200qmm: decode_plan: null argument]");
        DecodePlanImpl* p = nullptr;
        std::string e;
        int rc = DecodePlanImpl::create(
            g,
            [this](uint64_t h) -> const WeightDev* {
                Weight* w = find(h);
                return w ? &w->dev : nullptr;
            },
            sm_count, planes_read(), tokens, prefill, &p, e);
        if (rc) {
            err = e;
            return rc;
        }
        uint64_t h = next_handle++;
        decode_plans[h] = p;
        if (!prefill) launches += p->launches_per_step();  // the eager first pass
        for (int nt = 2; nt <= tokens && !prefill; nt++) launches += p->launches_per_step((size_t)nt);
        *out = h;
        return B2_OK;
    }
    DecodePlanImpl* find_plan(uint64_t h) {
        auto it = decode_plans.find(h);
        return it == decode_plans.end() ? nullptr : it->second;
    }
    int plan_free(uint64_t h) {
        auto it = decode_plans.find(h);
        if (it == decode_plans.end()) return fail(B2_ERR_ARG, "[b200qmm: plan_free: unknown plan]");
        cudaStreamSynchronize(stream);
        delete it->second;
        decode_plans.erase(it);
        return B2_OK;
    }
    int plan_step(uint64_t h, size_t pos, const float* x, const float* rope_cs, float* hidden, float* logits) {
        DecodePlanImpl* p = find_plan(h);
        if (!p) return fail(B2_ERR_ARG, "[b200qmm: plan_step: unknown plan]");
        std::string e;
        int rc = p->step(stream, pos, x, rope_cs, hidden, logits, e);
        launches += p->launches_per_step() + 1;
        calls++;
        if (rc) err = e;
        return rc;
    }
    int plan_step_multi(uint64_t h, size_t pos, size_t t, const float* x, const float* rope_cs, float* hidden, float* logits) {
        DecodePlanImpl* p = find_plan(h);
        if (!p) return fail(B2_ERR_ARG, "[b200qmm: plan_step_multi: unknown plan]");
        std::string e;
        int rc = p->step_multi(stream, pos, t, x, rope_cs, hidden, logits, e);
        launches += p->launches_per_step(t) + 1;
        calls++;
        if (rc) err = e;
        return rc;
    }
    int plan_kv(uint64_t h, bool write, uint32_t kv, size_t pos0, size_t n, float* k, float* v) {
        DecodePlanImpl* p = find_plan(h);
        if (!p) return fail(B2_ERR_ARG, "[b200qmm: plan_kv: unknown plan]");
        std::string e;
        int rc = write ? p->kv_write(stream, kv, pos0, n, k, v, e) : p->kv_read(stream, kv, pos0, n, k, v, e);
        if (rc) err = e;
        return rc;
    }
    int plan_generate(uint64_t h, uint64_t embed, int32_t first, size_t pos0, size_t n, const float* rope, int32_t* out, float* ms) {
        DecodePlanImpl* p = find_plan(h);
        if (!p) return fail(B2_ERR_ARG, "[b200qmm: plan_generate: unknown plan]");
        Weight* w = find(embed);
        if (!w) return fail(B2_ERR_ARG, "[b200qmm: plan_generate: unknown embedding weight]");
        std::string e;
        int rc = p->generate(stream, embed, w->dev, first, pos0, n, rope, out, ms, e);
        launches += (p->launches_per_step() + 2) * n + 1;
        calls++;
        if (rc) err = e;
        return rc;
    }

    int plan_export(uint64_t h, void* out) {
        DecodePlanImpl* p = find_plan(h);
        if (!p || !out) return fail(B2_ERR_ARG, "[b200qmm: plan_export: unknown plan]");
        std::string e;
        int rc = p->export_handle(out, e);
        if (rc) err = e;
        return rc;
    }
    int plan_attach(uint64_t h, uint32_t rank, uint32_t world, const void* handles) {
        DecodePlanImpl* p = find_plan(h);
        if (!p) return fail(B2_ERR_ARG, "[b200qmm: plan_attach_peers: unknown plan]");
        std::string e;
        int rc = p->attach_peers(rank, world, handles, e);
        if (rc) err = e;
        return rc;
    }

    void close() {
        cudaStreamSynchronize(stream);
        for (auto& dp : decode_plans) delete dp.second;
        decode_plans.clear();
        for (auto& kv : weights) drop(kv.second.owned);
        weights.clear();
        for (auto& kv : moes) {
            cudaFree(kv.second.gate_up);
            cudaFree(kv.second.down);
        }
        moes.clear();
        comm_free();
        for (Scratch* sc : {&tp_stage, &tp_gather, &ep_idx, &ep_send, &ep_recv, &ep_out, &ep_back}) sc->release();
        moe_idx.release();
        moe_xg.release();
        moe_g.release();
        moe_a.release();
        moe_o.release();
        x_dev.release();
        y_dev.release();
        x16.release();
        x8.release();
        xplanes.release();
        pair_tmp.release();
        if (gemm_status) cudaFree(gemm_status);
        gemm_status = nullptr;
        for (GemmPlan* p : plans) gemm_tc_plan_destroy(p);
        plans.clear();
    }
};

}  // namespace b2

// =============================================================================================
// C ABI
// =============================================================================================
using b2::Backend;

struct b2_ctx {
    Backend be;
};

static std::string g_open_error;
static std::mutex g_open_mu;

#define B2_EXPORT extern "C" __attribute__((visibility("default")))
#define LOCKED(ctx)                                  \
    if (!(ctx)) return B2_ERR_ARG;                   \
    std::lock_guard<std::mutex> lock_((ctx)->be.mu); \
    if (!(ctx)->be.bind()) return (ctx)->be.fail(B2_ERR_CUDA, "[b200qmm: cudaSetDevice failed]");

B2_EXPORT int b2_open(int ordinal, b2_ctx** out) {
    std::lock_guard<std::mutex> lock(g_open_mu);
    if (!out) return B2_ERR_ARG;
    *out = nullptr;
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess || n == 0) {
        g_open_error = std::string("[b200qmm: no CUDA device: ") + cudaGetErrorString(e) + "]";
        cudaGetLastError();
        return B2_DECLINED;
    }
    if (ordinal < 0 || ordinal >= n) {
        g_open_error = "[b200qmm: no such device ordinal]";
        return B2_DECLINED;
    }
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, ordinal) != cudaSuccess) {
        g_open_error = "[b200qmm: cudaGetDeviceProperties failed]";
        return B2_ERR_CUDA;
    }
    if (prop.major != 10) {
        g_open_error = "[b200qmm: device is sm_" + std::to_string(prop.major) + std::to_string(prop.minor) +
                       ", the kernels are built for sm_100a only]";
        return B2_DECLINED;
    }
    if (cudaSetDevice(ordinal) != cudaSuccess) {
        g_open_error = "[b200qmm: cudaSetDevice failed]";
        return B2_ERR_CUDA;
    }
    b2_ctx* c = new b2_ctx();
    c->be.device = ordinal;
    c->be.sm_count = prop.multiProcessorCount;
    *out = c;
    return B2_OK;
}

B2_EXPORT void b2_close(b2_ctx* ctx) {
    if (!ctx) return;
    {
        std::lock_guard<std::mutex> lock(ctx->be.mu);
        if (ctx->be.bind()) ctx->be.close();
    }
    delete ctx;
}

B2_EXPORT const char* b2_last_error(b2_ctx* ctx) { return ctx ? ctx->be.err.c_str() : "[b200qmm: null context]"; }
B2_EXPORT const char* b2_open_error(void) { return g_open_error.c_str(); }

B2_EXPORT int b2_set_chained(b2_ctx* ctx, int on) {
    LOCKED(ctx);
    ctx->be.chained = on != 0;
    return B2_OK;
}

B2_EXPORT int b2_set_fast_planes(b2_ctx* ctx, int on) {
    if (!ctx) return B2_ERR_ARG;
    ctx->be.fast_planes = on != 0;
    return B2_OK;
}
B2_EXPORT int b2_set_exact(b2_ctx* ctx, int on) {
    LOCKED(ctx);
    ctx->be.exact = on != 0;
    return B2_OK;
}

B2_EXPORT int b2_set_fp8_activations(b2_ctx* ctx, int on) {
    LOCKED(ctx);
    ctx->be.fp8_act = on != 0;
    return B2_OK;
}

B2_EXPORT int b2_set_stream(b2_ctx* ctx, void* s) {
    LOCKED(ctx);
    ctx->be.stream = (cudaStream_t)s;
    return B2_OK;
}

B2_EXPORT const char* b2_stats(b2_ctx* ctx) {
    if (!ctx) return "";
    std::lock_guard<std::mutex> lock(ctx->be.mu);
    return ctx->be.stats();
}

B2_EXPORT uint64_t b2_launch_count(b2_ctx* ctx) { return ctx ? ctx->be.launches : 0; }

B2_EXPORT int b2_wants(b2_ctx* ctx, size_t n_out, size_t n_in, size_t t) { return ctx && ctx->be.wants(n_out, n_in, t) ? 1 : 0; }

B2_EXPORT int b2_upload_mlx4(b2_ctx* ctx, const uint32_t* w, const uint16_t* scales, const uint16_t* biases, size_t n_out, size_t n_in,
                             size_t group, b2_weight* out) {
    LOCKED(ctx);
    return ctx->be.upload_mlx4(w, scales, biases, n_out, n_in, group, out);
}

B2_EXPORT int b2_upload_q4(b2_ctx* ctx, const uint8_t* q, const uint16_t* scales, const uint16_t* offsets, size_t group, size_t n_out, size_t n_in,
                           b2_weight* out) {
    LOCKED(ctx);
    return ctx->be.upload_q4(q, scales, offsets, group, n_out, n_in, out);
}

B2_EXPORT int b2_upload_gguf(b2_ctx* ctx, int fmt, const uint8_t* data, size_t n_out, size_t n_in, const float* block_scales,
                             size_t bs_rows, size_t bs_cols, b2_weight* out) {
    LOCKED(ctx);
    return ctx->be.upload_gguf(fmt, data, n_out, n_in, block_scales, bs_rows, bs_cols, out);
}

B2_EXPORT int b2_shard_rows(b2_ctx* ctx, b2_weight w, size_t r0, size_t r1, b2_weight* out) {
    LOCKED(ctx);
    return ctx->be.shard_rows(w, r0, r1, out);
}

B2_EXPORT int b2_free_weight(b2_ctx* ctx, b2_weight w) {
    LOCKED(ctx);
    return ctx->be.free_weight(w);
}

B2_EXPORT size_t b2_weight_bytes(b2_ctx* ctx, b2_weight w) {
    if (!ctx) return 0;
    std::lock_guard<std::mutex> lock(ctx->be.mu);
    b2::Weight* p = ctx->be.find(w);
    return p ? p->bytes : 0;
}

B2_EXPORT int b2_dequantize_rows(b2_ctx* ctx, b2_weight w, size_t r0, size_t r1, float* out) {
    LOCKED(ctx);
    return ctx->be.dequantize_rows(w, r0, r1, out);
}

B2_EXPORT int b2_dequantize_rows_dev(b2_ctx* ctx, b2_weight w, size_t r0, size_t r1, float* out_dev) {
    LOCKED(ctx);
    return ctx->be.dequantize_rows_dev(w, r0, r1, out_dev);
}

B2_EXPORT int b2_matmul(b2_ctx* ctx, const float* x, size_t t, size_t n_in, b2_job* jobs, size_t n_jobs) {
    LOCKED(ctx);
    return ctx->be.matmul(x, t, n_in, jobs, n_jobs);
}

B2_EXPORT int b2_matvec_rows(b2_ctx* ctx, const float* x, size_t t, size_t n_in, b2_rows_job* jobs, size_t n_jobs) {
    LOCKED(ctx);
    return ctx->be.matvec_rows(x, t, n_in, jobs, n_jobs);
}

B2_EXPORT int b2_matmul_dev(b2_ctx* ctx, b2_weight w, const void* x_dev, int x_dtype, size_t t, void* y_dev, int y_dtype) {
    LOCKED(ctx);
    return ctx->be.matmul_dev(w, x_dev, x_dtype, t, y_dev, y_dtype);
}

B2_EXPORT int b2_matvec_dev(b2_ctx* ctx, b2_weight w, b2_weight up, const float* x_dev, float* y_dev, int mode, const float* gate_dev) {
    LOCKED(ctx);
    return ctx->be.matvec_dev(w, up, x_dev, y_dev, mode, gate_dev);
}

B2_EXPORT int b2_upload_moe(b2_ctx* ctx, const b2_weight* gate_up, const b2_weight* down, size_t experts, size_t h, size_t inter, b2_moe_handle* out) {
    LOCKED(ctx);
    return ctx->be.upload_moe(gate_up, nullptr, down, experts, h, inter, B2_ACT_SILU, 0.0f, out);
}

B2_EXPORT int b2_upload_moe_ex(b2_ctx* ctx, const b2_weight* gate_up, const b2_weight* up, const b2_weight* down, size_t experts, size_t h, size_t inter,
                               int act, float act_limit, b2_moe_handle* out) {
    LOCKED(ctx);
    return ctx->be.upload_moe(gate_up, up, down, experts, h, inter, act, act_limit, out);
}

B2_EXPORT int b2_free_moe(b2_ctx* ctx, b2_moe_handle m) {
    LOCKED(ctx);
    return ctx->be.free_moe(m);
}

B2_EXPORT int b2_moe(b2_ctx* ctx, b2_moe_handle m, const float* x, size_t t, const int32_t* route_ids, const float* route_w, size_t k, float* y) {
    LOCKED(ctx);
    return ctx->be.moe(m, x, t, route_ids, route_w, k, y);
}

B2_EXPORT int b2_moe_dev(b2_ctx* ctx, b2_moe_handle m, const float* x_dev, size_t t, const int32_t* route_ids, const float* route_w, size_t k,
                         float* y_dev) {
    LOCKED(ctx);
    return ctx->be.moe_dev(m, x_dev, t, route_ids, route_w, k, y_dev);
}

B2_EXPORT int b2_route_topk_dev(b2_ctx* ctx, const float* logits_dev, size_t t, size_t n_experts, size_t k, int32_t* ids_dev, float* w_dev) {
    LOCKED(ctx);
    return ctx->be.route_topk(logits_dev, t, n_experts, k, ids_dev, w_dev);
}

B2_EXPORT int b2_prepare_x_dev(b2_ctx* ctx, const float* x_dev, size_t n_in) {
    LOCKED(ctx);
    return ctx->be.prepare_x(x_dev, n_in);
}

B2_EXPORT int b2_matvec_prepared_dev(b2_ctx* ctx, b2_weight w, b2_weight up, const float* x_dev, float* y_dev, int mode,
                                     const float* gate_dev) {
    LOCKED(ctx);
    return ctx->be.matvec_prepared(w, up, x_dev, y_dev, mode, gate_dev);
}

// Reads (and clears) the status word of the tensor-core GEMM after the caller synchronized the
// stream: B2_OK, or B2_ERR_TIMEOUT with the place where a bounded device wait gave up.
B2_EXPORT int b2_check_status(b2_ctx* ctx) {
    LOCKED(ctx);
    return ctx->be.check_gemm_status();
}

B2_EXPORT int b2_comm_unique_id(void* id_out) {
    const b2::NcclApi& n = b2::nccl_api();
    if (!id_out) return B2_ERR_ARG;
    if (!n.ok) return B2_DECLINED;
    b2::NcclId id;
    if (n.GetUniqueId(&id)) return B2_ERR_CUDA;
    std::memcpy(id_out, &id, sizeof id);
    return B2_OK;
}

B2_EXPORT int b2_comm_init(b2_ctx* ctx, int world, int rank, const void* id) {
    LOCKED(ctx);
    return ctx->be.comm_init(world, rank, id);
}

B2_EXPORT int b2_comm_free(b2_ctx* ctx) {
    LOCKED(ctx);
    return ctx->be.comm_free();
}

B2_EXPORT int b2_matmul_sharded(b2_ctx* ctx, b2_weight w_shard, const void* x_dev, int x_dtype, size_t t, float* y_dev) {
    LOCKED(ctx);
    return ctx->be.matmul_sharded(w_shard, x_dev, x_dtype, t, y_dev);
}

B2_EXPORT int b2_matmul_sharded_peer(b2_ctx* ctx, b2_weight w_shard, const void* x_dev, int x_dtype, size_t t, float** y_full_dev) {
    LOCKED(ctx);
    return ctx->be.matmul_sharded_peer(w_shard, x_dev, x_dtype, t, y_full_dev);
}

B2_EXPORT int b2_moe_ep(b2_ctx* ctx, b2_moe_handle m, size_t n_experts_global, const float* x_dev, size_t t, const int32_t* route_ids,
                        const float* route_w, size_t k, float* y_dev) {
    LOCKED(ctx);
    return ctx->be.moe_ep(m, n_experts_global, x_dev, t, route_ids, route_w, k, y_dev);
}

B2_EXPORT int b2_decode_plan(b2_ctx* ctx, const b2_graph* graph, b2_plan* out) {
    LOCKED(ctx);
    return ctx->be.decode_plan(graph, out);
}

B2_EXPORT int b2_decode_plan_multi(b2_ctx* ctx, const b2_graph* graph, size_t tokens, b2_plan* out) {
    LOCKED(ctx);
    if (tokens == 0) return ctx->be.fail(B2_ERR_ARG, "[b200qmm: decode_plan_multi: a step has at least one token]");
    if (tokens > B2_PLAN_MAX_TOKENS) return ctx->be.fail(B2_DECLINED, "[b200qmm: decode_plan_multi: steps of at most four tokens are taken]");
    return ctx->be.decode_plan(graph, out, (int)tokens);
}

B2_EXPORT int b2_plan_step_multi(b2_ctx* ctx, b2_plan plan, size_t pos, size_t t, const float* x, const float* rope_cs, float* hidden,
                                 float* logits) {
    LOCKED(ctx);
    return ctx->be.plan_step_multi(plan, pos, t, x, rope_cs, hidden, logits);
}

B2_EXPORT int b2_decode_plan_prefill(b2_ctx* ctx, const b2_graph* graph, size_t tokens, b2_plan* out) {
    LOCKED(ctx);
    if (tokens == 0) return ctx->be.fail(B2_ERR_ARG, "[b200qmm: decode_plan_prefill: a step has at least one token]");
    if (tokens > B2_PREFILL_MAX_TOKENS) return ctx->be.fail(B2_DECLINED, "[b200qmm: decode_plan_prefill: steps of at most 8192 tokens are taken]");
    return ctx->be.decode_plan(graph, out, (int)tokens, true);
}

B2_EXPORT int b2_plan_last_step_ms(b2_ctx* ctx, b2_plan plan, float* ms) {
    LOCKED(ctx);
    b2::DecodePlanImpl* p = ctx->be.find_plan(plan);
    if (!p || !ms) return ctx->be.fail(B2_ERR_ARG, "[b200qmm: plan_last_step_ms: unknown plan or null argument]");
    *ms = p->last_step_ms();
    return B2_OK;
}

B2_EXPORT int b2_plan_tokens(b2_ctx* ctx, b2_plan plan, size_t* out) {
    LOCKED(ctx);
    b2::DecodePlanImpl* p = ctx->be.find_plan(plan);
    if (!p || !out) return ctx->be.fail(B2_ERR_ARG, "[b200qmm: plan_tokens: unknown plan or null argument]");
    *out = (size_t)p->tokens();
    return B2_OK;
}

B2_EXPORT int b2_plan_free(b2_ctx* ctx, b2_plan plan) {
    LOCKED(ctx);
    return ctx->be.plan_free(plan);
}

B2_EXPORT int b2_plan_step(b2_ctx* ctx, b2_plan plan, size_t pos, const float* x, const float* rope_cs, float* hidden, float* logits) {
    LOCKED(ctx);
    return ctx->be.plan_step(plan, pos, x, rope_cs, hidden, logits);
}

B2_EXPORT int b2_plan_kv_write(b2_ctx* ctx, b2_plan plan, uint32_t kv, size_t pos0, size_t n, const float* k, const float* v) {
    LOCKED(ctx);
    return ctx->be.plan_kv(plan, true, kv, pos0, n, const_cast<float*>(k), const_cast<float*>(v));
}

B2_EXPORT int b2_plan_kv_read(b2_ctx* ctx, b2_plan plan, uint32_t kv, size_t pos0, size_t n, float* k, float* v) {
    LOCKED(ctx);
    return ctx->be.plan_kv(plan, false, kv, pos0, n, k, v);
}

B2_EXPORT int b2_plan_generate(b2_ctx* ctx, b2_plan plan, b2_weight embed, int32_t first_token, size_t pos0, size_t n_tokens,
                               const float* rope_cs_table, int32_t* out_tokens, float* elapsed_ms) {
    LOCKED(ctx);
    return ctx->be.plan_generate(plan, embed, first_token, pos0, n_tokens, rope_cs_table, out_tokens, elapsed_ms);
}

B2_EXPORT int b2_plan_launches(b2_ctx* ctx, b2_plan plan, uint64_t* per_step) {
    LOCKED(ctx);
    b2::DecodePlanImpl* p = ctx->be.find_plan(plan);
    if (!p || !per_step) return ctx->be.fail(B2_ERR_ARG, "[b200qmm: plan_launches: unknown plan]");
    *per_step = p->launches_per_step();
    return B2_OK;
}

B2_EXPORT int b2_plan_export(b2_ctx* ctx, b2_plan plan, void* handle_out) {
    LOCKED(ctx);
    return ctx->be.plan_export(plan, handle_out);
}

B2_EXPORT int b2_plan_attach_peers(b2_ctx* ctx, b2_plan plan, uint32_t rank, uint32_t world, const void* handles) {
    LOCKED(ctx);
    return ctx->be.plan_attach(plan, rank, world, handles);
}
