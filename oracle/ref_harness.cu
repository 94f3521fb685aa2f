// Test infrastructure only: a host harness around the REFERENCE's own CUDA kernels, used as a second, GPU-side
// oracle and baseline: the MLX-4 matrix-vector product (dmv_q4a), the MLX-4 prefill product (gemm_q4a) and the decode
// ops around them (dnorm, dqk_rope, dattn_* + dattn_combine, dglu). The kernels are not in this repository:
// build_ref.py assembles them at build time from the reference's tree (the KERNEL_SRC string of src/cuda.rs followed
// by src/cuda_decode.cu, which is how src/cuda.rs:477 builds its NVRTC module) into _ref/ref_kernels.cuh, and this file
// includes that. Launch geometry as the reference's host code: for the matrix-vector product 4 warps per block,
// DMV_NR = 4 rows per warp (src/cuda_decode.rs:32-34), arguments as `DW` (src/cuda_decode.cu:27).
#include <cuda_runtime.h>

#include "_ref/ref_kernels.cuh"

#define REF_API extern "C" __attribute__((visibility("default")))

// y[n_out] = W x with the reference's dmv_q4a (affine Q4: Q4_0-layout nibbles, f16 scale per 32, bf16 offset per group).
// All pointers are device pointers. Runs `iters` launches and returns the mean device time of one in *ms_per_iter
// (CUDA events on `stream`); returns a cudaError_t value.
REF_API int ref_dmv_q4a(const void* q, const void* scales, const void* offsets, unsigned int groups_per_row, unsigned int blocks_per_group,
                        const float* x, float* y, unsigned int n_out, unsigned int n_in, int iters, float* ms_per_iter, void* stream) {
    DW w;
    w.q = (const unsigned char*)q;
    w.s = (const unsigned char*)scales;
    w.o = (const unsigned short*)offsets;
    w.gpr = groups_per_row;
    w.gk = blocks_per_group;
    cudaStream_t st = (cudaStream_t)stream;
    const unsigned int rows_per_block = 4 * DMV_NR;
    const dim3 grid((n_out + rows_per_block - 1) / rows_per_block), block(4 * 32);
    cudaEvent_t e0, e1;
    cudaEventCreate(&e0);
    cudaEventCreate(&e1);
    dmv_q4a<<<grid, block, 0, st>>>(w, w, x, y, n_out, n_in, 0u, nullptr);  // warm-up (and the result)
    cudaEventRecord(e0, st);
    for (int i = 0; i < iters; i++) dmv_q4a<<<grid, block, 0, st>>>(w, w, x, y, n_out, n_in, 0u, nullptr);
    cudaEventRecord(e1, st);
    cudaError_t e = cudaStreamSynchronize(st);
    float ms = 0.0f;
    if (e == cudaSuccess) e = cudaEventElapsedTime(&ms, e0, e1);
    if (ms_per_iter) *ms_per_iter = iters > 0 ? ms / iters : 0.0f;
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    if (e == cudaSuccess) e = cudaGetLastError();
    return (int)e;
}

// ---- the reference's decode ops other than the product (src/cuda_decode.cu), launched as src/cuda_decode.rs:1303-1365 launches them ----

// out[rows][n] = rmsnorm(x * pre) * w (w may be null): dnorm, a block per row of min(1024, n rounded up to 32) threads.
REF_API int ref_norm(const float* x, float* out, const float* w, unsigned int n, unsigned int rows, float eps, float pre, unsigned int add,
                     void* stream) {
    DNP p;
    p.n = n;
    p.eps = eps;
    p.has_w = w != nullptr;
    p.add = add;
    p.x_stride = n;
    p.o_stride = n;
    p.pre = pre;
    p._p = 0;
    unsigned int threads = (n + 31) / 32 * 32;
    if (threads > 1024) threads = 1024;
    dnorm<<<rows, threads, 0, (cudaStream_t)stream>>>(x, out, w, p);
    cudaError_t e = cudaStreamSynchronize((cudaStream_t)stream);
    return (int)(e == cudaSuccess ? cudaGetLastError() : e);
}

// The token's attention inputs: dqk_rope over qkv = [q heads | k heads | v heads]; caches [position][n_kv][hd] f32,
// position = sp[0] (a device word array of 4). qn / kn: per-head norm weights or null.
REF_API int ref_qk_rope(const float* qkv, float* q_out, float* kc, float* vc, float* k_out, float* v_out, const float* qn, const float* kn,
                        const float* cs, const unsigned int* sp, unsigned int nh, unsigned int nkv, unsigned int hd, unsigned int half_rot,
                        unsigned int interleaved, float eps, void* stream) {
    DQP p;
    p.nh = nh;
    p.nkv = nkv;
    p.hd = hd;
    p.half_rot = half_rot;
    p.q_stride = hd;
    p.k_off = nh * hd;
    p.v_off = (nh + nkv) * hd;
    p.interleaved = interleaved;
    p.has_qn = qn != nullptr;
    p.has_kn = kn != nullptr;
    p.v_norm = 0;
    p.v_from_k = 0;
    p.eps = eps;
    p._p[0] = p._p[1] = p._p[2] = 0;
    dqk_rope<<<nh + 2 * nkv, hd, 0, (cudaStream_t)stream>>>(qkv, q_out, kc, vc, k_out, v_out, qn, kn, cs, sp, p);
    cudaError_t e = cudaStreamSynchronize((cudaStream_t)stream);
    return (int)(e == cudaSuccess ? cudaGetLastError() : e);
}

// One query per head over cache positions 0 .. sp[0]: dattn_<hd/32>_<grp> then dattn_combine; `part` holds
// nh * 64 * (hd + 2) floats. grp = the largest of 8, 4, 2, 1 that divides the heads per KV head and has a kernel for hd
// (src/cuda_decode.rs:833). Runs the pair `iters` times after one warm-up and returns the mean device time of a pair.
REF_API int ref_attend(const float* q, const float* kc, const float* vc, float* out, float* part, const unsigned int* sp, unsigned int nh,
                       unsigned int nkv, unsigned int hd, float scale, unsigned int window, int iters, float* ms_per_iter, void* stream) {
    DAP p;
    p.nh = nh;
    p.nkv = nkv;
    p.window = window;
    p.has_gate = 0;
    p.g_stride = 0;
    p.block = 0;
    p.scale = scale;
    p._q = 0;
    typedef void (*attn_fn)(const float*, const float*, const float*, float*, const float*, float*, const unsigned int*, DAP);
    attn_fn f = nullptr;
    unsigned int grp = 0;
    const unsigned int rep = nh / nkv, cand[4] = {8, 4, 2, 1};
    for (int i = 0; i < 4 && !f; i++) {
        const unsigned int g = cand[i];
        if (rep % g) continue;
        if (hd == 64) f = g == 8 ? dattn_2_8 : g == 4 ? dattn_2_4 : g == 2 ? dattn_2_2 : dattn_2_1;
        else if (hd == 128) f = g == 8 ? nullptr : g == 4 ? dattn_4_4 : g == 2 ? dattn_4_2 : dattn_4_1;
        else if (hd == 256) f = g == 2 ? dattn_8_2 : g == 1 ? dattn_8_1 : nullptr;
        else if (hd == 512) f = g == 1 ? dattn_16_1 : nullptr;
        if (f) grp = g;
    }
    if (!f) return (int)cudaErrorInvalidValue;
    cudaStream_t st = (cudaStream_t)stream;
    cudaEvent_t e0, e1;
    cudaEventCreate(&e0);
    cudaEventCreate(&e1);
    const dim3 grid(nh / grp, 64);
    f<<<grid, 256, 0, st>>>(q, kc, vc, out, nullptr, part, sp, p);
    dattn_combine<<<nh, 256, 0, st>>>(part, out, nullptr, sp, p, hd);
    cudaEventRecord(e0, st);
    for (int i = 0; i < iters; i++) {
        f<<<grid, 256, 0, st>>>(q, kc, vc, out, nullptr, part, sp, p);
        dattn_combine<<<nh, 256, 0, st>>>(part, out, nullptr, sp, p, hd);
    }
    cudaEventRecord(e1, st);
    cudaError_t e = cudaStreamSynchronize(st);
    float ms = 0.0f;
    if (e == cudaSuccess) e = cudaEventElapsedTime(&ms, e0, e1);
    if (ms_per_iter) *ms_per_iter = iters > 0 ? ms / iters : 0.0f;
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    if (e == cudaSuccess) e = cudaGetLastError();
    return (int)e;
}

// out = silu(g) * u (gelu != 0: the tanh GELU): dglu.
REF_API int ref_glu(const float* g, const float* u, float* out, unsigned int n, unsigned int gelu, void* stream) {
    dglu<<<(n + 255) / 256, 256, 0, (cudaStream_t)stream>>>(g, u, out, n, gelu);
    cudaError_t e = cudaStreamSynchronize((cudaStream_t)stream);
    return (int)(e == cudaSuccess ? cudaGetLastError() : e);
}

// y[tokens][n_out] = x[tokens][n_in] W^T with the reference's prefill kernel gemm_q4a (the KERNEL_SRC string of
// src/cuda.rs: 64 x 64 tiles, f32 FMA, 256 threads); n_out and tokens must be multiples of 64 (its host code pads).
// Runs `iters` launches after one warm-up and returns the mean device time of one.
REF_API int ref_gemm_q4a(const void* q, const void* scales, const void* offsets, unsigned int groups_per_row, unsigned int blocks_per_group,
                         const float* x, float* y, unsigned int n_out, unsigned int n_in, unsigned int tokens, int iters, float* ms_per_iter,
                         void* stream) {
    if (n_out % 64 || tokens % 64 || n_in % 32) return (int)cudaErrorInvalidValue;
    cudaStream_t st = (cudaStream_t)stream;
    const dim3 grid(n_out / 64, tokens / 64);
    cudaEvent_t e0, e1;
    cudaEventCreate(&e0);
    cudaEventCreate(&e1);
    gemm_q4a<<<grid, 256, 0, st>>>((const unsigned char*)q, (const unsigned short*)scales, x, y, n_out, n_in, (const unsigned short*)offsets,
                                   groups_per_row, blocks_per_group);
    cudaEventRecord(e0, st);
    for (int i = 0; i < iters; i++)
        gemm_q4a<<<grid, 256, 0, st>>>((const unsigned char*)q, (const unsigned short*)scales, x, y, n_out, n_in,
                                       (const unsigned short*)offsets, groups_per_row, blocks_per_group);
    cudaEventRecord(e1, st);
    cudaError_t e = cudaStreamSynchronize(st);
    float ms = 0.0f;
    if (e == cudaSuccess) e = cudaEventElapsedTime(&ms, e0, e1);
    if (ms_per_iter) *ms_per_iter = iters > 0 ? ms / iters : 0.0f;
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    if (e == cudaSuccess) e = cudaGetLastError();
    return (int)e;
}

// One routed-expert layer with the reference's own kernels, launched as CudaBackend::moe_run launches them
// (src/cuda.rs:798-966): moe_gather over per-expert segments padded to the GEMM's 64-row tile, one gemm_q4a per touched
// expert for the fused gate_up projection, moe_act (SiLU), one gemm_q4a per touched expert for the down projection,
// moe_combine in route order. The caller builds the segment tables the way moe_run does (host arrays seg_start / seg_len in
// rows, device arrays src [rows] and slots [2 t k] = (row, weight bits) pairs) and passes the experts' Q4Matrix arrays as
// host tables of device pointers. Scratch (device): xs [rows][h], gu [rows][2 mi], a [rows][mi], o [rows][h] f32.
// y [t][h] is added to (the caller resets it between calls if it wants one layer's result). Runs the sequence `iters`
// times after one warm-up and returns the mean device time of one sequence.
REF_API int ref_moe_q4a(const void* const* gu_q, const void* const* gu_s, const void* const* gu_o, const void* const* dn_q, const void* const* dn_s,
                        const void* const* dn_o, unsigned int n_experts, unsigned int h, unsigned int mi, unsigned int group, const float* x,
                        unsigned int t, unsigned int k, const unsigned int* src, const unsigned int* slots, const unsigned int* seg_start,
                        const unsigned int* seg_len, unsigned int rows, float* xs, float* gu, float* a, float* o, float* y, int iters,
                        float* ms_per_iter, void* stream) {
    if (h % 64 || mi % 64 || (2 * mi) % 64 || h % 32 || mi % 32) return (int)cudaErrorInvalidValue;
    cudaStream_t st = (cudaStream_t)stream;
    const unsigned int cols = (h + 255) / 256 < 64 ? (h + 255) / 256 : 64;
    auto once = [&]() {
        moe_gather<<<dim3(cols, rows), 256, 0, st>>>(x, src, xs, h, t);
        for (unsigned int e = 0; e < n_experts; e++) {
            if (!seg_len[e]) continue;
            gemm_q4a<<<dim3(2 * mi / 64, seg_len[e] / 64), 256, 0, st>>>((const unsigned char*)gu_q[e], (const unsigned short*)gu_s[e],
                                                                          xs + (size_t)seg_start[e] * h, gu + (size_t)seg_start[e] * 2 * mi, 2 * mi, h,
                                                                          (const unsigned short*)gu_o[e], h / group, group / 32);
        }
        moe_act<<<(unsigned int)(((size_t)rows * mi + 255) / 256), 256, 0, st>>>(gu, a, rows, mi, 0u, 0u, 0.0f);
        for (unsigned int e = 0; e < n_experts; e++) {
            if (!seg_len[e]) continue;
            gemm_q4a<<<dim3(h / 64, seg_len[e] / 64), 256, 0, st>>>((const unsigned char*)dn_q[e], (const unsigned short*)dn_s[e],
                                                                     a + (size_t)seg_start[e] * mi, o + (size_t)seg_start[e] * h, h, mi,
                                                                     (const unsigned short*)dn_o[e], mi / group, group / 32);
        }
        moe_combine<<<dim3(cols, t), 256, 0, st>>>(o, slots, y, h, k);
    };
    cudaEvent_t e0, e1;
    cudaEventCreate(&e0);
    cudaEventCreate(&e1);
    once();
    cudaEventRecord(e0, st);
    for (int i = 0; i < iters; i++) once();
    cudaEventRecord(e1, st);
    cudaError_t e = cudaStreamSynchronize(st);
    float ms = 0.0f;
    if (e == cudaSuccess) e = cudaEventElapsedTime(&ms, e0, e1);
    if (ms_per_iter) *ms_per_iter = iters > 0 ? ms / iters : 0.0f;
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    if (e == cudaSuccess) e = cudaGetLastError();
    return (int)e;
}
