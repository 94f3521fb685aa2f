/*
 * b200qmm - C ABI of the B200 (sm_100a) quantized-matmul engine for oxinfer.
 *
 * The library is loaded at run time (dlopen / libloading / ctypes); nothing here needs to be
 * linked when the host program is built. It carries its CUDA runtime statically and finds the
 * driver (libcuda.so.1) itself on first use, so it loads on machines without a GPU and every
 * entry point then returns an error instead of crashing.
 *
 * Each entry point replaces one method of oxinfer's accelerator boundary, the `Backend` trait of
 * src/gpu.rs:151-294 as implemented for CUDA in src/cuda.rs; the citation beside each
 * declaration names the method. Conventions carried over from that trait:
 *   - nothing panics or aborts across the boundary (src/gpu.rs:158-160): a return of 0 means the
 *     work was done, > 0 means "declined, run it on the CPU" (B2_DECLINED), < 0 is an error whose
 *     text b2_last_error returns. In both non-zero cases no output was written.
 *   - host buffers stay owned by the caller and are only read during the call;
 *   - weights are uploaded once and referred to by opaque 64-bit handles.
 *
 * Matrices are row-major `[n_out][n_in]` ("out x in"), activations `[t][n_in]`, results
 * `[t][n_out]`, exactly as src/gpu.rs:60-75 lays them out.
 */
#ifndef B200QMM_H
#define B200QMM_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B2_OK 0
#define B2_DECLINED 1
#define B2_ERR_CUDA (-1)
#define B2_ERR_ARG (-2)
#define B2_ERR_NOMEM (-3)
#define B2_ERR_TIMEOUT (-4)

/* Weight formats. The GGUF ones keep the ids of src/ggml.rs:42-93. */
#define B2_FMT_MLX4 1      /* MLX affine 4-bit, u32 words + bf16 scale/bias per group (src/quant.rs:518-563) */
#define B2_FMT_Q8_0 8      /* GGUF Q8_0  (src/ggml.rs:707-712) */
#define B2_FMT_Q4_K 12     /* GGUF Q4_K  (src/ggml.rs:750-773) */
#define B2_FMT_Q6_K 14     /* GGUF Q6_K  (src/ggml.rs:774-793) */
#define B2_FMT_F8E4M3 4096 /* FP8 e4m3fn + f32 block scales (src/ggml.rs:240-293,433-443) */
/* The other GGUF block formats b2_upload_gguf takes (ids of src/ggml.rs:42-93; decode arms src/ggml.rs:665-706, 713-773,
 * 915-960): kept as raw GGUF rows on the device, dequantized bit-exactly, multiplied by one generic (untuned) matrix-vector
 * kernel at any number of tokens, f32 activations and results; no MoE / decode-plan use. */
#define B2_FMT_Q4_0 2
#define B2_FMT_Q4_1 3
#define B2_FMT_Q5_0 6
#define B2_FMT_Q5_1 7
#define B2_FMT_Q2_K 10
#define B2_FMT_Q3_K 11
#define B2_FMT_Q5_K 13
#define B2_FMT_IQ4_NL 20
#define B2_FMT_IQ4_XS 23
#define B2_FMT_MXFP4 39
#define B2_FMT_NVFP4 40 /* blocks of 64 E2M1 values, an unsigned E4M3 scale per 16 (src/ggml.rs:79-83, 936-947); block_scales may
                          carry the tensor's global scale (one value for the whole matrix: bs_rows >= n_out, bs_cols >= n_in) */

/* Element types of device-resident activations / results. */
#define B2_F32 0
#define B2_BF16 1
#define B2_F16 2

/* Output modes of a matrix-vector product: the five modes of dmv_out, src/cuda_decode.cu:131-137. */
#define B2_MODE_STORE 0     /* y = a */
#define B2_MODE_ADD 1       /* y += a */
#define B2_MODE_SILU_PAIR 2 /* y = silu(a) * b, b from a second matrix of the same shape */
#define B2_MODE_GELU_PAIR 3 /* y = gelu_tanh(a) * b */
#define B2_MODE_ADD_GATED 4 /* y += a * sigmoid(gate[0]) */

typedef struct b2_ctx b2_ctx;
typedef uint64_t b2_weight;
typedef uint64_t b2_moe_handle;

/* One matmul of a batch sharing the input x: `Job` of src/gpu.rs:60-65. */
typedef struct {
    b2_weight w;
    size_t n_out;
    float* y; /* host, [t][n_out] */
} b2_job;

/* One matrix-vector job of `matvec_rows`: `RowsJob` of src/gpu.rs:69-75. `up` = 0 for a plain
 * product, else y = silu(W x) * (U x). */
typedef struct {
    b2_weight w;
    b2_weight up;
    size_t n_out;
    float* y; /* host, [t][n_out] */
} b2_rows_job;

/* ---- lifetime ---------------------------------------------------------------------------- */

/* Replaces CudaBackend::new(ordinal), src/cuda.rs:448-570: binds device `ordinal` (its primary
 * context, shared with any other CUDA runtime user in the process) and checks that it is an
 * sm_100 part. B2_DECLINED when there is no driver, no such device or another architecture. */
int b2_open(int ordinal, b2_ctx** out);
void b2_close(b2_ctx* ctx);
/* Text of the last error on this context (valid until the next call on it). */
const char* b2_last_error(b2_ctx* ctx);
/* Library-level error for calls that have no context yet (b2_open). */
const char* b2_open_error(void);
/* Kernels are launched on `cuda_stream` (a cudaStream_t / CUstream; NULL = the default stream,
 * which is what src/cuda.rs:609-629 uses). Host-buffer entry points synchronize that stream. */
int b2_set_stream(b2_ctx* ctx, void* cuda_stream);
/* No counterpart in the reference. While on, the device-resident matrix-vector calls (b2_matvec_dev,
 * b2_matvec_prepared_dev, b2_prepare_x_dev) launch with the programmatic-dependent-launch attribute: each kernel may
 * start, and fetch its first weights, while the kernel ahead of it on the stream drains; it waits for that kernel before
 * it reads the vector or writes its output, so results are unchanged. Meant for a caller that queues a token's
 * products back to back (the decode plan does this by itself). Off by default. */
int b2_set_chained(b2_ctx* ctx, int on);
/* The boundary's exactness switch, `gpu::set_exact` / `exact()` (src/gpu.rs:313-338: "no reduced-precision matrix units").
 * Off (the default), a many-token matmul rounds activations and expanded weights to f16 operands once: results within 1e-3
 * of the f64 product per output row (FP8: 2e-3). On, the tensor-core GEMM takes every f32 / bf16 activation as two f16
 * terms and, for Q4_K, every weight as two f16 terms too (the other 4-bit and 8-bit formats' values need no second term):
 * results within 1e-4 per output row, the bound the reference holds its own f32 CUDA kernels to (src/cuda.rs:1684), at two to
 * four times the tensor-core work. Matrix-vector products (t <= 8) carry 21-bit activations either way. */
int b2_set_exact(b2_ctx* ctx, int on);
/* No counterpart in the reference, whose FP8 matrices multiply unquantized activations (src/ggml.rs:433-443; that stays the
 * default here and is what the 2e-3 parity bound refers to). On: b2_matmul / b2_matmul_dev over F8E4M3 weights with 128 x 128
 * scale blocks quantize the activations per token and per 128 k to e4m3 (scale = amax / 448, round to nearest even) and run
 * FP8 x FP8 on the tensor cores (tcgen05 kind::f8f6f4), every 128-k partial sum scaled by both scales and added in f32: the
 * large-projection form in which both operands stay 8 bits wide. The result equals the f64 product of the dequantized
 * weights with the DEQUANTIZED quantized activations to about 1e-6 per row; against unquantized activations it carries
 * e4m3's quantization noise (about 2e-2 per row). b2_set_exact takes precedence. */
int b2_set_fp8_activations(b2_ctx* ctx, int on);
/* No counterpart in the reference. Matrix-vector products (t <= 8, the decode plan, small MoE batches) multiply exact integer
 * digits of the activations, 21 bits per block of 32 in three planes; that is the default and holds a decoder layer to 1e-6
 * of the f64 oracle. On, the products read only the upper two planes (16 bits: every element rounded to 1.6e-5 of its
 * block's largest): a third fewer integer dot products, 5 % more decode tokens per second and 13 % on Q6_K, with errors of
 * 2e-5 .. 2e-4 per product row and 3e-4 through a decoder layer (inside the 1e-3 bound, not inside the default's). Read by
 * calls made, and by decode plans created, after it is set. b2_set_exact takes precedence. */
int b2_set_fast_planes(b2_ctx* ctx, int on);
/* `Backend::stats`, src/cuda.rs:1120-1132: cumulative copy-in / kernel / copy-out time as text. */
const char* b2_stats(b2_ctx* ctx);
/* Count of kernel launches issued by this context since it was opened. */
uint64_t b2_launch_count(b2_ctx* ctx);

/* ---- weights ----------------------------------------------------------------------------- */

/* `Backend::wants`, src/cuda.rs:1134-1136. 1 = offer this matmul, 0 = keep it on the CPU. */
int b2_wants(b2_ctx* ctx, size_t n_out, size_t n_in, size_t t);

/* `Backend::upload` for WeightRef::Q4 with offsets, src/cuda.rs:640-699, taking the MLX triple as
 * it is on disk (src/safetensors.rs:767-853): w `[n_out][n_in/8]` u32, scales and biases
 * `[n_out][n_in/group]` bf16 bits. group must be 64; n_in a multiple of 256. Repacked on the device into Q4_K-shaped blocks
 * that carry from_mlx_q4's values (d = f16(scale), offset = bf16(bias + 8 scale), src/quant.rs:518-563). */
int b2_upload_mlx4(b2_ctx* ctx, const uint32_t* w, const uint16_t* scales, const uint16_t* biases, size_t n_out, size_t n_in,
                   size_t group, b2_weight* out);
/* `Backend::upload` for WeightRef::Q4(&Q4Matrix) (src/gpu.rs:15-21, src/cuda.rs:640-699), the layout a backend is actually
 * handed (src/quant.rs:427-440; on the device the reference keeps it as DW{q, s, o, gpr, gk}, src/cuda_decode.cu:27):
 * q `[n_out][n_in/2]` in Q4_0 order (byte j of a 32-block = element j low nibble, element j+16 high), scales
 * `[n_out][n_in/32]` f16 bits, offsets `[n_out][n_in/group]` bf16 bits (Offsets, the affine term from_mlx_q4 adds,
 * src/quant.rs:518-563). group a multiple of 64, n_in a multiple of 256. Gives the same device blocks, bit for bit,
 * as b2_upload_mlx4 gives for the MLX triple the matrix was made from. offsets == NULL: a plain Q4 matrix (one scale per 32
 * weights, w = (nibble - 8) * scale; group is ignored, n_in a multiple of 32): what GGUF Q4_0 blocks hold, so it becomes a
 * B2_FMT_Q4_0 weight on the generic kernels. Declined (> 0): an affine matrix whose 64-groups do not share one scale. */
int b2_upload_q4(b2_ctx* ctx, const uint8_t* q, const uint16_t* scales, const uint16_t* offsets, size_t group, size_t n_out, size_t n_in,
                 b2_weight* out);
/* `Backend::upload` for WeightRef::Gguf (declined by the reference at src/cuda.rs:642): raw GGUF
 * rows of `fmt` (B2_FMT_Q4_K / Q6_K / Q8_0 / F8E4M3, or one of the other block formats above). For F8E4M3, `block_scales` is
 * `[ceil(n_out/bs_rows)][ceil(n_in/bs_cols)]` f32 (BlockScales, src/ggml.rs:250-256), else NULL. */
int b2_upload_gguf(b2_ctx* ctx, int fmt, const uint8_t* data, size_t n_out, size_t n_in, const float* block_scales, size_t bs_rows,
                   size_t bs_cols, b2_weight* out);
/* Rows [r0, r1) of an uploaded matrix as their own handle sharing the device memory (tensor-
 * parallel row shards; no counterpart in the reference, which has a single device). */
int b2_shard_rows(b2_ctx* ctx, b2_weight w, size_t r0, size_t r1, b2_weight* out);
int b2_free_weight(b2_ctx* ctx, b2_weight w);
size_t b2_weight_bytes(b2_ctx* ctx, b2_weight w);

/* The dequantized f32 values of rows [r0, r1), bit-exact with the reference's CPU decode:
 * dequantize_rows_q4 (src/quant.rs:586-606) for MLX4, GgufMatrix::dequantize_rows
 * (src/ggml.rs:409-460) for the GGUF / FP8 formats. `out` is host memory, [r1-r0][n_in]. */
int b2_dequantize_rows(b2_ctx* ctx, b2_weight w, size_t r0, size_t r1, float* out);
/* Same, into device memory. */
int b2_dequantize_rows_dev(b2_ctx* ctx, b2_weight w, size_t r0, size_t r1, float* out_dev);

/* ---- matmul ------------------------------------------------------------------------------ */

/* `Backend::matmul`, src/cuda.rs:1428-1493: y_j[t][n_out_j] = x[t][n_in] * W_j^T for every job,
 * host x and y, one submission, synchronous. */
int b2_matmul(b2_ctx* ctx, const float* x, size_t t, size_t n_in, b2_job* jobs, size_t n_jobs);

/* `Backend::matvec_rows`, src/gpu.rs:165-167 / src/cuda.rs (dmv_* kernels,
 * src/cuda_decode.cu:139-174): t in 1..4 rows of x against every job, host buffers. */
int b2_matvec_rows(b2_ctx* ctx, const float* x, size_t t, size_t n_in, b2_rows_job* jobs, size_t n_jobs);

/* Device-resident forms of the two calls above (what a decode plan issues per op,
 * src/cuda_decode.rs:1233-1410): no copies, no synchronization, launched on the context's stream.
 * x_dev is [t][n_in] of x_dtype, y_dev is [t][n_out] of y_dtype. */
int b2_matmul_dev(b2_ctx* ctx, b2_weight w, const void* x_dev, int x_dtype, size_t t, void* y_dev, int y_dtype);
/* One token: y = mode(W x [, U x]). x_dev f32 [n_in]; y_dev f32 [n_out]; gate_dev f32[1] or NULL. */
int b2_matvec_dev(b2_ctx* ctx, b2_weight w, b2_weight up, const float* x_dev, float* y_dev, int mode, const float* gate_dev);

/* ---- routed experts (MoE) ----------------------------------------------------------------- */

/* `Backend::upload_moe`, src/gpu.rs:200-215 / src/cuda.rs:777-796. The experts' matrices are uploaded
 * one by one with b2_upload_mlx4 / b2_upload_gguf (all MLX-4 or all Q4_K): gate_up[e] is the fused
 * gate/up projection [2 inter][h] (gate rows, then up rows), down[e] is [h][inter]. Their blocks are
 * copied into two stacked device buffers; the per-expert handles may be freed afterwards. h and inter
 * must be multiples of 256. The activation is SiLU (MoeAct::Silu, src/gpu.rs:36-54). */
int b2_upload_moe(b2_ctx* ctx, const b2_weight* gate_up, const b2_weight* down, size_t experts, size_t h, size_t inter, b2_moe_handle* out);
/* The full `Backend::upload_moe` (src/gpu.rs:200-215): with `up` != NULL, gate_up[e] is the gate projection [inter][h] and
 * up[e] the up projection [inter][h] (GGUF files store them apart); `act` is the layer's gated activation (MoeAct,
 * src/gpu.rs:36-54), act_limit the clamp of B2_ACT_SILU_CLAMP. Activations the reference's own CUDA backend keeps on the CPU
 * (SwigluOai, SiTU: src/cuda.rs:900-906) are declined here too. `upload_moe_transient` (src/gpu.rs:217-231) is this call
 * followed by b2_free_moe when the pass over the streamed experts is done. */
#define B2_ACT_SILU 0       /* MoeAct::Silu */
#define B2_ACT_GELU_TANH 1  /* MoeAct::GeluTanh */
#define B2_ACT_SILU_CLAMP 2 /* MoeAct::SiluClamp(limit) */
int b2_upload_moe_ex(b2_ctx* ctx, const b2_weight* gate_up, const b2_weight* up, const b2_weight* down, size_t experts, size_t h, size_t inter,
                     int act, float act_limit, b2_moe_handle* out);
int b2_free_moe(b2_ctx* ctx, b2_moe_handle m);
/* `Backend::moe`, src/gpu.rs:232-248 / src/cuda.rs:798-966: token i of x [t][h] goes through its k routes
 * (route_ids[i k + j], route_w[i k + j]) and y[i] += sum_j w_ij down(silu(gate x_i) * up x_i), added in
 * route order. Host x and y (y is read and written); routes are host arrays in both forms. */
int b2_moe(b2_ctx* ctx, b2_moe_handle m, const float* x, size_t t, const int32_t* route_ids, const float* route_w, size_t k, float* y);
/* Same with x and y resident on the device (no synchronization of the result). */
int b2_moe_dev(b2_ctx* ctx, b2_moe_handle m, const float* x_dev, size_t t, const int32_t* route_ids, const float* route_w, size_t k, float* y_dev);
/* route_top_k (src/moe.rs:180-193) / dtopk (src/cuda_decode.cu:285-312) on the device: for each of t rows
 * of n_experts logits, the k largest (ties to the lower index) and exp(l - max) / sum over the chosen. */
int b2_route_topk_dev(b2_ctx* ctx, const float* logits_dev, size_t t, size_t n_experts, size_t k, int32_t* ids_dev, float* w_dev);

/* The two halves of b2_matvec_dev, for a plan in which one vector feeds several products (q, k, v;
 * gate and up): b2_prepare_x_dev splits x into the integer planes the 4- / 6- / 8-bit kernels read
 * (the role of quantize_act, which the reference's CPU driver runs once per batch of jobs,
 * src/kernels.rs:1731-1879), b2_matvec_prepared_dev runs one product over the planes prepared last.
 * n_in must match; FP8 weights read x_dev itself. */
int b2_prepare_x_dev(b2_ctx* ctx, const float* x_dev, size_t n_in);
int b2_matvec_prepared_dev(b2_ctx* ctx, b2_weight w, b2_weight up, const float* x_dev, float* y_dev, int mode, const float* gate_dev);

/* After the caller has synchronized the stream: B2_OK, or B2_ERR_TIMEOUT when a device-side wait of
 * the tensor-core GEMM ran into its time limit (the kernel then returned early and its output is
 * not valid). The reference logs a failed launch and returns false (src/cuda.rs:625-628); this is
 * the same report for the device-resident calls, which do not synchronize themselves. */
int b2_check_status(b2_ctx* ctx);

/* ---- decode plan: one token's whole forward pass in one submission ---------------------------
 * Mirrors gpu::decode (src/gpu_decode.rs): the model describes a token as a list of ops over
 * activation buffers (Graph, src/gpu_decode.rs:378-416), Backend::decode_plan turns it into a plan
 * (src/gpu.rs:262-289; CUDA: CudaPlan, src/cuda_decode.rs:1233-1658) and DecodePlan::step runs it
 * (src/gpu_decode.rs:538-587). Here the op list is captured once into a CUDA graph whose kernels read
 * the position from device memory, so a step is one graph launch. Ops taken: the set a dense Llama /
 * Qwen3 layer uses (Norm, Linear in the five modes, QkRope, Attend, Glu); a graph with any other op
 * is declined (> 0), as decode_plan returns None and the model decodes on the CPU.
 *
 * Differences by design: the KV caches live on the device inside the plan ([n_kv][max_len][hd], f32, or
 * f16 when asked) and are the authoritative copy during device decoding; b2_plan_kv_write / _read move
 * rows between them and the host's LayerCache layout ([len][n_kv][hd] f32, src/model.rs LayerCache)
 * where the reference's Slot appends and pushes back on every step (src/cuda_decode.rs:1466-1658). */
typedef uint64_t b2_plan;
typedef struct b2_view {
    uint32_t buf; /* activation buffer */
    uint32_t off; /* offset in floats */
} b2_view;

#define B2_OP_NORM 1    /* Op::Norm */
#define B2_OP_LINEAR 2  /* Op::Linear */
#define B2_OP_QK_ROPE 3 /* Op::QkRope */
#define B2_OP_ATTEND 4  /* Op::Attend (window optional; no gate, no draft block) */
#define B2_OP_GLU 5     /* Op::Glu */
/* No counterpart in the reference (one device only): tensor-parallel plans. The vector at `x` (n values) is sharded over
 * the ranks in equal contiguous parts; every rank wrote its own part, and after the op every rank holds all of it
 * (an all-gather). Done with stores into the peers' activation buffers over NVLink and a flag barrier between the
 * GPUs (b2_plan_attach_peers), not with a library collective. */
#define B2_OP_EXCHANGE 6

typedef struct b2_op {
    uint32_t kind;
    /* NORM: x -> y.  LINEAR: y = mode(W x), z = the gate scalar of B2_MODE_ADD_GATED.
     * QK_ROPE: x = qkv, y = q_out.  ATTEND: x = q, y = out.  GLU: y = act(x) * z. */
    b2_view x, y, z;
    b2_weight w, w2;     /* LINEAR: the matrix, and the second matrix of a pair mode */
    uint32_t mode;       /* LINEAR: B2_MODE_* */
    uint32_t n_out, n_in;
    const float* p0;     /* host f32: NORM weights [n] or NULL; QK_ROPE q_norm [hd] or NULL */
    const float* p1;     /* host f32: QK_ROPE k_norm [hd] or NULL */
    uint32_t n, rows, x_stride, out_stride, add; /* NORM; GLU uses n */
    float pre, eps;      /* NORM (pre, eps); QK_ROPE (eps) */
    uint32_t kv;         /* QK_ROPE, ATTEND: index of the KV cache */
    uint32_t nh, nkv, hd;
    uint32_t half_rot, q_stride, k_off, v_off, interleaved, rope, v_norm, v_from_k; /* QK_ROPE */
    float scale;         /* ATTEND */
    uint32_t window;     /* ATTEND: 0 = all positions */
    uint32_t gelu;       /* GLU */
} b2_op;

typedef struct b2_graph {
    const uint64_t* bufs; /* floats in each activation buffer */
    uint32_t n_bufs;
    const b2_op* ops;
    uint32_t n_ops;
    b2_view input;        /* where a step's x goes */
    uint32_t n_input;
    b2_view hidden;       /* read back after a step */
    uint32_t n_hidden;
    b2_view logits;       /* read back when n_logits > 0 and the step asks for them */
    uint32_t n_logits;
    const uint32_t* kv_nkv; /* per KV cache: KV heads and head dimension (Graph::kv) */
    const uint32_t* kv_hd;
    uint32_t n_kv;
    const uint32_t* rope_halves; /* Graph::rope_halves: a step's rope_cs holds, per entry, cos[half] then sin[half] */
    uint32_t n_rope;
    uint32_t max_len;     /* positions each KV cache holds */
    uint32_t kv_f16;      /* 0: f32 caches (the reference's); 1: f16 caches */
} b2_graph;

/* B2_OK and a plan, B2_DECLINED (> 0) for an op or shape outside the supported set, < 0 on error. */
int b2_decode_plan(b2_ctx* ctx, const b2_graph* graph, b2_plan* out);
int b2_plan_free(b2_ctx* ctx, b2_plan plan);
/* DecodePlan::step for one token at `pos` (positions 0 .. pos-1 of every cache filled): x [n_input] and
 * rope_cs from the host, hidden [n_hidden] and (if not NULL) logits [n_logits] back to the host.
 * Synchronous. Nonzero: nothing valid was written. */
int b2_plan_step(b2_ctx* ctx, b2_plan plan, size_t pos, const float* x, const float* rope_cs, float* hidden, float* logits);
/* Backend::decode_plan_multi (src/gpu.rs:273-276): a plan whose steps take up to `tokens` tokens (speculative verification).
 * `tokens` 1 .. B2_PLAN_MAX_TOKENS; more is declined. A tensor-parallel graph (B2_OP_EXCHANGE) is declined for tokens > 1.
 * The plan is exact in the sense of the reference's multi-token kernels (src/cuda_decode.cu:176-179): every token's hidden
 * state, logits and cache rows equal those of one-token steps bit for bit; the products read their weights once for all
 * tokens of the step. It also serves Backend::decode_plan_multi_fast (src/gpu.rs:281-283), whose default is the exact plan.
 * All other plan calls (b2_plan_step, the KV calls, b2_plan_generate, b2_plan_free) take such a plan too. */
#define B2_PLAN_MAX_TOKENS 4
int b2_decode_plan_multi(b2_ctx* ctx, const b2_graph* graph, size_t tokens, b2_plan* out);
/* DecodePlan::tokens (src/gpu_decode.rs:575-577): the most tokens of a step of this plan. */
int b2_plan_tokens(b2_ctx* ctx, b2_plan plan, size_t* tokens);
/* DecodePlan::step with Step::t = t tokens at positions pos .. pos + t - 1, each attending to the ones before it
 * (src/gpu_decode.rs:538-570): x [t][n_input], hidden [t][n_hidden], logits [t][n_logits] or NULL, all on the host.
 * rope_cs as Step::rope_cs: for each table of rope_halves, one after the other, t rows of cos[half] then sin[half].
 * The step's keys and values are appended to the plan's caches at pos .. pos + t - 1; a caller that accepts only the first
 * m tokens simply continues at pos + m (the rows behind are overwritten). Synchronous. Nonzero: nothing valid was written. */
int b2_plan_step_multi(b2_ctx* ctx, b2_plan plan, size_t pos, size_t t, const float* x, const float* rope_cs, float* hidden,
                       float* logits);
/* Backend::decode_plan_prefill (src/gpu.rs:283-289): a plan whose steps take up to `tokens` tokens (1 .. B2_PREFILL_MAX_TOKENS)
 * on batched kernels, the activations on the device for the whole step: every product is a tensor-core GEMM over all token
 * rows (b2_matmul's kernel), attention a causal tensor-core kernel over the step's queries and the plan's KV cache. Its
 * results differ from one-token steps in rounding (as the reference says of its own prefill plans). The graph is the decode
 * graph without the head (n_logits == 0: the reference builds its prefill graph that way, src/model_gpu.rs:398-400); products
 * need a format with a tensor-core kernel (Q4_K, MLX-4, Q6_K, Q8_0, FP8), otherwise B2_DECLINED. Steps go through b2_plan_step_multi
 * (logits NULL); the KV calls, b2_plan_tokens and b2_plan_free apply. */
#define B2_PREFILL_MAX_TOKENS 8192
int b2_decode_plan_prefill(b2_ctx* ctx, const b2_graph* graph, size_t tokens, b2_plan* out);
/* Device time in milliseconds of the kernels of the plan's last prefill step (between the host copies); 0 before one. */
int b2_plan_last_step_ms(b2_ctx* ctx, b2_plan plan, float* ms);
/* Rows pos0 .. pos0+n-1 of KV cache `kv` from / to host arrays laid out [n][n_kv][hd] f32. */
int b2_plan_kv_write(b2_ctx* ctx, b2_plan plan, uint32_t kv, size_t pos0, size_t n, const float* k, const float* v);
int b2_plan_kv_read(b2_ctx* ctx, b2_plan plan, uint32_t kv, size_t pos0, size_t n, float* k, float* v);
/* Greedy decoding without the host in the loop: n_tokens steps starting at position pos0 with token
 * `first_token`; each step looks the token's row up in `embed` (any uploaded format, n_in = n_input),
 * runs the graph, takes the first largest logit as the next token (the reference's host loop does the
 * lookup and the argmax on the CPU between steps, src/generate.rs). rope_cs_table: host
 * [n_tokens][sum of 2 * rope_halves], row i for position pos0 + i. out_tokens: host [n_tokens].
 * elapsed_ms (optional): device time of the n_tokens steps. Needs n_logits > 0. */
int b2_plan_generate(b2_ctx* ctx, b2_plan plan, b2_weight embed, int32_t first_token, size_t pos0, size_t n_tokens,
                     const float* rope_cs_table, int32_t* out_tokens, float* elapsed_ms);
/* Kernel launches of one step of the plan (for launch accounting). */
int b2_plan_launches(b2_ctx* ctx, b2_plan plan, uint64_t* per_step);

/* Tensor-parallel plans (one process per GPU; no counterpart in the reference). A graph with B2_OP_EXCHANGE ops
 * needs its peers before the first step: every rank exports a handle to its plan's activation memory
 * (b2_plan_export: B2_PLAN_HANDLE_BYTES bytes, to be passed to the other processes by any means, e.g. an all-gather on
 * the host), then attaches all ranks' handles in rank order (its own entry is ignored). The ranks must build the same
 * graph (same buffers, same exchanges) over their own weight shards. Steps are collective: every rank calls
 * b2_plan_step / b2_plan_generate with the same arguments; a rank that does not arrive makes the others' exchange
 * give up after a bounded wait (B2_ERR_TIMEOUT), it does not hang them. */
#define B2_PLAN_HANDLE_BYTES 128
int b2_plan_export(b2_ctx* ctx, b2_plan plan, void* handle_out);
int b2_plan_attach_peers(b2_ctx* ctx, b2_plan plan, uint32_t rank, uint32_t world, const void* handles);

/* ---- several GPUs: one process per GPU, collectives over NCCL (no counterpart in the reference, which drives one device) ----
 * The library opens libnccl.so.2 itself with dlopen on the first of these calls (nothing is linked at build time; without
 * NCCL they return B2_DECLINED). Rank 0 makes an id with b2_comm_unique_id and hands its B2_COMM_ID_BYTES bytes to the other
 * processes by any host channel; then every process calls b2_comm_init on its own context (ncclCommInitRank on that
 * context's device). The calls below are collective: every rank makes them in the same order, on its context's stream. */
#define B2_COMM_ID_BYTES 128
int b2_comm_unique_id(void* id_out);
int b2_comm_init(b2_ctx* ctx, int world, int rank, const void* id);
int b2_comm_free(b2_ctx* ctx);
/* Tensor-parallel dense matmul: the rows of W are sharded over the ranks in equal contiguous parts and `w_shard` is this
 * rank's part [n_local][n_in] (an upload of its rows, or b2_shard_rows of a full upload); x_dev [t][n_in] is the same on
 * every rank; y_dev [t][world * n_local] f32 receives the FULL product on every rank (the shard's product, one
 * ncclAllGather, a copy of the ranks' blocks into their columns). Bit-identical to the unsharded b2_matmul_dev: every
 * column is computed by the kernel that computes it on one GPU. Not synchronized. */
int b2_matmul_sharded(b2_ctx* ctx, b2_weight w_shard, const void* x_dev, int x_dtype, size_t t, float* y_dev);
/* The same product with the all-gather done by the GEMM kernel itself (no library collective in the step): every rank keeps a
 * result buffer that the other ranks map (CUDA IPC, exchanged once through the communicator when the buffer is first made or
 * grows: that part is collective and synchronizes); the tensor-core GEMM's epilogue stores each finished tile into this
 * rank's columns of its own buffer and of every peer's buffer with bulk tensor stores over NVLink, and a one-CTA kernel then
 * makes the ranks meet (flags in the peers' buffers, bounded polling: a missing rank gives B2_ERR_TIMEOUT from
 * b2_check_status, not a hang). *y_full_dev is this rank's buffer [t][world * n_local] f32: complete once the stream reaches
 * the end of the call, valid until the call after the next one (two areas alternate). Bit-identical to b2_matmul_sharded.
 * Declined (> 0): up to 8 tokens, formats without a tensor-core kernel, FP8 x FP8 mode, n_local % 4 != 0, more than 8 ranks:
 * use b2_matmul_sharded then. 2 to 8 ranks of one NVLink domain, one process per GPU. */
int b2_matmul_sharded_peer(b2_ctx* ctx, b2_weight w_shard, const void* x_dev, int x_dtype, size_t t, float** y_full_dev);
/* Expert-parallel `Backend::moe`: the layer's n_experts_global experts are sharded over the ranks in equal contiguous parts
 * and `m` holds this rank's (b2_upload_moe over them, local numbering); x_dev / y_dev [t][h] are THIS rank's tokens,
 * route_ids [t][k] (host) are global expert numbers, route_w [t][k] (host) their weights. Every (token, route) pair goes to
 * the rank that owns its expert and its result comes back (counts by ncclAllGather, rows by grouped ncclSend / ncclRecv),
 * then y[i] += sum_j w_ij o_ij in route order: bit-identical to b2_moe_dev over all experts on one GPU. Synchronizes the
 * stream (the route tables are host arrays). */
int b2_moe_ep(b2_ctx* ctx, b2_moe_handle m, size_t n_experts_global, const float* x_dev, size_t t, const int32_t* route_ids,
              const float* route_w, size_t k, float* y_dev);

/* No counterpart in the reference (its CUDA backend allocates staging and arena memory freely,
 * src/cuda.rs:572-699). One Q4_K matrix-vector product, y[n_out] = W x, that allocates nothing, for
 * hosts that cannot call cudaMalloc when they need it: a server whose own arena already owns the
 * whole device, or a decode loop that must stay out of the allocator. The activation planes the
 * kernel needs live in a fixed device array inside the library (57,344 bytes per GPU for as long as
 * the library is loaded), which limits n_in to B2_NOALLOC_MAX_K; larger inputs are refused with
 * B2_ERR_ARG and a message, and go through b2_matvec_dev instead.
 *   w_blocks_dev : raw GGUF Q4_K super-blocks on the device, [n_out][n_in/256][144], 16-byte aligned
 *   x_dev, y_dev : f32 on the device; cuda_stream : the stream to launch on (NULL = default)
 *   err, err_len : optional buffer that receives the error text
 * The first call on a device looks up the array's device address; make it before any stream
 * capture. All calls share the one array: calls that may overlap on the GPU race on it. */
#define B2_NOALLOC_MAX_K 16384
int b2_matvec_q4k_noalloc(const void* w_blocks_dev, size_t n_out, size_t n_in, const float* x_dev, float* y_dev, void* cuda_stream,
                          char* err, size_t err_len);

#ifdef __cplusplus
}
#endif
#endif /* B200QMM_H */
