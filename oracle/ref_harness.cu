// Test infrastructure only: a host harness around the REFERENCE's own CUDA kernels, used as a second, GPU-side
// oracle and baseline for the MLX-4 matrix-vector product (config 0). The kernels are not in this repository:
// build_ref.py assembles them at build time from the reference's tree (the KERNEL_SRC string of src/cuda.rs followed
// by src/cuda_decode.cu, which is how src/cuda.rs:477 builds its NVRTC module) into _ref/ref_kernels.cuh, and this file
// includes that. Launch geometry as the reference's host code: 4 warps per block, DMV_NR = 4 rows per warp
// (src/cuda_decode.rs:32-34), arguments as `DW` (src/cuda_decode.cu:27).
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
