// The per-block step of the activation split (see XPlanes in kernels.h): a warp holds one block of 32
// values, one per lane, and writes its three int8 planes, scale, sums. Shared by the stand-alone plane
// kernel and by the kernels that produce a GEMV's input (norm, attention) and write the planes themselves.
#pragma once
#include "kernels.h"

namespace b2 {

// Programmatic dependent launch: a kernel launched with the attribute may start before the kernel ahead of it in
// the stream has finished; it must not touch anything that kernel writes until pdl_wait() returns. Both are
// no-ops in a kernel launched the ordinary way.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// The block's integers q = round(x / s) have 21 significant bits, |q| <= XQ_MAX, and are stored as three signed digits
// q = q0 + 32 (q1 + 256 q2): q0 in [-16, 15], q1 in [-128, 127], |q2| <= 127. The product kernels read all three (exact to
// 21 bits, the default) or, on request, only q1 and q2 (the nearest multiple of 32: 16 bits, an error of at most 1.6e-5
// of the block's largest element per element) and save a third of their integer dot products.
constexpr float XQ_MAX = 1040000.0f;

// One block of 32 values split by a warp (one value per lane, all 32 lanes call it): the lane's three plane bytes,
// the block scale, the integer sums of the lane's half block and of the block.
struct XSplit {
    int q0, q1, q2, sum16, sum32;
    float s;
};
__device__ __forceinline__ XSplit xplanes_split(float v) {
    // the block's largest magnitude: non-negative floats order like their bit patterns, so one integer warp reduction
    float a = __uint_as_float(__reduce_max_sync(0xffffffffu, __float_as_uint(fabsf(v))));
    XSplit r;
    r.s = a / XQ_MAX;
    int q = a > 0.0f ? __float2int_rn(v * (XQ_MAX / a)) : 0;
    q = max(-(int)XQ_MAX, min((int)XQ_MAX, q));
    r.q0 = ((q + 16) & 31) - 16;
    int r1 = (q - r.q0) >> 5;
    r.q1 = ((r1 + 128) & 255) - 128;
    r.q2 = (r1 - r.q1) >> 8;
    const unsigned half = (threadIdx.x & 16) ? 0xffff0000u : 0x0000ffffu;  // the lane's half warp
    r.sum16 = __reduce_add_sync(half, q);
    r.sum32 = __reduce_add_sync(0xffffffffu, q);
    return r;
}

// The split of block `blk` written to the global-memory layout (XPlanes).
__device__ __forceinline__ void xplanes_block(float v, int blk, int lane, int K, const XPlanes& out) {
    const XSplit r = xplanes_split(v);
    const size_t at = (size_t)xplanes_slot(blk * 2 + (lane >> 4)) * 16 + (lane & 15);
    out.planes[at] = (int8_t)r.q0;
    out.planes[(size_t)K + at] = (int8_t)r.q1;
    out.planes[2 * (size_t)K + at] = (int8_t)r.q2;
    if ((lane & 15) == 0) out.v16[blk * 2 + (lane >> 4)] = r.sum16;
    if (lane == 0) out.sx[blk] = make_float2(r.s, r.s * (float)r.sum32);
}

// The record (planes, scales, sums) -> shared memory, a plain copy by the calling threads; the caller synchronizes.
__device__ __forceinline__ void xplanes_stage(const XPlanes& xp, int K, uint8_t* sm, int tid, int nthreads) {
    const uint4* src = (const uint4*)xp.planes;
    uint4* dst = (uint4*)sm;
    const int n = (int)(xplanes_bytes((size_t)K) / 16);
    for (int i = tid; i < n; i += nthreads) dst[i] = __ldcg(src + i);
}

}  // namespace b2
