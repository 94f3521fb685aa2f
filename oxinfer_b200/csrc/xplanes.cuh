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

constexpr float XQ_MAX = 1040000.0f;  // |q0 + 128 q1 + 16384 q2| <= 63 + 128*63 + 16384*63 = 1040319

// All 32 lanes of the warp must call this with the block's values in lane order.
__device__ __forceinline__ void xplanes_block(float v, int blk, int lane, int K, const XPlanes& out) {
    float a = fabsf(v);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, o));
    float s = a / XQ_MAX;
    int q = a > 0.0f ? __float2int_rn(v * (XQ_MAX / a)) : 0;
    q = max(-(int)XQ_MAX, min((int)XQ_MAX, q));
    int q0 = ((q + 64) & 127) - 64;
    int r1 = (q - q0) >> 7;
    int q1 = ((r1 + 64) & 127) - 64;
    int q2 = (r1 - q1) >> 7;
    size_t at = (size_t)blk * 32 + lane;
    out.planes[at] = (int8_t)q0;
    out.planes[(size_t)K + at] = (int8_t)q1;
    out.planes[2 * (size_t)K + at] = (int8_t)q2;
    int sum16 = q;
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) sum16 += __shfl_xor_sync(0xffffffffu, sum16, o);
    int sum32 = sum16 + __shfl_xor_sync(0xffffffffu, sum16, 16);
    if ((lane & 15) == 0) out.v16[blk * 2 + (lane >> 4)] = sum16;
    if (lane == 0) {
        out.xs[blk] = s;
        out.xsum[blk] = s * (float)sum32;
    }
}

}  // namespace b2
