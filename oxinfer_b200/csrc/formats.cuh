// Device-side layouts of the weight formats and the scalar decoders shared by every kernel.
//
// Device layouts (all 16-byte aligned per row for n_in a multiple of 256):
//   MLX4   : repacked at upload into Q4_K-shaped blocks of 256 weights, 144 bytes: 4 f16 d @0, 4 bf16 offsets @8
//            (one per 64-group; d = f16(scale), offset = bf16(bias + 8 scale), the fields of the reference's
//            Q4Matrix, src/quant.rs:427-440,518-563), qs[128] @16 with Q4_K's nibble order (byte l of
//            64-group j = element 64j+l low, 64j+32+l high), so that every 4-bit kernel is shared
//   Q4_K   : raw GGUF super-blocks, 144 bytes per 256 weights: d f16 @0, dmin f16 @2,
//            scales[12] @4, qs[128] @16                       (unchanged)
//   Q6_K   : split at upload into four row-major planes so that every load is aligned:
//            ql u8 [n_out][n_in/2], qh u8 [n_out][n_in/4], sc i8 [n_out][n_in/16], d f16 [n_out][n_in/256]
//            (GGUF's 210-byte blocks are only 2-byte aligned)
//   Q8_0   : split at upload: qs i8 [n_out][n_in], d f16 [n_out][n_in/32]   (GGUF: 34-byte blocks)
//   F8E4M3 : w u8 [n_out][n_in] + f32 scales [ceil(n_out/bs_rows)][ceil(n_in/bs_cols)]
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/b200qmm.h"

namespace b2 {

struct WeightDev {
    int fmt;
    size_t n_out, n_in;
    size_t group;             // MLX4 group size
    const uint8_t* p0;        // MLX4 w | Q4_K blocks | Q6_K ql | Q8_0 qs | F8 w
    const uint8_t* p1;        // MLX4 scales | Q6_K qh | Q8_0 d | F8 block scales
    const uint8_t* p2;        // MLX4 biases | Q6_K sc
    const uint8_t* p3;        // Q6_K d
    size_t bs_rows, bs_cols;  // F8 scale-block shape
    size_t bs_ncb;            // F8: scale blocks per scale row = ceil(full n_in / bs_cols)
    size_t bs_row0;           // F8: first row of this (possibly sharded) matrix in the full matrix
};

__device__ __forceinline__ float bf16_bits_to_f32(uint32_t h) { return __uint_as_float(h << 16); }
__device__ __forceinline__ float f16_bits_to_f32(uint16_t h) { return __half2float(__ushort_as_half(h)); }

// Round-to-nearest-even f32 -> bf16 bits, as `half::bf16::from_f32` (src/quant.rs:580-583).
__device__ __forceinline__ uint32_t f32_to_bf16_bits(float f) {
    uint32_t x = __float_as_uint(f);
    if ((x & 0x7fffffffu) > 0x7f800000u) return (x >> 16) | 0x40u;
    return (x + 0x7fffu + ((x >> 16) & 1u)) >> 16;
}

// e4m3fn byte -> f32, the value table of src/ggml.rs:258-271 (0x7f / 0xff are NaN, no infinities).
__device__ __forceinline__ float e4m3_to_f32(uint32_t b) {
    uint32_t e = (b >> 3) & 0xF, m = b & 7;
    uint32_t mag;
    if (e == 0)
        mag = __float_as_uint((float)m * (1.0f / 512.0f));
    else
        mag = ((e + 120u) << 23) | (m << 20);
    if ((b & 0x7F) == 0x7F) mag = 0x7FC00000u;
    return __uint_as_float(mag | ((b & 0x80u) << 24));
}

// The (scale, min) pair `i` (0..8) of a Q4_K super-block from its 12 packed bytes
// (get_scale_min_k4, src/ggml.rs:501-509). q0..q2 are the three little-endian words of scales[12].
__device__ __forceinline__ void q4k_scale_min(int i, uint32_t q0, uint32_t q1, uint32_t q2, uint32_t& sc, uint32_t& mn) {
    // byte n of the 12: word n/4, shift 8*(n%4)
    if (i < 4) {
        sc = (q0 >> (8 * i)) & 63;
        mn = (q1 >> (8 * i)) & 63;
    } else {
        int s = 8 * (i - 4);
        uint32_t t = (q2 >> s) & 0xff;   // q[i+4]
        uint32_t a = (q0 >> s) & 0xff;   // q[i-4]
        uint32_t b = (q1 >> s) & 0xff;   // q[i]
        sc = (t & 0xF) | ((a >> 6) << 4);
        mn = (t >> 4) | ((b >> 6) << 4);
    }
}

}  // namespace b2
