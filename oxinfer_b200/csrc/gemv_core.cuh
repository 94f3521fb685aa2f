// Device code shared by the matrix-vector kernels (gemv.cu: register-load, ring and generic forms): the shared-memory
// view of the activation planes, and per weight format the loads of one step of a row pair and its integer dot
// products (see the design notes at the top of gemv.cu).
#pragma once
#include <cuda_fp8.h>

#include "kernels.h"
#include "xplanes.cuh"

namespace b2 {
namespace gemv_core {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// The vector as the kernels see it in shared memory. Plane p is K bytes at p0 + p K with its 16-byte
// slots permuted by swz(); `sx` holds {block scale, block sum} pairs per block of 32.
struct XS {
    const uint8_t* p0;
    const float2* sx;
    const int32_t* v16;
    const float* xf;  // FP8: the f32 vector (slots permuted the same way)
    int K;
};

__device__ __forceinline__ int swz(int g) { return xplanes_slot(g); }  // the slot permutation of the planes (kernels.h)

__device__ __forceinline__ uint4 plane16(const XS& x, int p, int k) {  // 16 plane bytes at element k (k % 16 == 0)
    return *(const uint4*)(x.p0 + (size_t)p * x.K + ((size_t)swz(k >> 4) << 4));
}
__device__ __forceinline__ void plane64(const XS& x, int p, int k0, uint32_t (&w)[16]) {  // 64 plane bytes at k0 (k0 % 64 == 0)
    const uint8_t* base = x.p0 + (size_t)p * x.K;
    const int g0 = k0 >> 4, c = (((g0 >> 3) & 1) << 1) | ((g0 >> 4) & 1);
#pragma unroll
    for (int i = 0; i < 4; i++) {
        uint4 v = *(const uint4*)(base + ((size_t)(g0 + (i ^ c)) << 4));
        w[4 * i] = v.x;
        w[4 * i + 1] = v.y;
        w[4 * i + 2] = v.z;
        w[4 * i + 3] = v.w;
    }
}

__device__ __forceinline__ int dp(uint32_t a, uint32_t b, int c) { return __dp4a((int)a, (int)b, c); }
// unsigned weight bytes (0 .. 255) times signed plane bytes
__device__ __forceinline__ int dp_us(uint32_t a, uint32_t b, int c) {
    int d;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
// The integer sum over a run of k of w * q from the per-plane sums (q = q0 + 32 q1 + 8192 q2). NP = 2 leaves q0 out. The
// partial terms may wrap; the total fits 32 bits and unsigned arithmetic keeps it.
template <int NP>
__device__ __forceinline__ int planes_sum(int a0, int a1, int a2) {
    const uint32_t hi = ((uint32_t)a1 << 5) + ((uint32_t)a2 << 13);
    return (int)(NP == 3 ? hi + (uint32_t)a0 : hi);
}
__device__ __forceinline__ uint4 ldg_stream(const void* p) {  // streamed once: keep it out of L1
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

// A small non-negative integer (< 2^23) as a float without the conversion unit: the integer becomes the mantissa of
// 2^23 + n, and subtracting 2^23 is exact. (Integer-to-float conversions run on a quarter-rate pipe that the
// sub-block tails were saturating.)
__device__ __forceinline__ float small_uint_to_float(uint32_t n) { return __uint_as_float(0x4B000000u | n) - 8388608.0f; }
// The same for a signed byte value in -128 .. 127 held in the low 8 bits of `b`.
__device__ __forceinline__ float int8_to_float(uint32_t b) { return __uint_as_float(0x4B000000u | ((b ^ 0x80u) & 0xffu)) - 8388736.0f; }

// The deferred norm factor (NormScale), computed by every warp for itself in the same order: lane-strided partial sums,
// then a butterfly, so that all warps of all CTAs get the same bits.
__device__ __forceinline__ float norm_scale_factor(const NormScale& ns, int lane) {
    if (!ns.partial) return 1.0f;
    float s = 0.0f;
    for (uint32_t i = (uint32_t)lane; i < ns.count; i += 32) s += __ldcg(ns.partial + i);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    return 1.0f / sqrtf(s * ns.inv_n + ns.eps);
}

__device__ __forceinline__ float silu(float a) { return a / (1.0f + __expf(-a)); }
__device__ __forceinline__ float gelu_tanh(float a) {
    float t = 0.7978845608f * (a + 0.044715f * a * a * a);
    return 0.5f * a * (1.0f + tanhf(t));
}

// ---- per-format pieces: `load` issues the global loads of one warp-iteration of one row, `dot2`
// consumes two rows' loads against the vector (planes read once). An iteration covers ITER_K k.

// Q4_K and the repacked MLX-4 share the block shape: 16 header bytes + 128 bytes of nibbles per 256
// weights, byte l of 64-group j holding element 64 j + l (low nibble) and 64 j + 32 + l (high nibble).
// A warp iteration covers 8 blocks, 4 lanes each (one 64-group per lane).
struct Q4Regs {
    uint4 hdr, q0, q1;
};
__device__ __forceinline__ void q4_load(const WeightDev& w, size_t row, int it, int lane, Q4Regs& r) {
    const uint8_t* blk = w.p0 + (row * (w.n_in / 256) + it * 8 + (lane >> 2)) * 144;
    r.hdr = __ldg((const uint4*)blk);  // shared by the four lanes of the block: let it hit L1
    r.q0 = ldg_stream(blk + 16 + 32 * (lane & 3));
    r.q1 = ldg_stream(blk + 32 + 32 * (lane & 3));
}
// Integer dot products of the low / high nibbles of two rows' 64-groups with the planes.
template <int NP>
__device__ __forceinline__ void q4_int_dots(const Q4Regs& a, const Q4Regs& b, const XS& x, int k0, int& la, int& ha, int& lb, int& hb) {
    const uint32_t qa[8] = {a.q0.x, a.q0.y, a.q0.z, a.q0.w, a.q1.x, a.q1.y, a.q1.z, a.q1.w};
    const uint32_t qb[8] = {b.q0.x, b.q0.y, b.q0.z, b.q0.w, b.q1.x, b.q1.y, b.q1.z, b.q1.w};
    // Half a 32-byte run at a time: the sixteen masked nibble words are made once and used against all three planes while
    // they are live (the other order, plane by plane, makes the compiler mask the same words three times).
    int s[3][4] = {{0, 0, 0, 0}, {0, 0, 0, 0}, {0, 0, 0, 0}};
#pragma unroll
    for (int h = 0; h < 2; h++) {
        uint32_t al[4], ah[4], bl[4], bh[4];
#pragma unroll
        for (int i = 0; i < 4; i++) {
            al[i] = qa[4 * h + i] & 0x0F0F0F0Fu;
            ah[i] = NP == 3 ? (qa[4 * h + i] >> 4) & 0x0F0F0F0Fu : qa[4 * h + i] & 0xF0F0F0F0u;  // NP 2: 16 x the nibble, no shift
            bl[i] = qb[4 * h + i] & 0x0F0F0F0Fu;
            bh[i] = NP == 3 ? (qb[4 * h + i] >> 4) & 0x0F0F0F0Fu : qb[4 * h + i] & 0xF0F0F0F0u;
        }
#pragma unroll
        for (int p = 3 - NP; p < 3; p++) {
            const uint4 lo = plane16(x, p, k0 + 16 * h), hi = plane16(x, p, k0 + 32 + 16 * h);
            const uint32_t xl[4] = {lo.x, lo.y, lo.z, lo.w}, xh[4] = {hi.x, hi.y, hi.z, hi.w};
#pragma unroll
            for (int i = 0; i < 4; i++) {
                s[p][0] = dp(al[i], xl[i], s[p][0]);
                s[p][1] = NP == 3 ? dp(ah[i], xh[i], s[p][1]) : dp_us(ah[i], xh[i], s[p][1]);
                s[p][2] = dp(bl[i], xl[i], s[p][2]);
                s[p][3] = NP == 3 ? dp(bh[i], xh[i], s[p][3]) : dp_us(bh[i], xh[i], s[p][3]);
            }
        }
    }
    la = planes_sum<NP>(s[0][0], s[1][0], s[2][0]);
    lb = planes_sum<NP>(s[0][2], s[1][2], s[2][2]);
    if (NP == 3) {
        ha = planes_sum<3>(s[0][1], s[1][1], s[2][1]);
        hb = planes_sum<3>(s[0][3], s[1][3], s[2][3]);
    } else {  // the high sums carry a factor of 16 (exactly): 32 q1 + 8192 q2 over 16 = 2 q1 + 512 q2
        ha = (int)(((uint32_t)s[1][1] << 1) + ((uint32_t)s[2][1] << 9));
        hb = (int)(((uint32_t)s[1][3] << 1) + ((uint32_t)s[2][3] << 9));
    }
}

template <int NP>
struct FmtQ4K_T {
    static constexpr int ITER_K = 2048;
    using Regs = Q4Regs;
    __device__ static __forceinline__ bool active(int K, int it, int lane) { return it * 8 + (lane >> 2) < K / 256; }
    __device__ static __forceinline__ void load(const WeightDev& w, size_t row, int it, int lane, Regs& r) { q4_load(w, row, it, lane, r); }
    // scales / mins of sub-blocks 2j, 2j+1 without a branch on j (lanes of a warp differ in j):
    // bytes a = B[i & 3], b = B[4 + (i & 3)], c = B[8 + (i & 3)] of the 12 (get_scale_min_k4, src/ggml.rs:501-509)
    __device__ static __forceinline__ void tail(const Regs& r, int j, float4 sx, int lo, int hi, float& acc) {
        const float d = __half2float(__ushort_as_half((unsigned short)(r.hdr.x & 0xffff)));
        const float dmin = __half2float(__ushort_as_half((unsigned short)(r.hdr.x >> 16)));
        const int sh = 16 * (j & 1);                 // the pair (2j, 2j+1) = bytes 2(j&1), 2(j&1)+1 of each word
        const uint32_t a = (r.hdr.y >> sh) & 0xffffu, b = (r.hdr.z >> sh) & 0xffffu, c = (r.hdr.w >> sh) & 0xffffu;
        const uint32_t sc = (j < 2) ? (a & 0x3f3fu) : ((c & 0x0f0fu) | ((a >> 2) & 0x3030u));
        const uint32_t mn = (j < 2) ? (b & 0x3f3fu) : (((c >> 4) & 0x0f0fu) | ((b >> 2) & 0x3030u));
        acc = fmaf((d * small_uint_to_float(sc & 0xff)) * sx.x, (float)lo, acc);
        acc = fmaf((d * small_uint_to_float(sc >> 8)) * sx.z, (float)hi, acc);
        acc = fmaf(-(dmin * small_uint_to_float(mn & 0xff)), sx.y, acc);
        acc = fmaf(-(dmin * small_uint_to_float(mn >> 8)), sx.w, acc);
    }
    __device__ static __forceinline__ void dot2(const Regs& a, const Regs& b, const XS& x, int it, int lane, float& accA, float& accB) {
        const int j = lane & 3;
        const int k0 = (it * 8 + (lane >> 2)) * 256 + 64 * j;
        int la, ha, lb, hb;
        q4_int_dots<NP>(a, b, x, k0, la, ha, lb, hb);
        const float4 sx = *(const float4*)(x.sx + (k0 >> 5));  // {xs, xsum} of the two blocks of 32
        tail(a, j, sx, la, ha, accA);
        tail(b, j, sx, lb, hb, accB);
    }
};

// MLX affine 4-bit, repacked at upload into Q4_K-shaped blocks: header = 4 f16 d + 4 bf16 offsets
// (one per 64-group: the fields of the reference's Q4Matrix), then the 128 nibble bytes in the order above.
template <int NP>
struct FmtMLX4_T {
    static constexpr int ITER_K = 2048;
    using Regs = Q4Regs;
    __device__ static __forceinline__ bool active(int K, int it, int lane) { return it * 8 + (lane >> 2) < K / 256; }
    __device__ static __forceinline__ void load(const WeightDev& w, size_t row, int it, int lane, Regs& r) { q4_load(w, row, it, lane, r); }
    // The CPU path's values (src/quant.rs:518-563,586-606): d = f16(scale), offset = bf16(bias + 8 scale),
    // w = (nib - 8) d + offset = nib d + (offset - 8 d).
    __device__ static __forceinline__ void tail(const Regs& r, int j, float4 sx, int lo, int hi, float& acc) {
        const uint32_t sw = (j & 2) ? r.hdr.y : r.hdr.x, bw = (j & 2) ? r.hdr.w : r.hdr.z;
        const float d = __half2float(__ushort_as_half((unsigned short)((sw >> (16 * (j & 1))) & 0xffffu)));
        const float off = bf16_bits_to_f32((bw >> (16 * (j & 1))) & 0xffffu);
        const float dots = fmaf(sx.z, (float)hi, sx.x * (float)lo);
        acc = fmaf(d, dots, acc);
        acc = fmaf(off - 8.0f * d, sx.y + sx.w, acc);
    }
    __device__ static __forceinline__ void dot2(const Regs& a, const Regs& b, const XS& x, int it, int lane, float& accA, float& accB) {
        const int j = lane & 3;
        const int k0 = (it * 8 + (lane >> 2)) * 256 + 64 * j;
        int la, ha, lb, hb;
        q4_int_dots<NP>(a, b, x, k0, la, ha, lb, hb);
        const float4 sx = *(const float4*)(x.sx + (k0 >> 5));
        tail(a, j, sx, la, ha, accA);
        tail(b, j, sx, lb, hb, accB);
    }
};

template <int NP>
struct FmtQ6K_T {
    static constexpr int ITER_K = 2048;  // 8 blocks of 256, 4 lanes each (64 elements per lane)
    struct Regs {
        uint4 qh, qa, qb;
        uint2 sc;
        uint32_t d;
    };
    __device__ static __forceinline__ bool active(int K, int it, int lane) { return it * 8 + (lane >> 2) < K / 256; }
    __device__ static __forceinline__ void load(const WeightDev& w, size_t row, int it, int lane, Regs& r) {
        size_t K = w.n_in;
        size_t blk = it * 8 + (lane >> 2);
        int n = (lane >> 1) & 1, u = lane & 1;
        r.qh = ldg_stream(w.p1 + row * (K / 4) + blk * 64 + 32 * n + 16 * u);
        r.qa = ldg_stream(w.p0 + row * (K / 2) + blk * 128 + 64 * n + 16 * u);
        r.qb = ldg_stream(w.p0 + row * (K / 2) + blk * 128 + 64 * n + 32 + 16 * u);
        r.sc = __ldg((const uint2*)(w.p2 + row * (K / 16) + blk * 16 + 8 * n));
        r.d = __ldg((const uint16_t*)w.p3 + row * (K / 256) + blk);
    }
    __device__ static __forceinline__ void dot2(const Regs& a, const Regs& b, const XS& x, int it, int lane, float& accA, float& accB) {
        const int n = (lane >> 1) & 1, u = lane & 1;
        const int kb = (it * 8 + (lane >> 2)) * 256 + 128 * n + 16 * u;  // quarter k4 adds 32 k4
        const float da = __half2float(__ushort_as_half((unsigned short)a.d)), db = __half2float(__ushort_as_half((unsigned short)b.d));
        const uint32_t HA[4] = {a.qh.x, a.qh.y, a.qh.z, a.qh.w}, AA[4] = {a.qa.x, a.qa.y, a.qa.z, a.qa.w}, BA[4] = {a.qb.x, a.qb.y, a.qb.z, a.qb.w};
        const uint32_t HB[4] = {b.qh.x, b.qh.y, b.qh.z, b.qh.w}, AB[4] = {b.qa.x, b.qa.y, b.qa.z, b.qa.w}, BB[4] = {b.qb.x, b.qb.y, b.qb.z, b.qb.w};
        const uint64_t sca = (uint64_t)a.sc.x | ((uint64_t)a.sc.y << 32), scb = (uint64_t)b.sc.x | ((uint64_t)b.sc.y << 32);
#pragma unroll
        for (int k4 = 0; k4 < 4; k4++) {
            uint32_t qa[4], qb[4];
#pragma unroll
            for (int i = 0; i < 4; i++) {
                uint32_t lo = (k4 & 1) ? BA[i] : AA[i];
                lo = (k4 & 2) ? (lo >> 4) : lo;
                uint32_t hb = (k4 == 0) ? (HA[i] << 4) : (k4 == 1) ? (HA[i] << 2) : (k4 == 2) ? HA[i] : (HA[i] >> 2);
                qa[i] = (lo & 0x0F0F0F0Fu) | (hb & 0x30303030u);
                lo = (k4 & 1) ? BB[i] : AB[i];
                lo = (k4 & 2) ? (lo >> 4) : lo;
                hb = (k4 == 0) ? (HB[i] << 4) : (k4 == 1) ? (HB[i] << 2) : (k4 == 2) ? HB[i] : (HB[i] >> 2);
                qb[i] = (lo & 0x0F0F0F0Fu) | (hb & 0x30303030u);
            }
            const int k0 = kb + 32 * k4;
            int sa[3] = {0, 0, 0}, sb[3] = {0, 0, 0};
#pragma unroll
            for (int p = 3 - NP; p < 3; p++) {
                uint4 xv = plane16(x, p, k0);
                int t = dp(qa[0], xv.x, 0);
                t = dp(qa[1], xv.y, t);
                t = dp(qa[2], xv.z, t);
                sa[p] = dp(qa[3], xv.w, t);
                t = dp(qb[0], xv.x, 0);
                t = dp(qb[1], xv.y, t);
                t = dp(qb[2], xv.z, t);
                sb[p] = dp(qb[3], xv.w, t);
            }
            const int off32 = 32 * x.v16[k0 >> 4];
            const float xs = x.sx[k0 >> 5].x;
            const float scale_a = int8_to_float((uint32_t)(sca >> (8 * (u + 2 * k4))));
            const float scale_b = int8_to_float((uint32_t)(scb >> (8 * (u + 2 * k4))));
            accA = fmaf((da * scale_a) * xs, (float)(planes_sum<NP>(sa[0], sa[1], sa[2]) - off32), accA);
            accB = fmaf((db * scale_b) * xs, (float)(planes_sum<NP>(sb[0], sb[1], sb[2]) - off32), accB);
        }
    }
};

template <int NP>
struct FmtQ8_0_T {
    static constexpr int ITER_K = 512;  // 16 bytes = 16 weights per lane
    struct Regs {
        uint4 q;
        uint32_t d;
    };
    __device__ static __forceinline__ bool active(int K, int it, int lane) { return it * 512 + lane * 16 < K; }
    __device__ static __forceinline__ void load(const WeightDev& w, size_t row, int it, int lane, Regs& r) {
        size_t k0 = (size_t)it * 512 + lane * 16;
        r.q = ldg_stream(w.p0 + row * w.n_in + k0);
        r.d = __ldg((const uint16_t*)w.p1 + row * (w.n_in / 32) + k0 / 32);
    }
    __device__ static __forceinline__ void dot2(const Regs& a, const Regs& b, const XS& x, int it, int lane, float& accA, float& accB) {
        const int k0 = it * 512 + lane * 16;
        int sa[3] = {0, 0, 0}, sb[3] = {0, 0, 0};
#pragma unroll
        for (int p = 3 - NP; p < 3; p++) {
            uint4 xv = plane16(x, p, k0);
            int t = dp(a.q.x, xv.x, 0);
            t = dp(a.q.y, xv.y, t);
            t = dp(a.q.z, xv.z, t);
            sa[p] = dp(a.q.w, xv.w, t);
            t = dp(b.q.x, xv.x, 0);
            t = dp(b.q.y, xv.y, t);
            t = dp(b.q.z, xv.z, t);
            sb[p] = dp(b.q.w, xv.w, t);
        }
        const float xs = x.sx[k0 >> 5].x;
        accA = fmaf(__half2float(__ushort_as_half((unsigned short)a.d)) * xs, (float)planes_sum<NP>(sa[0], sa[1], sa[2]), accA);
        accB = fmaf(__half2float(__ushort_as_half((unsigned short)b.d)) * xs, (float)planes_sum<NP>(sb[0], sb[1], sb[2]), accB);
    }
};

template <int NP>  // reads the f32 vector, not the planes: NP is ignored and every use names 3
struct FmtF8_T {
    static constexpr int ITER_K = 512;  // 16 e4m3 bytes per lane
    struct Regs {
        uint4 q;
        float s;
    };
    __device__ static __forceinline__ bool active(int K, int it, int lane) { return it * 512 + lane * 16 < K; }
    __device__ static __forceinline__ void load(const WeightDev& w, size_t row, int it, int lane, Regs& r) {
        size_t k0 = (size_t)it * 512 + lane * 16;
        r.q = ldg_stream(w.p0 + row * w.n_in + k0);
        r.s = w.p1 ? __ldg((const float*)w.p1 + ((w.bs_row0 + row) / w.bs_rows) * w.bs_ncb + k0 / w.bs_cols) : 1.0f;
    }
    __device__ static __forceinline__ float part(uint32_t q, float4 xx, float acc) {
        __half2_raw h01 = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(q & 0xffff), __NV_E4M3);
        __half2_raw h23 = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(q >> 16), __NV_E4M3);
        float2 f01 = __half22float2(*(const __half2*)&h01), f23 = __half22float2(*(const __half2*)&h23);
        acc = fmaf(f01.x, xx.x, acc);
        acc = fmaf(f01.y, xx.y, acc);
        acc = fmaf(f23.x, xx.z, acc);
        return fmaf(f23.y, xx.w, acc);
    }
    __device__ static __forceinline__ void dot2(const Regs& a, const Regs& b, const XS& x, int it, int lane, float& accA, float& accB) {
        const int k0 = it * 512 + lane * 16;  // 16 floats = four 16-byte slots, permuted like the planes
        const int g0 = k0 >> 2, c = (((g0 >> 3) & 1) << 1) | ((g0 >> 4) & 1);
        const uint32_t qa[4] = {a.q.x, a.q.y, a.q.z, a.q.w}, qb[4] = {b.q.x, b.q.y, b.q.z, b.q.w};
        float pa = 0.0f, pb = 0.0f;
#pragma unroll
        for (int i = 0; i < 4; i++) {
            float4 xx = *(const float4*)(x.xf + ((size_t)(g0 + (i ^ c)) << 2));
            pa = part(qa[i], xx, pa);
            pb = part(qb[i], xx, pb);
        }
        accA = fmaf(pa, a.s, accA);
        accB = fmaf(pb, b.s, accB);
    }
};

}  // namespace gemv_core
}  // namespace b2
