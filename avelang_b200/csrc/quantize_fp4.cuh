// bf16 -> NVFP4 / MXFP4 quantise kernels (bandwidth-bound).
//
// The reference has no quantise operator; its only quantise-like primitive is the
// packed fp8 conversion python/avelang/language/amdgpu.py:90-94.  The arithmetic
// here is, operation for operation, the CPU oracle's (oracle/fp4_oracle.c): every
// fp32 step is a single round-to-nearest-even operation (explicit _rn intrinsics,
// IEEE division), so packed nibbles and scale bytes are bit-identical.
//
// Mapping: a warp takes 1024 consecutive K elements of one row per step and lane L owns the 32
// consecutive elements 32L .. 32L+31: four 128-bit loads, two whole 16-element NVFP4 blocks or one
// 32-element MXFP4 block per lane (the block maximum stays inside the lane), one 128-bit store of
// the 32 packed nibbles (512 contiguous bytes per warp) and one 16-bit or 8-bit scale store.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp4.h>
#include <cuda_fp8.h>

#include <cstdint>

namespace avefp4 {

constexpr int kFmtNvfp4 = 0;
constexpr int kFmtMxfp4 = 1;
constexpr int kSfRowMajor = 0;
constexpr int kSfTiled = 1;

// max |x| over a (rows, k) bf16 matrix with row stride ldx; result = fp32 bit pattern
// in *amax_bits (must be zero on entry; non-negative floats order like unsigned ints).
__global__ void __launch_bounds__(256)
amax_bf16_kernel(const __nv_bfloat16* __restrict__ x, long long rows, long long k, long long ldx,
                 unsigned int* __restrict__ amax_bits) {
    const long long groups_per_row = k / 8;
    const long long total = rows * groups_per_row;
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    // running maximum of the bf16 magnitudes as packed unsigned 16-bit pairs (finite bf16 magnitudes order like integers)
    constexpr uint32_t kMag = 0x7fff7fffu;
    uint32_t m = 0;
    // four independent 128-bit loads in flight per thread
    for (long long g0 = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; g0 < total; g0 += 4 * stride) {
        uint4 v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const long long g = g0 + u * stride;
            v[u] = make_uint4(0, 0, 0, 0);
            if (g < total) {
                long long off = g * 8;          // rows back to back: no division
                if (ldx != k) {
                    const long long r = g / groups_per_row;
                    off = r * ldx + (g - r * groups_per_row) * 8;
                }
                v[u] = __ldcs(reinterpret_cast<const uint4*>(x + off));
            }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            m = __vimax3_u16x2(m, v[u].x & kMag, v[u].y & kMag);
            m = __vimax3_u16x2(m, v[u].z & kMag, v[u].w & kMag);
        }
    }
    uint32_t a = max(m & 0xffffu, m >> 16);
    a = __reduce_max_sync(0xffffffffu, a);
    if ((threadIdx.x & 31) == 0 && a != 0) atomicMax(amax_bits, a << 16);   // fp32 bit pattern of the bf16 maximum
}

__device__ __forceinline__ float e4m3_decode(uint32_t c) {
    const uint32_t e = (c >> 3) & 0xfu, m = c & 7u;
    if (e == 0) return static_cast<float>(m) * 0.001953125f;  // m * 2^-9, exact
    return __uint_as_float(((e + 120u) << 23) | (m << 20));
}

// Offset of scale (row r, scale column c) in the 128x4 tiled layout with `k_atoms` tiles along K.
__device__ __forceinline__ long long sf_tiled_offset(long long r, long long c, long long k_atoms) {
    const long long rr = r & 127;
    return ((r >> 7) * k_atoms + (c >> 2)) * 512 + (rr & 31) * 16 + (rr >> 5) * 4 + (c & 3);
}

// Pack 8 floats (already divided by the block scale) into 8 E2M1 nibbles, element i in nibble i.
__device__ __forceinline__ uint32_t pack8_e2m1(const float (&y)[8]) {
    uint32_t w = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const __nv_fp4x2_storage_t b = __nv_cvt_float2_to_fp4x2(make_float2(y[2 * i], y[2 * i + 1]), __NV_E2M1, cudaRoundNearest);
        w |= static_cast<uint32_t>(b) << (8 * i);
    }
    return w;
}

// The same for four (even, odd) element pairs.
__device__ __forceinline__ uint32_t pack8_e2m1_pairs(const float2 (&y)[4]) {
    uint32_t w = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const __nv_fp4x2_storage_t b = __nv_cvt_float2_to_fp4x2(y[i], __NV_E2M1, cudaRoundNearest);
        w |= static_cast<uint32_t>(b) << (8 * i);
    }
    return w;
}

// max |x| over N words of bf16 pairs, as the bf16 bit pattern of the maximum (magnitudes of finite bf16 values
// order like unsigned 16-bit integers): one AND per word and one three-input packed maximum per two words.
template <int N>
__device__ __forceinline__ uint32_t block_amax_bits(const uint32_t* __restrict__ rw) {
    constexpr uint32_t kMag = 0x7fff7fffu;
    uint32_t m = rw[0] & kMag;
#pragma unroll
    for (int i = 1; i + 1 < N; i += 2) m = __vimax3_u16x2(m, rw[i] & kMag, rw[i + 1] & kMag);
    if ((N & 1) == 0) m = __vimax3_u16x2(m, rw[N - 1] & kMag, 0u);
    return max(m & 0xffffu, m >> 16);
}

// FMT: kFmtNvfp4 (16-element blocks, E4M3 scale relative to the tensor scale gs) or
// kFmtMxfp4 (32-element blocks, E8M0 scale).  TILED: scale bytes go to the 128x4 tiled
// layout (rows padded to 128 and scale columns to 4, padding written as zero).
//
// amax_bits != nullptr: gs = amax / 2688 (1 when amax == 0), also stored to *gs_io.
// amax_bits == nullptr: gs = *gs_io (caller-supplied static scale).
// x / d for d > 0, bit-identical to IEEE division, at the cost of a multiply and two fused
// multiply-adds: with r the correctly rounded reciprocal of d, q0 = RN(x*r) is within one ulp of
// x/d, rem = x - q0*d is exact in an FMA, and RN(q0 + rem*r) is the correctly rounded quotient
// (Markstein's theorem).  The theorem excludes a divisor whose significand is all ones, and the
// reciprocal must neither overflow nor lose bits, so those divisors take the plain division.
// The sign of a zero quotient is taken from x, as division would give.
__device__ __forceinline__ bool divisor_is_plain(float d) {
    const uint32_t b = __float_as_uint(d);
    const uint32_t e = (b >> 23) & 0xffu;
    return (b & 0x7fffffu) != 0x7fffffu && e >= 32u && e <= 222u;
}

__device__ __forceinline__ float div_by_recip(float x, float d, float r) {
    const float q0 = __fmul_rn(x, r);
    const float rem = __fmaf_rn(-q0, d, x);
    return copysignf(__fmaf_rn(rem, r, q0), x);
}

// One block of BLK consecutive elements held by a single lane: block maximum, scale code, then the
// BLK elements divided by the block scale and packed, 8 nibbles per 32-bit word.
template <int FMT>
__device__ __forceinline__ uint32_t quantize_block(const uint32_t* __restrict__ rw, float gs, bool gs_plain, float gs_recip,
                                                   float sixth, uint32_t* __restrict__ out_words) {
    constexpr int BLK = (FMT == kFmtNvfp4) ? 16 : 32;
    const float a = __uint_as_float(block_amax_bits<BLK / 2>(rw) << 16);
    uint32_t code;
    if (FMT == kFmtNvfp4) {
        // 6 is a plain divisor; a quotient in the subnormal range takes the plain division
        const float t = (__float_as_uint(a) >= (32u << 23)) ? div_by_recip(a, 6.0f, sixth) : __fdiv_rn(a, 6.0f);
        const float u = fminf(gs_plain ? div_by_recip(t, gs, gs_recip) : __fdiv_rn(t, gs), 448.0f);
        code = static_cast<uint32_t>(__nv_cvt_float_to_fp8(u, __NV_SATFINITE, __NV_E4M3));
        const float d = __fmul_rn(e4m3_decode(code), gs);
        // one of three paths per block, chosen outside the element loops: the common one (reciprocal
        // division), all-zero block scale, and the rare divisors that need the plain division
        if (d != 0.0f && divisor_is_plain(d)) {
            // x / d by the reciprocal (see div_by_recip), two elements per instruction with the packed fp32
            // multiply and FMA of sm_100, and computed as -(x / d): with nr = -RN(1/d), q0 = x*nr, t = x + q0*d,
            // -q = q0 + t*nr.  Every step is the mirror image of the positive-sign sequence, so the rounding is
            // the same, and a zero quotient comes out with the sign opposite to x's in every case (x = -0
            // included), which the final XOR of the eight sign bits turns into x's sign -- no per-element fix-up.
            const float nr = -__frcp_rn(d);
            const float2 d2 = make_float2(d, d), nr2 = make_float2(nr, nr);
#pragma unroll
            for (int w = 0; w < BLK / 8; ++w) {
                float2 y[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float2 x2 = make_float2(__uint_as_float(rw[w * 4 + i] << 16), __uint_as_float(rw[w * 4 + i] & 0xffff0000u));
                    const float2 q0 = __fmul2_rn(x2, nr2);
                    const float2 t = __ffma2_rn(q0, d2, x2);
                    y[i] = __ffma2_rn(t, nr2, q0);
                }
                out_words[w] = pack8_e2m1_pairs(y) ^ 0x88888888u;
            }
        } else if (d == 0.0f) {
#pragma unroll
            for (int w = 0; w < BLK / 8; ++w) {
                // magnitudes are zero, each nibble keeps the sign bit of its element
                uint32_t word = 0;
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const uint32_t v = rw[w * 4 + i];
                    word |= ((v >> 15) & 1u) << (8 * i + 3);      // low half = even element
                    word |= ((v >> 31) & 1u) << (8 * i + 7);      // high half = odd element
                }
                out_words[w] = word;
            }
        } else {
#pragma unroll
            for (int w = 0; w < BLK / 8; ++w) {
                float y[8];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    y[2 * i] = __fdiv_rn(__uint_as_float(rw[w * 4 + i] << 16), d);
                    y[2 * i + 1] = __fdiv_rn(__uint_as_float(rw[w * 4 + i] & 0xffff0000u), d);
                }
                out_words[w] = pack8_e2m1(y);
            }
        }
    } else {
        if (a == 0.0f) {
            code = 127u;
        } else {
            const int E = static_cast<int>((__float_as_uint(a) >> 23) & 0xffu);
            code = static_cast<uint32_t>(max(E - 2, 0));
        }
        const float inv = __uint_as_float((254u - code) << 23);  // 2^(127-code), exact scaling
        const float2 inv2 = make_float2(inv, inv);
#pragma unroll
        for (int w = 0; w < BLK / 8; ++w) {
            float2 y[4];
#pragma unroll
            for (int i = 0; i < 4; ++i)
                y[i] = __fmul2_rn(make_float2(__uint_as_float(rw[w * 4 + i] << 16), __uint_as_float(rw[w * 4 + i] & 0xffff0000u)), inv2);
            out_words[w] = pack8_e2m1_pairs(y);
        }
    }
    return code;
}

// ---- NVFP4 items without branches on the common path --------------------------------------------------------
// quantize_block picks one of three paths per block, and every such branch ends the stretch of code the compiler
// can schedule as one, so a lane works through its blocks one dependent chain after the other.  The functions below
// split the work in two phases over NI items (2 * NI blocks of 16 elements) held by one lane: first the scale
// chain of every block (block maximum -> a / 6 / gs -> E4M3 code -> d = code value * gs -> -1 / d), all independent
// of one another, then the element divisions of every block.  The common case needs no branch at all: a block whose
// scale rounds to zero takes -0 as its "reciprocal" (every quotient becomes a zero of the sign opposite to x's,
// which the final XOR turns into x's sign, exactly what the all-zero path of quantize_block writes), and the rare
// cases the reciprocal method does not cover (a tiny non-zero maximum, a divisor with an all-ones significand or an
// extreme exponent, a tensor scale that is not a plain divisor) raise a flag, upon which the lane redoes all of
// its items with quantize_block.  The bytes are those of quantize_block in every case.
__device__ __forceinline__ void nvfp4_scale_chain(const uint32_t* __restrict__ rw, float gs, float gs_recip, float sixth,
                                                  uint32_t& code, float& d, float& nr, bool& rare) {
    const uint32_t abits = block_amax_bits<8>(rw) << 16;
    const float a = __uint_as_float(abits);
    const float t = div_by_recip(a, 6.0f, sixth);
    const float u = fminf(div_by_recip(t, gs, gs_recip), 448.0f);
    code = static_cast<uint32_t>(__nv_cvt_float_to_fp8(u, __NV_SATFINITE, __NV_E4M3));
    d = __fmul_rn(e4m3_decode(code), gs);
    // a non-zero maximum below 2^-95 (its quotient by 6 may be subnormal) and divisors outside the theorem
    rare = (abits - 1u < (32u << 23) - 1u) || (d != 0.0f && !divisor_is_plain(d));
    nr = (d != 0.0f) ? -__frcp_rn(d) : -0.0f;
}

__device__ __forceinline__ void nvfp4_pack_block(const uint32_t* __restrict__ rw, float d, float nr, uint32_t* __restrict__ out_words) {
    const float2 d2 = make_float2(d, d), nr2 = make_float2(nr, nr);
#pragma unroll
    for (int w = 0; w < 2; ++w) {
        float2 y[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 x2 = make_float2(__uint_as_float(rw[w * 4 + i] << 16), __uint_as_float(rw[w * 4 + i] & 0xffff0000u));
            const float2 q0 = __fmul2_rn(x2, nr2);
            const float2 t = __ffma2_rn(q0, d2, x2);
            y[i] = __ffma2_rn(t, nr2, q0);
        }
        out_words[w] = pack8_e2m1_pairs(y) ^ 0x88888888u;
    }
}

// NI items of 32 elements (rw[i][0..15] = 16 words of bf16 pairs) -> o[i][0..3] packed nibbles, codes[i] = the two
// scale bytes (block 0 in bits 7:0, block 1 in bits 15:8).
template <int NI>
__device__ __forceinline__ void quantize_items_nvfp4(const uint32_t (&rw)[NI][16], float gs, bool gs_plain, float gs_recip, float sixth,
                                                     uint32_t (&o)[NI][4], uint32_t (&codes)[NI]) {
    uint32_t code[2 * NI];
    float d[2 * NI], nr[2 * NI];
    bool rare = !gs_plain;
#pragma unroll
    for (int b = 0; b < 2 * NI; ++b) {
        bool r;
        nvfp4_scale_chain(&rw[b >> 1][(b & 1) * 8], gs, gs_recip, sixth, code[b], d[b], nr[b], r);
        rare = rare || r;
    }
    if (!rare) {
#pragma unroll
        for (int b = 0; b < 2 * NI; ++b) nvfp4_pack_block(&rw[b >> 1][(b & 1) * 8], d[b], nr[b], &o[b >> 1][(b & 1) * 2]);
#pragma unroll
        for (int i = 0; i < NI; ++i) codes[i] = code[2 * i] | (code[2 * i + 1] << 8);
    } else {
#pragma unroll 1
        for (int i = 0; i < NI; ++i) {
            const uint32_t c0 = quantize_block<kFmtNvfp4>(&rw[i][0], gs, gs_plain, gs_recip, sixth, &o[i][0]);
            const uint32_t c1 = quantize_block<kFmtNvfp4>(&rw[i][8], gs, gs_plain, gs_recip, sixth, &o[i][2]);
            codes[i] = c0 | (c1 << 8);
        }
    }
}

// ---- per-launch tables for the scale chain ------------------------------------------------------------------
// With the tensor scale fixed for a launch, the scale chain of a block depends only on the block maximum a, a bf16
// value m * 2^e with one of 128 significands m in [1, 2):  RN(RN(a / 6) / gs) = RN(RN(m / 6) / gs) * 2^e, because
// scaling by a power of two is exact as long as nothing leaves the normal range (outside it the E4M3 code is 0 or
// saturates either way).  So a CTA computes u_m = RN(RN(m / 6) / gs) once for the 128 significands with true
// divisions, and for each of the 127 E4M3 codes the divisor d = value(code) * gs with its negated reciprocal; a
// block then needs two shared-memory reads, a multiply by 2^e and the E4M3 conversion instead of two emulated
// divisions, a decode, a reciprocal and the checks on d.  An entry whose divisor the reciprocal method does not
// cover carries +0 as its reciprocal (a real one is negative, a zero divisor has -0), which sends the lane to
// quantize_block like the other rare cases.  `usable` is false when gs is so large or small that u_m itself
// leaves the normal range; the launch then takes the path without tables.
struct Nvfp4Tables {
    float u[128];        // u_m for m = 1 + i / 128
    float2 dn[128];      // (d, -1/d) per E4M3 code 0 .. 126 (127 unused)
    int usable;
};

__device__ __forceinline__ void nvfp4_build_tables(Nvfp4Tables& t, float gs, int tid, int nthreads) {
    if (tid == 0) t.usable = 1;
    __syncthreads();
    for (int i = tid; i < 256; i += nthreads) {
        if (i < 128) {
            const float m = __uint_as_float(0x3f800000u | (static_cast<uint32_t>(i) << 16));
            const float u = __fdiv_rn(__fdiv_rn(m, 6.0f), gs);
            t.u[i] = u;
            const uint32_t e = (__float_as_uint(u) >> 23) & 0xffu;
            if (e < 40u || e > 214u) t.usable = 0;     // scaling by 2^e of any bf16 maximum must stay exact (or saturate)
        } else {
            const uint32_t c = static_cast<uint32_t>(i - 128);
            const float d = __fmul_rn(e4m3_decode(c), gs);
            float nr = -0.0f;
            if (d != 0.0f) nr = divisor_is_plain(d) ? -__frcp_rn(d) : 0.0f;
            t.dn[c] = make_float2(d, nr);
        }
    }
    __syncthreads();
}

__device__ __forceinline__ void nvfp4_scale_chain_tab(const uint32_t* __restrict__ rw, const Nvfp4Tables& t,
                                                      uint32_t& code, float& d, float& nr, bool& rare) {
    const uint32_t abits = block_amax_bits<8>(rw) << 16;
    const float u = fminf(__fmul_rn(t.u[(abits >> 16) & 0x7fu], __uint_as_float(abits & 0x7f800000u)), 448.0f);
    code = static_cast<uint32_t>(__nv_cvt_float_to_fp8(u, __NV_SATFINITE, __NV_E4M3));
    const float2 dn = t.dn[code];
    d = dn.x;
    nr = dn.y;
    // a non-zero maximum below 2^-95 (its quotient by 6 may be subnormal) and divisors outside the theorem
    rare = (abits - 1u < (32u << 23) - 1u) || (__float_as_uint(nr) == 0u);
}

// As quantize_items_nvfp4, with the scale chains read from the launch's tables.
template <int NI>
__device__ __forceinline__ void quantize_items_nvfp4_tab(const uint32_t (&rw)[NI][16], const Nvfp4Tables& t, float gs, bool gs_plain,
                                                         float gs_recip, float sixth, uint32_t (&o)[NI][4], uint32_t (&codes)[NI]) {
    uint32_t code[2 * NI];
    float d[2 * NI], nr[2 * NI];
    bool rare = false;
#pragma unroll
    for (int b = 0; b < 2 * NI; ++b) {
        bool r;
        nvfp4_scale_chain_tab(&rw[b >> 1][(b & 1) * 8], t, code[b], d[b], nr[b], r);
        rare = rare || r;
    }
    if (!rare) {
#pragma unroll
        for (int b = 0; b < 2 * NI; ++b) nvfp4_pack_block(&rw[b >> 1][(b & 1) * 8], d[b], nr[b], &o[b >> 1][(b & 1) * 2]);
#pragma unroll
        for (int i = 0; i < NI; ++i) codes[i] = code[2 * i] | (code[2 * i + 1] << 8);
    } else {
#pragma unroll 1
        for (int i = 0; i < NI; ++i) {
            const uint32_t c0 = quantize_block<kFmtNvfp4>(&rw[i][0], gs, gs_plain, gs_recip, sixth, &o[i][0]);
            const uint32_t c1 = quantize_block<kFmtNvfp4>(&rw[i][8], gs, gs_plain, gs_recip, sixth, &o[i][2]);
            codes[i] = c0 | (c1 << 8);
        }
    }
}

// The quantise loop shared by the kernels below: warp `warp_global` of `warps_total` takes the
// 1024-element steps warp_global, warp_global + warps_total, ... of the (rows, k) matrix.  Inside a
// step lane L owns the 32 consecutive elements 32L .. 32L+31: four 128-bit loads (64 contiguous bytes),
// two whole NVFP4 blocks or one MXFP4 block (so a block maximum needs no exchange between lanes),
// one 128-bit store of 32 nibbles and one 16-bit / 8-bit scale store.
template <int FMT, bool TILED>
__device__ __forceinline__ void quantize_rows(const __nv_bfloat16* __restrict__ x, long long rows, long long k, long long ldx,
                                              float gs, uint8_t* __restrict__ packed, uint8_t* __restrict__ sf,
                                              long long warp_global, long long warps_total, const Nvfp4Tables* tab = nullptr) {
    constexpr int BLK = (FMT == kFmtNvfp4) ? 16 : 32;
    const int lane = threadIdx.x & 31;
    // a / 6 / gs is needed once per block; both divisors are fixed for the launch
    const bool gs_plain = divisor_is_plain(gs);
    const float gs_recip = __frcp_rn(gs);
    const float sixth = __frcp_rn(6.0f);

    const int kk = static_cast<int>(k);
    const int sf_cols = kk / BLK;
    const int k_atoms = (sf_cols + 3) / 4;
    const long long rows_pad = TILED ? ((rows + 127) / 128) * 128 : rows;
    const int k_pad = TILED ? k_atoms * 4 * BLK : kk;
    const int chunks = (k_pad + 1023) / 1024;
    const long long items = rows_pad * chunks;

    // (row, chunk) of the current item, advanced without a division per item
    long long r = warp_global / chunks;
    int ch = static_cast<int>(warp_global - r * chunks);
    const long long step_r = warps_total / chunks;
    const int step_c = static_cast<int>(warps_total - step_r * chunks);
    // The loads of the next item are issued before the arithmetic of the current one, so that a warp always has
    // 64 bytes per lane on their way while it computes (the scale chain and the exact divisions are long enough
    // for memory latency to show otherwise).
    auto fetch = [&](long long rr, int cc, uint32_t (&dst)[16]) -> bool {
        const int e = cc * 1024 + lane * 32;
        const bool in = (rr < rows) && (e < kk);
        if (in) {
            const uint4* src = reinterpret_cast<const uint4*>(x + rr * ldx + e);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const uint4 v = __ldg(src + i);
                dst[4 * i] = v.x; dst[4 * i + 1] = v.y; dst[4 * i + 2] = v.z; dst[4 * i + 3] = v.w;
            }
        }
        return in;
    };
    uint32_t rw1[1][16];
    uint32_t (&rw)[16] = rw1[0];
    bool in = (warp_global < items) && fetch(r, ch, rw);
    for (long long item = warp_global; item < items; item += warps_total) {
        // next item of this warp
        long long rn = r + step_r;
        int cn = ch + step_c;
        if (cn >= chunks) { cn -= chunks; ++rn; }
        uint32_t nx[16];
        const bool in_next = (item + warps_total < items) && fetch(rn, cn, nx);
        const int e = ch * 1024 + lane * 32;   // this lane's first element
        const int c = e / BLK;                 // ... and first scale column
        if (!in) {
            // padding of the tiled scale layout (rows up to a multiple of 128, columns of 4): zero bytes
            if (TILED && e < k_pad) {
                uint8_t* p = sf + sf_tiled_offset(r, c, k_atoms);
                if (FMT == kFmtNvfp4) *reinterpret_cast<uint16_t*>(p) = 0;
                else *p = 0;
            }
        } else {
            uint32_t o1[1][4];
            uint32_t (&o)[4] = o1[0];
            uint32_t codes;
            if (FMT == kFmtNvfp4) {
                uint32_t c1[1];
                if (tab != nullptr) quantize_items_nvfp4_tab<1>(rw1, *tab, gs, gs_plain, gs_recip, sixth, o1, c1);
                else quantize_items_nvfp4<1>(rw1, gs, gs_plain, gs_recip, sixth, o1, c1);
                codes = c1[0];
            } else {
                codes = quantize_block<FMT>(rw, gs, gs_plain, gs_recip, sixth, o);
            }
            __stcs(reinterpret_cast<uint4*>(packed + r * (kk / 2) + e / 2), make_uint4(o[0], o[1], o[2], o[3]));
            uint8_t* p = TILED ? sf + sf_tiled_offset(r, c, k_atoms) : sf + r * sf_cols + c;
            if (FMT == kFmtNvfp4) *reinterpret_cast<uint16_t*>(p) = static_cast<uint16_t>(codes);   // columns c, c+1 (c even)
            else *p = static_cast<uint8_t>(codes);
        }
        r = rn;
        ch = cn;
        in = in_next;
#pragma unroll
        for (int i = 0; i < 16; ++i) rw[i] = nx[i];
    }
}

// 128 threads per block: at the NVFP4 kernel's 70-71 registers 7 such blocks (28 warps) are resident on an SM where
// 256-thread blocks give 3 (24 warps); NVFP4 at 8192^2 33.1 -> 31.8 us, MXFP4 unchanged (64 threads, 14 blocks, more
// scale tables to build: 33.1 us).
constexpr int kQuantThreads = 128;

template <int FMT, bool TILED>
__global__ void __launch_bounds__(kQuantThreads)
quantize_fp4_kernel(const __nv_bfloat16* __restrict__ x, long long rows, long long k, long long ldx,
                    const unsigned int* __restrict__ amax_bits, float* __restrict__ gs_io,
                    uint8_t* __restrict__ packed, uint8_t* __restrict__ sf) {
    // a kernel queued behind this one with programmatic stream serialisation may start its prologue now
    // (it still waits for this grid to finish before it reads what is written here); this kernel is launched
    // the same way and waits for its own predecessor before it touches memory
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const long long warp_global = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
    const long long warps_total = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
    float gs = 1.0f;
    if (FMT == kFmtNvfp4) {
        if (amax_bits != nullptr) {
            const float amax = __uint_as_float(*amax_bits);
            gs = (amax == 0.0f) ? 1.0f : __fdiv_rn(amax, 2688.0f);
            if (blockIdx.x == 0 && threadIdx.x == 0) *gs_io = gs;
        } else {
            gs = *gs_io;
        }
    }
    if constexpr (FMT == kFmtNvfp4) {
        __shared__ Nvfp4Tables tab;
        nvfp4_build_tables(tab, gs, threadIdx.x, blockDim.x);
        quantize_rows<FMT, TILED>(x, rows, k, ldx, gs, packed, sf, warp_global, warps_total, tab.usable ? &tab : nullptr);
    } else {
        quantize_rows<FMT, TILED>(x, rows, k, ldx, gs, packed, sf, warp_global, warps_total);
    }
}

// Small activations (decode: 16 x 8192): tensor amax and NVFP4 quantise in ONE launch of one
// 8-CTA cluster.  Each CTA reduces its share of |x|, the eight partial maxima are exchanged through
// distributed shared memory, and every CTA then quantises its share with the same tensor scale --
// instead of a memset, an amax kernel and a quantise kernel (three launches on the decode path).
constexpr int kFusedClusterCtas = 8;
constexpr int kFusedThreads = 512;

template <bool TILED>
__global__ void __cluster_dims__(kFusedClusterCtas, 1, 1) __launch_bounds__(kFusedThreads)
quantize_nvfp4_fused_small_kernel(const __nv_bfloat16* __restrict__ x, long long rows, long long k, long long ldx,
                                  float* __restrict__ gs_out, uint8_t* __restrict__ packed, uint8_t* __restrict__ sf) {
    __shared__ float s_warp[kFusedThreads / 32];
    __shared__ float s_cta;
    // Launched with programmatic stream serialisation: this grid may be scheduled while the previous kernel in
    // the stream is still running, which hides its launch latency on the decode path; it touches memory only after
    // that kernel has finished, and lets the kernel behind it start its own set-up right away.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    uint32_t rank;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
    const int tid = threadIdx.x;
    const long long groups_per_row = k / 8;
    const long long total = rows * groups_per_row;
    const long long stride = static_cast<long long>(kFusedClusterCtas) * kFusedThreads;
    float a = 0.0f;
    for (long long g0 = static_cast<long long>(rank) * kFusedThreads + tid; g0 < total; g0 += 4 * stride) {
        uint4 v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const long long g = g0 + u * stride;
            v[u] = make_uint4(0, 0, 0, 0);
            if (g < total) {
                const long long r = g / groups_per_row;
                v[u] = __ldg(reinterpret_cast<const uint4*>(x + r * ldx + (g - r * groups_per_row) * 8));
            }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const uint32_t w[4] = {v[u].x, v[u].y, v[u].z, v[u].w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                a = fmaxf(a, fabsf(__uint_as_float(w[i] << 16)));
                a = fmaxf(a, fabsf(__uint_as_float(w[i] & 0xffff0000u)));
            }
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, o));
    if ((tid & 31) == 0) s_warp[tid >> 5] = a;
    __syncthreads();
    if (tid < 32) {
        float b = (tid < kFusedThreads / 32) ? s_warp[tid] : 0.0f;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) b = fmaxf(b, __shfl_xor_sync(0xffffffffu, b, o));
        if (tid == 0) s_cta = b;
    }
    // cluster barrier (release/acquire): every CTA's maximum is visible to the others afterwards
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
    float amax = 0.0f;
    const uint32_t mine = static_cast<uint32_t>(__cvta_generic_to_shared(&s_cta));
#pragma unroll
    for (int c = 0; c < kFusedClusterCtas; ++c) {
        uint32_t remote;
        float v;
        asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(mine), "r"(c));
        asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(remote) : "memory");
        amax = fmaxf(amax, v);
    }
    const float gs = (amax == 0.0f) ? 1.0f : __fdiv_rn(amax, 2688.0f);
    if (rank == 0 && tid == 0) *gs_out = gs;
    const long long warp_global = (static_cast<long long>(rank) * kFusedThreads + tid) >> 5;
    const long long warps_total = (static_cast<long long>(kFusedClusterCtas) * kFusedThreads) >> 5;
    quantize_rows<kFmtNvfp4, TILED>(x, rows, k, ldx, gs, packed, sf, warp_global, warps_total);
    // no CTA may exit while another can still read its shared memory
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// Decode-sized activations (up to 8192 blocks of 16 elements, e.g. 16 x 8192): the same single launch of one 8-CTA
// cluster, arranged for the shortest dependent chain, because the decode GEMM queued behind it can do nothing but
// prefetch weights until these bytes exist.  One 16-element block per thread (8 x 1024 threads): the thread loads
// its 32 bytes once and keeps them in registers across the cluster-wide amax exchange, so the chain is
// load -> block maximum -> warp / CTA / cluster maximum -> one block's scale chain and 16 divisions -> store,
// instead of two passes over memory with a 32-element item per lane.  Same bytes as the kernels above.
constexpr int kDecodeQuantThreads = 1024;
constexpr long long kDecodeQuantBlocks = static_cast<long long>(kFusedClusterCtas) * kDecodeQuantThreads;   // 8192

template <bool TILED>
__global__ void __cluster_dims__(kFusedClusterCtas, 1, 1) __launch_bounds__(kDecodeQuantThreads, 1)
quantize_nvfp4_decode_kernel(const __nv_bfloat16* __restrict__ x, int rows, int k, long long ldx,
                             float* __restrict__ gs_out, uint8_t* __restrict__ packed, uint8_t* __restrict__ sf) {
    __shared__ uint32_t s_warp[kDecodeQuantThreads / 32];
    __shared__ uint32_t s_all[kFusedClusterCtas];     // every CTA's maximum, written here by the CTAs themselves
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    uint32_t rank;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
    const int tid = threadIdx.x;
    const int gtid = static_cast<int>(rank) * kDecodeQuantThreads + tid;
    const int sf_cols = k / 16;
    const int k_atoms = (sf_cols + 3) / 4;
    const int blocks = rows * sf_cols;
    const bool mine = gtid < blocks;
    const int row = mine ? gtid / sf_cols : 0;
    const int cb = mine ? gtid - row * sf_cols : 0;
    uint32_t rw[8] = {0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u};
    if (mine) {
        const uint4* src = reinterpret_cast<const uint4*>(x + static_cast<long long>(row) * ldx + cb * 16);
        const uint4 v0 = __ldg(src), v1 = __ldg(src + 1);
        rw[0] = v0.x; rw[1] = v0.y; rw[2] = v0.z; rw[3] = v0.w;
        rw[4] = v1.x; rw[5] = v1.y; rw[6] = v1.z; rw[7] = v1.w;
    }
    if (TILED) {
        // padding of the tiled scale layout (rows up to 128, scale columns up to a multiple of 4), independent of the data
        const int rows_pad = ((rows + 127) / 128) * 128;
        for (int i = gtid; i < rows_pad * k_atoms; i += static_cast<int>(kDecodeQuantBlocks)) {
            const int r = i / k_atoms, a = i - r * k_atoms;
            uint8_t* p = sf + sf_tiled_offset(r, a * 4, k_atoms);
            if (r >= rows) {
                *reinterpret_cast<uint32_t*>(p) = 0u;
            } else {
                for (int c = a * 4; c < a * 4 + 4; ++c)
                    if (c >= sf_cols) p[c & 3] = 0;
            }
        }
    }
    // block maximum as bf16 bits (kept for the scale chain), then warp -> CTA -> cluster
    const uint32_t a_bits = block_amax_bits<8>(rw);
    uint32_t a = __reduce_max_sync(0xffffffffu, a_bits);
    if ((tid & 31) == 0) s_warp[tid >> 5] = a;
    __syncthreads();
    if (tid < 32) {
        a = __reduce_max_sync(0xffffffffu, s_warp[tid]);
        // lane c pushes this CTA's maximum into slot `rank` of CTA c: after the one cluster barrier below every
        // CTA finds all eight maxima in its own shared memory, and nobody reads a remote CTA afterwards
        if (tid < kFusedClusterCtas) {
            const uint32_t slot = static_cast<uint32_t>(__cvta_generic_to_shared(&s_all[rank]));
            uint32_t remote;
            asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(slot), "r"(tid));
            asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(remote), "r"(a) : "memory");
        }
    }
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
    uint32_t amax_bits = 0;
#pragma unroll
    for (int c = 0; c < kFusedClusterCtas; ++c) amax_bits = max(amax_bits, s_all[c]);
    const float amax = __uint_as_float(amax_bits << 16);
    const float gs = (amax == 0.0f) ? 1.0f : __fdiv_rn(amax, 2688.0f);
    if (gtid == 0) *gs_out = gs;
    if (mine) {
        uint32_t o[2];
        const uint32_t code = quantize_block<kFmtNvfp4>(rw, gs, divisor_is_plain(gs), __frcp_rn(gs), __frcp_rn(6.0f), o);
        *reinterpret_cast<uint2*>(packed + static_cast<long long>(row) * (k / 2) + cb * 8) = make_uint2(o[0], o[1]);
        sf[TILED ? sf_tiled_offset(row, cb, k_atoms) : static_cast<long long>(row) * sf_cols + cb] = static_cast<uint8_t>(code);
    }
}

// Row-major (rows, cols) scale bytes -> 128x4 tiled layout (padding zero).
__global__ void __launch_bounds__(256)
sf_to_tiled_kernel(const uint8_t* __restrict__ src, long long rows, long long cols, uint8_t* __restrict__ dst) {
    const long long k_atoms = (cols + 3) / 4;
    const long long rows_pad = ((rows + 127) / 128) * 128;
    const long long total = rows_pad * k_atoms;  // one thread per (row, 4 scale columns)
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        const long long r = i / k_atoms;
        const long long a = i - r * k_atoms;
        uint32_t word = 0;
        if (r < rows) {
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const long long col = a * 4 + c;
                if (col < cols) word |= static_cast<uint32_t>(src[r * cols + col]) << (8 * c);
            }
        }
        *reinterpret_cast<uint32_t*>(dst + sf_tiled_offset(r, a * 4, k_atoms)) = word;
    }
}

}  // namespace avefp4

namespace avefp4 {

// Packed E2M1 weights, row-major (rows, k/2 bytes) -> tile-major: 16 KB tiles of 128 rows x 128
// bytes (256 K elements), ordered [row block][K block], rows and K padded with zero bytes.  A
// CTA that walks the K blocks of one row block then reads one contiguous stream from HBM.
__global__ void __launch_bounds__(256)
pack_weight_tiles_kernel(const uint8_t* __restrict__ src, long long rows, long long kbytes, uint8_t* __restrict__ dst) {
    const long long kb_n = (kbytes + 127) / 128;
    const long long rb_n = (rows + 127) / 128;
    const long long total = rb_n * kb_n * 128 * 8;  // one thread per 16 bytes
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        const long long c = i & 7;            // 16-byte chunk in the 128-byte row piece
        const long long r = (i >> 3) & 127;   // row inside the tile
        const long long tile = i >> 10;
        const long long rb = tile / kb_n, kb = tile - rb * kb_n;
        const long long row = rb * 128 + r;
        const long long col = kb * 128 + c * 16;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (row < rows && col < kbytes) v = __ldg(reinterpret_cast<const uint4*>(src + row * kbytes + col));
        *reinterpret_cast<uint4*>(dst + i * 16) = v;
    }
}

}  // namespace avefp4
