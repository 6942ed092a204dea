/*
 * CPU oracle for the block-scaled FP4 path (NVFP4 / MXFP4 quantise, dequantise,
 * D = A * B^T with fp32 result rounded to bf16).
 *
 * TEST INFRASTRUCTURE ONLY.  Nothing in the shipped package links, imports or
 * executes this file; it exists so that tests, the smoke check and the CPU leg
 * of the benchmark have an independent statement of the arithmetic.
 *
 * PARITY UNPINNED: the reference project (causalflow-ai/avelang) contains no FP4
 * code, golden vector or known-answer test.  What the reference does pin is the
 * GEMM half of the oracle, the expression
 *     expected = (A.float() @ B.float().T).to(torch.bfloat16)
 * (test/examples/gemm/amdgpu/test_amdgpu_gemm.py:27,
 *  benchmark/gemm/bench_amdgpu_gemm.py:63), and the operand convention
 * A (M,K), B (N,K), K contiguous, D = A * B^T
 * (python/avelang_kernels/amdgpu_gemm.py:458-494).  ave_oracle_gemm_bf16 below
 * restates exactly that expression.  The quantise / dequantise half follows the
 * public OCP Microscaling (MX) v1.0 element/scale formats and the NVFP4
 * convention (16-element blocks, E4M3 block scale, fp32 tensor scale); its
 * element and scale rounding is cross-checked in tests against ml_dtypes'
 * float4_e2m1fn / float8_e4m3fn casts.
 *
 * Every fp32 operation below is a single IEEE-754 binary32 round-to-nearest-even
 * operation: build with -ffp-contract=off and without -ffast-math.
 *
 * Storage convention (shared with the CUDA path):
 *   packed : uint8 (R, K/2); byte j of a row = element 2j in bits 3:0,
 *            element 2j+1 in bits 7:4.  Nibble = s e e m (E2M1, bias 1).
 *   scales : uint8 (R, K/blk) row-major; E4M3 (NVFP4, blk 16) or E8M0 (MXFP4, blk 32).
 *   global : one fp32 (NVFP4 only).
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define AVE_FMT_NVFP4 0
#define AVE_FMT_MXFP4 1

static inline float bits_to_f32(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }
static inline uint32_t f32_to_bits(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }
static inline float bf16_to_f32(uint16_t h) { return bits_to_f32((uint32_t)h << 16); }

/* fp32 -> bf16, round to nearest even (the rounding torch's .to(bfloat16) uses). */
uint16_t ave_oracle_f32_to_bf16(float f) {
    uint32_t u = f32_to_bits(f);
    if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40u); /* NaN */
    uint32_t lsb = (u >> 16) & 1u;
    u += 0x7fffu + lsb;
    return (uint16_t)(u >> 16);
}

/* E2M1 magnitudes for codes 0..7. */
static const float kE2M1[8] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f};

/* |y| -> E2M1 magnitude code, round to nearest, ties to the code with an even
 * mantissa bit, saturating at 6. */
uint8_t ave_oracle_e2m1_code(float ay) {
    if (ay <= 0.25f) return 0;
    if (ay < 0.75f) return 1;
    if (ay <= 1.25f) return 2;
    if (ay < 1.75f) return 3;
    if (ay <= 2.5f) return 4;
    if (ay < 3.5f) return 5;
    if (ay <= 5.0f) return 6;
    return 7;
}

/* u in [0, 448] -> E4M3 (float8_e4m3fn: bias 7, 3 mantissa bits, subnormal step
 * 2^-9) code, round to nearest even, saturating at 448 (0x7E); never NaN. */
uint8_t ave_oracle_e4m3_code(float u) {
    if (!(u > 0.0f)) return 0;
    if (u >= 448.0f) return 0x7e;
    if (u < 0.015625f) {                 /* below the smallest normal 2^-6 */
        float r = rintf(u * 512.0f);     /* exact scaling; rintf = RN-even */
        return (uint8_t)r;               /* 8 is the code of 2^-6 itself */
    }
    uint32_t b = f32_to_bits(u);
    uint32_t lsb = (b >> 20) & 1u;
    b += 0x7ffffu + lsb;
    b &= ~0xfffffu;
    int e = (int)(b >> 23) - 127 + 7;
    uint32_t m = (b >> 20) & 7u;
    uint32_t code = ((uint32_t)e << 3) | m;
    if (code > 0x7eu) code = 0x7e;
    return (uint8_t)code;
}

float ave_oracle_e4m3_decode(uint8_t c) {
    int e = (c >> 3) & 0xf;
    int m = c & 7;
    float v = (e == 0) ? ldexpf((float)m, -9) : ldexpf((float)(8 + m), e - 10);
    return (c & 0x80) ? -v : v;
}

float ave_oracle_e8m0_decode(uint8_t c) { return ldexpf(1.0f, (int)c - 127); }

/* max |x| over n bf16 values, as fp32. */
float ave_oracle_amax_bf16(const uint16_t *x, size_t n) {
    float t = 0.0f;
    for (size_t i = 0; i < n; ++i) {
        float a = fabsf(bf16_to_f32(x[i]));
        if (a > t) t = a;
    }
    return t;
}

/* global scale from the tensor amax: amax / (6 * 448); 1 when the tensor is all zero. */
float ave_oracle_global_scale(float amax) {
    if (amax == 0.0f) return 1.0f;
    return amax / 2688.0f;
}

/*
 * NVFP4 quantise of a (rows, k) bf16 matrix with row stride ldx (elements).
 *   per block of 16: a = max|x|; t = a/6; u = min(t/gs, 448); c = E4M3(u);
 *   d = decode(c)*gs; element code = E2M1(|x/d|) with the sign of x;
 *   d == 0 -> all magnitudes 0 (sign kept).
 */
void ave_oracle_quantize_nvfp4(const uint16_t *x, int64_t rows, int64_t k, int64_t ldx,
                               float gs, uint8_t *packed, uint8_t *scales) {
    int64_t nb = k / 16;
    #pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r) {
        const uint16_t *xr = x + r * ldx;
        for (int64_t b = 0; b < nb; ++b) {
            float v[16];
            float a = 0.0f;
            for (int i = 0; i < 16; ++i) {
                v[i] = bf16_to_f32(xr[b * 16 + i]);
                float av = fabsf(v[i]);
                if (av > a) a = av;
            }
            float t = a / 6.0f;
            float u = t / gs;
            if (u > 448.0f) u = 448.0f;
            uint8_t c = ave_oracle_e4m3_code(u);
            scales[r * nb + b] = c;
            float d = ave_oracle_e4m3_decode(c) * gs;
            for (int i = 0; i < 16; i += 2) {
                uint8_t q[2];
                for (int j = 0; j < 2; ++j) {
                    uint8_t sign = (uint8_t)((f32_to_bits(v[i + j]) >> 31) << 3);
                    uint8_t mag = 0;
                    if (d != 0.0f) mag = ave_oracle_e2m1_code(fabsf(v[i + j] / d));
                    q[j] = sign | mag;
                }
                packed[r * (k / 2) + (b * 16 + i) / 2] = (uint8_t)(q[0] | (q[1] << 4));
            }
        }
    }
}

/*
 * MXFP4 quantise (OCP MX v1.0 floor rule): per block of 32,
 *   a = max|x|; a == 0 -> scale code 127; else code = max(E - 2, 0) where E is
 *   the biased fp32 exponent field of a (so the shared exponent is
 *   floor(log2 a) - 2, clamped); d = 2^(code-127); element code = E2M1(|x/d|)
 *   (values in (6,8)*d saturate to 6).
 */
void ave_oracle_quantize_mxfp4(const uint16_t *x, int64_t rows, int64_t k, int64_t ldx,
                               uint8_t *packed, uint8_t *scales) {
    int64_t nb = k / 32;
    #pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r) {
        const uint16_t *xr = x + r * ldx;
        for (int64_t b = 0; b < nb; ++b) {
            float v[32];
            float a = 0.0f;
            for (int i = 0; i < 32; ++i) {
                v[i] = bf16_to_f32(xr[b * 32 + i]);
                float av = fabsf(v[i]);
                if (av > a) a = av;
            }
            int code;
            if (a == 0.0f) {
                code = 127;
            } else {
                int E = (int)((f32_to_bits(a) >> 23) & 0xffu);
                code = E - 2;
                if (code < 0) code = 0;
                if (code > 254) code = 254;
            }
            scales[r * nb + b] = (uint8_t)code;
            float d = ldexpf(1.0f, code - 127);
            for (int i = 0; i < 32; i += 2) {
                uint8_t q[2];
                for (int j = 0; j < 2; ++j) {
                    uint8_t sign = (uint8_t)((f32_to_bits(v[i + j]) >> 31) << 3);
                    uint8_t mag = ave_oracle_e2m1_code(fabsf(v[i + j] / d));
                    q[j] = sign | mag;
                }
                packed[r * (k / 2) + (b * 32 + i) / 2] = (uint8_t)(q[0] | (q[1] << 4));
            }
        }
    }
}

/* Dequantise to fp32: sign * ((mag * s_b) * gs) for NVFP4 (mag*s_b is exact, one
 * rounding in the multiply by gs); sign * mag * 2^(code-127) for MXFP4. */
void ave_oracle_dequantize(const uint8_t *packed, const uint8_t *scales, float gs, int fmt,
                           int64_t rows, int64_t k, float *out) {
    int blk = (fmt == AVE_FMT_NVFP4) ? 16 : 32;
    int64_t nb = k / blk;
    #pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r) {
        for (int64_t j = 0; j < k; ++j) {
            uint8_t byte = packed[r * (k / 2) + j / 2];
            uint8_t nib = (j & 1) ? (byte >> 4) : (byte & 0xf);
            float mag = kE2M1[nib & 7];
            uint8_t c = scales[r * nb + j / blk];
            float v;
            if (fmt == AVE_FMT_NVFP4) v = (mag * ave_oracle_e4m3_decode(c)) * gs;
            else v = mag * ave_oracle_e8m0_decode(c);
            out[r * k + j] = (nib & 8) ? -v : v;
        }
    }
}

/*
 * D32 = A * B^T for fp32 A (m,k), B (n,k), K contiguous.  Products are summed in
 * fp64 and rounded once to fp32, so the result is the correctly rounded value of
 * the reference's fp32 matmul expression up to fp64 accumulation error.
 * d32 (m,n) fp32 and/or dbf16 (m,n) bf16 (RN-even of d32) may be NULL.
 */
void ave_oracle_gemm_f32(const float *a, const float *b, int64_t m, int64_t n, int64_t k,
                         float *d32, uint16_t *dbf16) {
    enum { TM = 8, TN = 8 };
    #pragma omp parallel for collapse(2) schedule(static)
    for (int64_t i0 = 0; i0 < m; i0 += TM) {
        for (int64_t j0 = 0; j0 < n; j0 += TN) {
            double acc[TM][TN];
            memset(acc, 0, sizeof(acc));
            int64_t im = (m - i0 < TM) ? m - i0 : TM;
            int64_t jn = (n - j0 < TN) ? n - j0 : TN;
            for (int64_t kk = 0; kk < k; ++kk) {
                for (int64_t i = 0; i < im; ++i) {
                    double av = (double)a[(i0 + i) * k + kk];
                    for (int64_t j = 0; j < jn; ++j)
                        acc[i][j] += av * (double)b[(j0 + j) * k + kk];
                }
            }
            for (int64_t i = 0; i < im; ++i)
                for (int64_t j = 0; j < jn; ++j) {
                    float v = (float)acc[i][j];
                    if (d32) d32[(i0 + i) * n + j0 + j] = v;
                    if (dbf16) dbf16[(i0 + i) * n + j0 + j] = ave_oracle_f32_to_bf16(v);
                }
        }
    }
}

/*
 * The whole oracle path on already-quantised operands:
 * dequantise A (m,k) and B (n,k), D = bf16_rn(Ahat * Bhat^T).
 * Returns 0, or -1 when the temporaries cannot be allocated.
 */
int ave_oracle_gemm_fp4(const uint8_t *a_packed, const uint8_t *a_scales, float a_gs,
                        const uint8_t *b_packed, const uint8_t *b_scales, float b_gs,
                        int fmt, int64_t m, int64_t n, int64_t k,
                        float *d32, uint16_t *dbf16) {
    float *ah = (float *)malloc(sizeof(float) * (size_t)m * (size_t)k);
    float *bh = (float *)malloc(sizeof(float) * (size_t)n * (size_t)k);
    if (!ah || !bh) { free(ah); free(bh); return -1; }
    ave_oracle_dequantize(a_packed, a_scales, a_gs, fmt, m, k, ah);
    ave_oracle_dequantize(b_packed, b_scales, b_gs, fmt, n, k, bh);
    ave_oracle_gemm_f32(ah, bh, m, n, k, d32, dbf16);
    free(ah);
    free(bh);
    return 0;
}

/* Row-major (R, K/blk) scale bytes -> the 128x4 tiled layout the tensor core
 * path consumes: rows padded to 128, scale columns padded to 4, padding zero;
 * tile (rb, cb) of 512 bytes at ((rb * ceil(ncol/4)) + cb) * 512; inside a tile
 * scale (r, c) is at (r % 32) * 16 + (r / 32) * 4 + c. */
void ave_oracle_sf_to_tiled(const uint8_t *rowmajor, int64_t rows, int64_t ncol, uint8_t *tiled) {
    int64_t rb_n = (rows + 127) / 128, cb_n = (ncol + 3) / 4;
    memset(tiled, 0, (size_t)(rb_n * cb_n * 512));
    for (int64_t r = 0; r < rows; ++r)
        for (int64_t c = 0; c < ncol; ++c) {
            int64_t tile = (r / 128) * cb_n + c / 4;
            int64_t rr = r % 128;
            tiled[tile * 512 + (rr % 32) * 16 + (rr / 32) * 4 + (c % 4)] = rowmajor[r * ncol + c];
        }
}

/* Sets the OpenMP thread count of the loops above (launchers such as torch.distributed.run export
 * OMP_NUM_THREADS=1 to their workers; a CPU timing leg states its thread count explicitly instead). */
void ave_oracle_set_num_threads(int n) {
#ifdef _OPENMP
    extern void omp_set_num_threads(int);
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

int ave_oracle_num_threads(void) {
#ifdef _OPENMP
    extern int omp_get_max_threads(void);
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/*
 * Fused-epilogue restatement: y = act(d + bias[col]) on the fp32 GEMM result d (m, n), which already
 * carries the tensor scales, evaluated in double and rounded to fp32, then to bf16 (RN-even) like the
 * reference's oracle expression `.to(dtype=torch.bfloat16)` (test/examples/gemm/amdgpu/test_amdgpu_gemm.py:27).
 * The reference has no epilogue; activation codes are those of include/ave_fp4.h
 * (0 none, 1 relu, 2 gelu-erf, 3 gelu-tanh, 4 silu).  bias_bf16 may be NULL.
 */
void ave_oracle_bias_act(const float *d32, int64_t m, int64_t n, const uint16_t *bias_bf16, int act,
                         float *y32, uint16_t *ybf16) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < m; ++i) {
        for (int64_t j = 0; j < n; ++j) {
            double x = (double)d32[i * n + j];
            if (bias_bf16) x += (double)bits_to_f32((uint32_t)bias_bf16[j] << 16);
            double y;
            switch (act) {
                case 1: y = x > 0.0 ? x : 0.0; break;
                case 2: y = 0.5 * x * (1.0 + erf(x * 0.70710678118654752440)); break;
                case 3: y = 0.5 * x * (1.0 + tanh(0.79788456080286535588 * (x + 0.044715 * x * x * x))); break;
                case 4: y = x / (1.0 + exp(-x)); break;
                default: y = x; break;
            }
            const float yf = (float)y;
            if (y32) y32[i * n + j] = yf;
            if (ybf16) ybf16[i * n + j] = ave_oracle_f32_to_bf16(yf);
        }
    }
}
