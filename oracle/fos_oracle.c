/*
 * CPU oracle for the Four-Over-Six NVFP4 / IF4 quantize -> dequantize -> matmul path.
 *
 * THIS FILE IS TEST INFRASTRUCTURE. It is a plain-C restatement of the reference
 * project's eager PyTorch implementation and exists only so that the tests, the
 * smoke check and the benchmark's CPU-baseline leg have something to compare the
 * CUDA kernels with. Nothing in the shipped package may call it.
 *
 * Parity status: PINNED. tests/test_oracle_golden.py compares every function here,
 * byte for byte, with vectors produced by the reference's own PyTorch backend
 * (tests/golden/make_golden.py imports the reference and writes the fixtures).
 *
 * Every arithmetic step is IEEE binary32 with one rounding per operation; build
 * with -ffp-contract=off so the compiler never fuses a multiply with an add.
 *
 * Reference locations restated here (paths inside the reference project):
 *   src/fouroversix/quantize/pytorch/reference.py:30-51    e2m1 rounding
 *   src/fouroversix/quantize/pytorch/reference.py:54-63    int4 rounding
 *   src/fouroversix/quantize/pytorch/reference.py:82-132   nibble codes + packing
 *   src/fouroversix/quantize/pytorch/reference.py:184-241  block scale factors
 *   src/fouroversix/quantize/pytorch/reference.py:262-325  4-versus-6 selection
 *   src/fouroversix/quantize/pytorch/reference.py:328-425  int-versus-float selection (IF4)
 *   src/fouroversix/quantize/pytorch/reference.py:555-679  driver (transpose, 2-D blocks, amax)
 *   src/fouroversix/quantize/pytorch/backend.py:57-79      zero padding to 128 x 64
 *   src/fouroversix/quantize/utils.py:88-96                128x4 scale-factor tile order
 *   src/fouroversix/quantize/backend.py:88-160             dequantize
 *   src/fouroversix/quantize/dequantize_utils.py:4-86      unpacking helpers
 *   src/fouroversix/matmul/pytorch.py:33-52                fp32 matmul of dequantized operands
 *   src/fouroversix/matmul/cutlass/backend.py:85-98        GEMM alpha
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

enum { FOS_FMT_NVFP4 = 0, FOS_FMT_IF4 = 1, FOS_FMT_MXFP4 = 2 };
/* Same numbering as ScaleRule.cuda_id, src/fouroversix/utils.py:271-280. */
enum { RULE_STATIC_6 = 0, RULE_STATIC_4 = 1, RULE_MAE = 2, RULE_MSE = 3, RULE_ABS_MAX = 4 };
enum { OUT_BF16 = 0, OUT_FP16 = 1, OUT_FP32 = 2 };

/* ------------------------------------------------------------------ scalar formats */

static inline float u32_as_f32(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }
static inline uint32_t f32_as_u32(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }

static inline float bf16_bits_to_f32(uint16_t h) { return u32_as_f32((uint32_t)h << 16); }

static inline uint16_t f32_to_bf16_bits(float f) {
    uint32_t u = f32_as_u32(f);
    if ((u & 0x7fffffffu) > 0x7f800000u) return 0x7fc0;
    u += 0x7fffu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}

static inline float f16_bits_to_f32(uint16_t h) { _Float16 v; memcpy(&v, &h, 2); return (float)v; }
static inline uint16_t f32_to_f16_bits(float f) { _Float16 v = (_Float16)f; uint16_t h; memcpy(&h, &v, 2); return h; }
/* Round a binary32 value to binary16 and come back, i.e. "the value as fp16". */
static inline float round_to_f16(float f) { return (float)(_Float16)f; }

/* float8_e4m3fn <- binary32, round to nearest even, the way a tensor cast does it:
 * 4 exponent bits (bias 7), 3 mantissa bits, no infinities, 0x7f/0xff are NaN,
 * largest finite 448, smallest subnormal 2^-9. Anything that would round past 448
 * becomes NaN. */
static uint8_t f32_to_e4m3(float f) {
    uint32_t u = f32_as_u32(f);
    uint8_t sign = (uint8_t)((u >> 24) & 0x80u);
    u &= 0x7fffffffu;
    uint8_t out;
    if (u >= 0x43f00000u) {              /* |f| >= 480, inf or NaN */
        out = 0x7f;
    } else if (u < 0x3c800000u) {        /* |f| < 2^-6: subnormal result, step 2^-9 */
        float a = u32_as_f32(u);
        /* adding 2^14 * 2^-9 * ... : use the classic "magic add" at the subnormal step */
        float magic = u32_as_f32(0x46800000u); /* 16384 = 2^14; ulp there is 2^-9 */
        float t = a + magic;                 /* rounds a to a multiple of 2^-9 (RNE) */
        out = (uint8_t)(f32_as_u32(t) - 0x46800000u);
    } else {
        uint32_t odd = (u >> 20) & 1u;
        u += ((uint32_t)(7 - 127) << 23) + 0x7ffffu;
        u += odd;
        out = (uint8_t)(u >> 20);
    }
    return out | sign;
}

static float e4m3_to_f32(uint8_t b) {
    uint32_t e = (b >> 3) & 0xfu, m = b & 7u;
    float v;
    if (e == 0) v = ldexpf((float)m, -9);
    else if (e == 15 && m == 7) v = NAN;
    else v = ldexpf((float)(8 + m), (int)e - 10);
    return (b & 0x80u) ? -v : v;
}

/* ------------------------------------------------------------------ value grids */

static inline float round_half_even(float a) { return nearbyintf(a); }

/* Three-piece rounding onto {0, .5, 1, 1.5, 2, 3, 4, 6}; no clamp, like the reference. */
static inline float fake_e2m1(float xs) {
    float a = fabsf(xs);
    float v;
    if (a < 2.0f) v = round_half_even(2.0f * a) / 2.0f;
    else if (a < 4.0f) v = round_half_even(a);
    else v = 2.0f * round_half_even(a / 2.0f);
    float s = (xs > 0.0f) ? 1.0f : ((xs < 0.0f) ? -1.0f : 0.0f);
    return s * v;                        /* -1 * 0 = -0.0, 0 * v = +0.0 */
}

static inline float fake_int4(float xs) {
    float c = xs < -7.0f ? -7.0f : (xs > 7.0f ? 7.0f : xs);
    return round_half_even(c);
}

/* The reference reads the nibble out of the bf16 bit pattern of the rounded value. */
static inline uint8_t e2m1_code_from_value(float v) {
    uint16_t b = f32_to_bf16_bits(v);
    int s = (b >> 15) & 1, e = (b >> 7) & 0xff, m = b & 0x7f;
    int is_zero = (e == 0) && (m == 0);
    m = (m >> 6) & 1;
    if (e == 126 && m == 0) m = 1;       /* 0.5 is the subnormal with the mantissa bit set */
    e = e - 126;
    if (is_zero) { e = 0; m = 0; }
    return (uint8_t)(((s << 3) | (e << 1) | m) & 0xff);
}

static inline uint8_t int4_code_from_value(float v) {
    float b = bf16_bits_to_f32(f32_to_bf16_bits(v));
    float c = b < -7.0f ? -7.0f : (b > 7.0f ? 7.0f : b);
    return (uint8_t)((int8_t)c) & 0xf;
}

static const float E2M1_VALUE[8] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f};

/* ------------------------------------------------------------------ reductions */

/* Order in which an eager fp32 sum over a last axis of 16 adds its terms:
 * eight lane partials e[k] + e[k+8], then left to right over the lanes. */
static float sum16(const float *e) {
    float p[8];
    for (int k = 0; k < 8; ++k) p[k] = e[k] + e[k + 8];
    float r = p[0];
    for (int k = 1; k < 8; ++k) r = r + p[k];
    return r;
}

/* Same for a last axis of 256: the row is 32 vectors of 8 lanes; four interleaved
 * accumulators each take every fourth vector, are combined ((A0+A1)+A2)+A3 lane by
 * lane, and the eight lanes are then added left to right. */
static float sum256(const float *e) {
    float acc[4][8];
    for (int j = 0; j < 4; ++j)
        for (int k = 0; k < 8; ++k) {
            float a = e[j * 8 + k];
            for (int m = 1; m < 8; ++m) a = a + e[(4 * m + j) * 8 + k];
            acc[j][k] = a;
        }
    float lane[8];
    for (int k = 0; k < 8; ++k) lane[k] = ((acc[0][k] + acc[1][k]) + acc[2][k]) + acc[3][k];
    float r = lane[0];
    for (int k = 1; k < 8; ++k) r = r + lane[k];
    return r;
}

static float block_error(const float *deq, const float *x, int n, int rule) {
    float e[256];
    if (rule == RULE_ABS_MAX) {
        float m = 0.0f;
        for (int i = 0; i < n; ++i) { float d = fabsf(deq[i] - x[i]); if (d > m) m = d; }
        return m;
    }
    for (int i = 0; i < n; ++i) {
        float d = deq[i] - x[i];
        e[i] = (rule == RULE_MAE) ? fabsf(d) : d * d;
    }
    return n == 16 ? sum16(e) : sum256(e);
}

/* ------------------------------------------------------------------ one block */

/* Scale factor of one block and the block's values divided by it. */
static uint8_t block_scale(const float *x, int n, float amax, float maxq, float maxsf,
                           int expand, float *xs) {
    float bmax = 0.0f;
    for (int i = 0; i < n; ++i) { float a = fabsf(x[i]); if (a > bmax) bmax = a; }
    float hp;
    if (amax == 0.0f) hp = 0.0f;
    else {
        float encode = (maxq * maxsf) / amax;
        hp = (bmax / maxq) * encode;
    }
    if (expand) hp = hp * 1.5f;
    uint8_t sf = f32_to_e4m3(hp);
    float sff = e4m3_to_f32(sf);
    float decode = 1.0f / ((maxq * maxsf) / amax);
    if (sff != 0.0f) {
        float r = 1.0f / (decode * sff);
        for (int i = 0; i < n; ++i) xs[i] = x[i] * r;
    } else {
        for (int i = 0; i < n; ++i) xs[i] = 0.0f;
    }
    return sf;
}

/* Quantize one block of n (16 or 256) values. codes[] receives one nibble per value,
 * *sf the scale byte (sign bit = "int block" for IF4), *choice 1 when the alternative
 * (scale-to-4, or int) won. Returns the largest |scaled value| over every candidate tried. */
static float quantize_block(const float *x, int n, float amax, int format, int rule,
                            uint8_t *codes, uint8_t *sf_out, uint8_t *choice) {
    float xs_a[256], xs_b[256], fq_a[256], fq_b[256], dq[256];
    float worst = 0.0f;
    if (format == FOS_FMT_NVFP4 && (rule == RULE_STATIC_6 || rule == RULE_STATIC_4)) {
        float maxq = rule == RULE_STATIC_4 ? 4.0f : 6.0f;
        uint8_t sf = block_scale(x, n, amax, maxq, 448.0f, 0, xs_a);
        for (int i = 0; i < n; ++i) {
            codes[i] = e2m1_code_from_value(fake_e2m1(xs_a[i]));
            if (fabsf(xs_a[i]) > worst) worst = fabsf(xs_a[i]);
        }
        *sf_out = sf; *choice = 0;
        return worst;
    }
    if (format == FOS_FMT_NVFP4) {
        /* candidate "6" and candidate "4" (the same scale times 1.5), E4M3 ceiling 256 */
        uint8_t sf6 = block_scale(x, n, amax, 6.0f, 256.0f, 0, xs_a);
        uint8_t sf4 = block_scale(x, n, amax, 6.0f, 256.0f, 1, xs_b);
        float s6 = e4m3_to_f32(sf6), s4 = e4m3_to_f32(sf4);
        for (int i = 0; i < n; ++i) { fq_a[i] = fake_e2m1(xs_a[i]); fq_b[i] = fake_e2m1(xs_b[i]); }
        for (int i = 0; i < n; ++i) dq[i] = ((fq_b[i] * s4) * amax) / 1536.0f;
        float err4 = block_error(dq, x, n, rule);
        for (int i = 0; i < n; ++i) dq[i] = ((fq_a[i] * s6) * amax) / 1536.0f;
        float err6 = block_error(dq, x, n, rule);
        int pick4 = err4 < err6;
        const float *fq = pick4 ? fq_b : fq_a;
        for (int i = 0; i < n; ++i) {
            codes[i] = e2m1_code_from_value(fq[i]);
            if (fabsf(xs_a[i]) > worst) worst = fabsf(xs_a[i]);
            if (fabsf(xs_b[i]) > worst) worst = fabsf(xs_b[i]);
        }
        *sf_out = pick4 ? sf4 : sf6; *choice = (uint8_t)pick4;
        return worst;
    }
    /* IF4: one scale (6-rule, ceiling 448); float grid versus integer grid times 6/7 */
    uint8_t sf = block_scale(x, n, amax, 6.0f, 448.0f, 0, xs_a);
    float s = e4m3_to_f32(sf);
    const float to_int = (float)1.16666666, from_int = (float)0.8571428571;
    for (int i = 0; i < n; ++i) {
        fq_a[i] = fake_e2m1(xs_a[i]);
        fq_b[i] = fake_int4(xs_a[i] * to_int);
        if (fabsf(xs_a[i]) > worst) worst = fabsf(xs_a[i]);
    }
    for (int i = 0; i < n; ++i) dq[i] = ((fq_a[i] * s) * amax) / 2688.0f;
    float err_fp = block_error(dq, x, n, rule);
    for (int i = 0; i < n; ++i) dq[i] = (((fq_b[i] * s) * amax) * from_int) / 2688.0f;
    float err_int = block_error(dq, x, n, rule);
    int pick_int = err_int < err_fp;
    for (int i = 0; i < n; ++i)
        codes[i] = pick_int ? int4_code_from_value(fq_b[i]) : e2m1_code_from_value(fq_a[i]);
    *sf_out = (uint8_t)(sf + (pick_int ? 128 : 0)); *choice = (uint8_t)pick_int;
    return worst;
}

/* MXFP4 (src/fouroversix/quantize/pytorch/reference.py:149-181): one block of n (32 or 32 x 32)
 * values, scale = the power of two at or above max|x| / maxq stored as its biased exponent
 * (E8M0), values divided by it and rounded to E2M1. No per-tensor scale. */
static float quantize_block_mx(const float *x, int n, int rule, uint8_t *codes, uint8_t *sf_out) {
    float bmax = 0.0f, worst = 0.0f;
    for (int i = 0; i < n; ++i) { float a = fabsf(x[i]); if (a > bmax) bmax = a; }
    const float hp = bmax / (rule == RULE_STATIC_4 ? 4.0f : 6.0f);
    const uint32_t bits = f32_as_u32(hp);
    uint8_t e = (uint8_t)((bits >> 23) & 0xff);
    if (bits & 0x7fffff) e = (uint8_t)(e + 1);            /* round up; uint8 arithmetic as in the reference */
    const float scale = u32_as_f32((uint32_t)e << 23);
    for (int i = 0; i < n; ++i) {
        float xs = e != 0 ? x[i] / scale : 0.0f;
        if (fabsf(xs) > worst) worst = fabsf(xs);
        codes[i] = e2m1_code_from_value(fake_e2m1(xs));
    }
    *sf_out = e;
    return worst;
}

/* ------------------------------------------------------------------ layouts */

static inline int64_t round_up(int64_t v, int64_t m) { return (v + m - 1) / m * m; }

/* Offset of the scale of (row r, block column cb) in the 128x4-tile order. */
static inline int64_t sf_tiled_offset(int64_t r, int64_t cb, int64_t n_cb) {
    int64_t tile = (r / 128) * (n_cb / 4) + cb / 4;
    return tile * 512 + (r % 32) * 16 + ((r % 128) / 32) * 4 + (cb % 4);
}

/* ------------------------------------------------------------------ exported: quantize */

/*
 * x: R x C values (bf16 bits, or fp16 bits when x_is_fp16), row stride ld elements.
 * The output describes Y = x (or x^T when transpose) zero padded to Rp x Cp with
 * Rp a multiple of 128 and Cp a multiple of 64:
 *   codes   Rp x Cp/2 bytes, low nibble = even column
 *   sf      Rp*Cp/16 bytes, tiled (sf_tiled != 0) or row-major Rp x Cp/16
 *   amax_out one float: max |x| (or *amax_in when given)
 *   choice  optional Rp*Cp/16 bytes row-major: 1 where the alternative candidate won
 *   worst_scaled optional: max |x / scale| over all candidates (must stay < 7 for the
 *                reference's unclamped rounding and the hardware's saturating one to agree)
 */
int fos_oracle_quantize(const uint16_t *x, int x_is_fp16, int64_t R, int64_t C, int64_t ld,
                        int format, int rule, int block_2d, int transpose, int sf_tiled,
                        const float *amax_in, uint8_t *codes, uint8_t *sf, float *amax_out,
                        uint8_t *choice, float *worst_scaled) {
    if (format != FOS_FMT_NVFP4 && format != FOS_FMT_IF4 && format != FOS_FMT_MXFP4) return -1;
    if (rule < 0 || rule > 4) return -1;
    if (format == FOS_FMT_IF4 && (rule == RULE_STATIC_6 || rule == RULE_STATIC_4)) return -1;
    if (format == FOS_FMT_MXFP4 && rule != RULE_STATIC_6 && rule != RULE_STATIC_4) return -1;
    const int mx = format == FOS_FMT_MXFP4;
    const int bw = mx ? 32 : 16;                    /* block width; four blocks per scale tile column group */
    const int64_t Ro = transpose ? C : R, Co = transpose ? R : C;
    const int64_t Rp = round_up(Ro, 128), Cp = round_up(Co, 4 * bw), ncb = Cp / bw;

    float amax = 0.0f;
    if (mx) amax = 1.0f;                            /* reference.py:573-578: ones for MXFP4 */
    else if (amax_in) amax = *amax_in;
    else {
        #pragma omp parallel for reduction(max : amax) schedule(static)
        for (int64_t i = 0; i < R; ++i)
            for (int64_t j = 0; j < C; ++j) {
                uint16_t h = x[i * ld + j];
                float a = fabsf(x_is_fp16 ? f16_bits_to_f32(h) : bf16_bits_to_f32(h));
                if (a > amax) amax = a;
            }
    }
    *amax_out = amax;

    float worst_all = 0.0f;
    const int bh = block_2d ? bw : 1;               /* block height in rows of Y */
    #pragma omp parallel for reduction(max : worst_all) schedule(static)
    for (int64_t r0 = 0; r0 < Rp; r0 += bh) {
        float v[1024];
        uint8_t cd[1024];
        for (int64_t cb = 0; cb < ncb; ++cb) {
            for (int dr = 0; dr < bh; ++dr)
                for (int dc = 0; dc < bw; ++dc) {
                    int64_t i = r0 + dr, j = cb * bw + dc;
                    float f = 0.0f;
                    if (i < Ro && j < Co) {
                        uint16_t h = transpose ? x[j * ld + i] : x[i * ld + j];
                        f = x_is_fp16 ? f16_bits_to_f32(h) : bf16_bits_to_f32(h);
                    }
                    v[dr * bw + dc] = f;
                }
            uint8_t sfb, ch = 0;
            float w = mx ? quantize_block_mx(v, bh * bw, rule, cd, &sfb)
                         : quantize_block(v, bh * bw, amax, format, rule, cd, &sfb, &ch);
            if (w > worst_all) worst_all = w;
            for (int dr = 0; dr < bh; ++dr) {
                int64_t i = r0 + dr;
                uint8_t *dst = codes + i * (Cp / 2) + cb * (bw / 2);
                for (int p = 0; p < bw / 2; ++p)
                    dst[p] = (uint8_t)((cd[dr * bw + 2 * p + 1] << 4) | (cd[dr * bw + 2 * p] & 0xf));
                int64_t off = sf_tiled ? sf_tiled_offset(i, cb, ncb) : i * ncb + cb;
                sf[off] = sfb;
                if (choice) choice[i * ncb + cb] = ch;
            }
        }
    }
    if (worst_scaled) *worst_scaled = worst_all;
    return 0;
}

/* ------------------------------------------------------------------ exported: dequantize */

static inline float dequant_divisor(int format, int rule) {
    if (format == FOS_FMT_IF4) return 2688.0f;              /* 6 * 448 */
    if (rule == RULE_STATIC_6) return 2688.0f;
    if (rule == RULE_STATIC_4) return 1792.0f;              /* 4 * 448 */
    return 1536.0f;                                         /* 6 * 256 */
}

/* One dequantized element as binary32, before the cast to the output type:
 * fp16(value) * fp16(scale) in fp16, then (fp32 * amax) / divisor. */
static inline float dequant_one(uint8_t nib, uint8_t sfb, int format, float amax, float div) {
    float v16, s16;
    if (format == FOS_FMT_IF4) {
        s16 = round_to_f16(e4m3_to_f32(sfb & 0x7f));
        if (sfb & 0x80) {
            int iv = (int)(int8_t)(uint8_t)(nib << 4) >> 4;
            v16 = round_to_f16((float)iv * (float)(6.0 / 7.0));
        } else {
            float m = E2M1_VALUE[nib & 7];
            v16 = (nib & 8) ? -m : m;
        }
    } else {
        s16 = round_to_f16(e4m3_to_f32(sfb));
        float m = E2M1_VALUE[nib & 7];
        v16 = (nib & 8) ? -m : m;
    }
    float r16 = round_to_f16(v16 * s16);
    return (r16 * amax) / div;
}

static inline void store_out(void *out, int64_t idx, int out_type, float v) {
    if (out_type == OUT_FP32) ((float *)out)[idx] = v;
    else if (out_type == OUT_FP16) ((uint16_t *)out)[idx] = f32_to_f16_bits(v);
    else ((uint16_t *)out)[idx] = f32_to_bf16_bits(v);
}

/* codes Rp x Cp/2, sf as written by fos_oracle_quantize; out is R x C (cropped), row-major. */
int fos_oracle_dequantize(const uint8_t *codes, const uint8_t *sf, const float *amax_p,
                          int format, int rule, int sf_tiled, int64_t Rp, int64_t Cp,
                          int64_t R, int64_t C, int out_type, void *out) {
    if (format == FOS_FMT_MXFP4) {
        /* quantize/backend.py:88-160: fp16(value) * fp16(2^(e-127)) in fp16, nothing else (the
         * E8M0 -> fp16 conversion overflows to inf above 2^15 and flushes below 2^-24) */
        const int64_t nb = Cp / 32;
        #pragma omp parallel for schedule(static)
        for (int64_t i = 0; i < R; ++i)
            for (int64_t j = 0; j < C; ++j) {
                uint8_t byte = codes[i * (Cp / 2) + j / 2];
                uint8_t nib = (j & 1) ? (byte >> 4) : (byte & 0xf);
                uint8_t e = sf[sf_tiled ? sf_tiled_offset(i, j / 32, nb) : i * nb + j / 32];
                float s16 = e == 255 ? NAN : round_to_f16(e == 0 ? 0x1p-127f : u32_as_f32((uint32_t)e << 23));
                float m = E2M1_VALUE[nib & 7];
                store_out(out, i * C + j, out_type, round_to_f16(((nib & 8) ? -m : m) * s16));
            }
        return 0;
    }
    const float amax = *amax_p, div = dequant_divisor(format, rule);
    const int64_t ncb = Cp / 16;
    #pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < R; ++i)
        for (int64_t j = 0; j < C; ++j) {
            uint8_t byte = codes[i * (Cp / 2) + j / 2];
            uint8_t nib = (j & 1) ? (byte >> 4) : (byte & 0xf);
            int64_t off = sf_tiled ? sf_tiled_offset(i, j / 16, ncb) : i * ncb + j / 16;
            store_out(out, i * C + j, out_type, dequant_one(nib, sf[off], format, amax, div));
        }
    return 0;
}

/* ------------------------------------------------------------------ exported: matmul */

/* alpha = amaxA * amaxB / (divisorA * divisorB), one rounding per operation. */
float fos_oracle_alpha(float amax_a, int format_a, int rule_a, float amax_b, int format_b, int rule_b) {
    if (format_a == FOS_FMT_MXFP4 && format_b == FOS_FMT_MXFP4) return 1.0f;   /* matmul/cutlass/backend.py:79-84 */
    float num = amax_a * amax_b;
    /* the reference multiplies the four integer constants in Python before dividing */
    double den = (double)dequant_divisor(format_a, rule_a) * (double)dequant_divisor(format_b, rule_b);
    return num / (float)den;
}

/* out[M x N] = deq32(A)[M x K] * deq32(B)[N x K]^T with fp32 accumulation, cast to out_type.
 * A and B are given as packed tensors (padded shapes Mp x Kp and Np x Kp). */
int fos_oracle_matmul(const uint8_t *a_codes, const uint8_t *a_sf, const float *a_amax,
                      int a_format, int a_rule, int a_tiled, int64_t Mp,
                      const uint8_t *b_codes, const uint8_t *b_sf, const float *b_amax,
                      int b_format, int b_rule, int b_tiled, int64_t Np,
                      int64_t Kp, int64_t M, int64_t N, int64_t K, int out_type, void *out) {
    float *A = (float *)malloc((size_t)M * K * sizeof(float));
    float *B = (float *)malloc((size_t)N * K * sizeof(float));
    if (!A || !B) { free(A); free(B); return -2; }
    (void)Mp; (void)Np;
    fos_oracle_dequantize(a_codes, a_sf, a_amax, a_format, a_rule, a_tiled, Mp, Kp, M, K, OUT_FP32, A);
    fos_oracle_dequantize(b_codes, b_sf, b_amax, b_format, b_rule, b_tiled, Np, Kp, N, K, OUT_FP32, B);
    enum { TI = 8, TJ = 8 };
    #pragma omp parallel for schedule(dynamic, 1)
    for (int64_t i0 = 0; i0 < M; i0 += TI)
        for (int64_t j0 = 0; j0 < N; j0 += TJ) {
            float acc[TI][TJ];
            memset(acc, 0, sizeof acc);
            int64_t ni = M - i0 < TI ? M - i0 : TI, nj = N - j0 < TJ ? N - j0 : TJ;
            for (int64_t i = 0; i < ni; ++i)
                for (int64_t j = 0; j < nj; ++j) {
                    const float *pa = A + (i0 + i) * K, *pb = B + (j0 + j) * K;
                    float lanes[16] = {0};
                    int64_t k = 0;
                    for (; k + 16 <= K; k += 16)
                        for (int l = 0; l < 16; ++l) lanes[l] += pa[k + l] * pb[k + l];
                    float s = 0.0f;
                    for (int l = 0; l < 16; ++l) s += lanes[l];
                    for (; k < K; ++k) s += pa[k] * pb[k];
                    acc[i][j] = s;
                }
            for (int64_t i = 0; i < ni; ++i)
                for (int64_t j = 0; j < nj; ++j)
                    store_out(out, (i0 + i) * N + (j0 + j), out_type, acc[i][j]);
        }
    free(A); free(B);
    return 0;
}

/* The CUDA kernels divide a block maximum by 6 with one multiply and two fused multiply-adds
 * instead of an IEEE division. A block maximum is always a bf16 or fp16 value, so the
 * shortcut can be checked against a true division for every possible input. Returns the
 * number of inputs for which the two differ (expected: 0). */
long fos_oracle_check_div6(void) {
    long bad = 0;
    const float y = 1.0f / 6.0f;
    for (int fmt = 0; fmt < 2; ++fmt)
        for (uint32_t h = 0; h < 0x8000u; ++h) {
            float a = fmt == 0 ? bf16_bits_to_f32((uint16_t)h) : f16_bits_to_f32((uint16_t)h);
            if (!isfinite(a)) continue;
            float q0 = a * y;
            float q1 = fmaf(fmaf(-6.0f, q0, a), y, q0);
            if (q1 != a / 6.0f) ++bad;
            if (a * 0.25f != a / 4.0f) ++bad;
        }
    return bad;
}

/* The 16-point random Hadamard transform the reference applies before quantizing when
 * QuantizationConfig.rht is set (src/fouroversix/quantize/pytorch/reference.py:568-570 with the
 * matrix of src/fouroversix/quantize/utils.py:19-85): y = x_block @ (diag(signs) @ H16 / 4), computed
 * per block of 16 along the last axis of x (of x^T when `transpose`), in binary32, rounded once to
 * x's type. The sum is evaluated as a fast Walsh-Hadamard transform (four stages of 16 additions
 * and subtractions); against the reference's matrix product the result is identical unless the
 * 16 values span more than about ten binades, where single last-place differences occur in a few
 * values per million. `out` is the rotated tensor, [R][C] or, when `transpose`, [C][R], contiguous.
 * Returns -1 when the rotated axis is not a multiple of 16. */
int fos_oracle_rht(const uint16_t *x, int x_is_fp16, int64_t R, int64_t C, int64_t ld, int transpose,
                   uint16_t *out) {
    static const float signs[16] = {1, 1, 1, -1, 1, -1, -1, -1, -1, -1, -1, 1, -1, 1, -1, -1};
    const int64_t Ro = transpose ? C : R, Co = transpose ? R : C;
    if (Co % 16 != 0) return -1;
#ifdef _OPENMP
#pragma omp parallel for schedule(static)
#endif
    for (int64_t r = 0; r < Ro; ++r) {
        for (int64_t c0 = 0; c0 < Co; c0 += 16) {
            float v[16];
            for (int i = 0; i < 16; ++i) {
                const uint16_t h = transpose ? x[(c0 + i) * ld + r] : x[r * ld + c0 + i];
                v[i] = signs[i] * (x_is_fp16 ? f16_bits_to_f32(h) : bf16_bits_to_f32(h));
            }
            for (int h = 1; h < 16; h *= 2) {
                for (int base = 0; base < 16; base += 2 * h) {
                    for (int k = 0; k < h; ++k) {
                        const float a = v[base + k], b = v[base + h + k];
                        v[base + k] = a + b;
                        v[base + h + k] = a - b;
                    }
                }
            }
            for (int i = 0; i < 16; ++i) {
                const float y = v[i] * 0.25f;
                out[r * Co + c0 + i] = x_is_fp16 ? f32_to_f16_bits(y) : f32_to_bf16_bits(y);
            }
        }
    }
    return 0;
}

/* How many finite binary32 a with |a| >= min_abs (bit patterns start, start + stride, ...) have
 * fma(fma(-d, a * y, a), y, a * y) != a / d, y = fl(1 / d), ignoring the sign of a zero: the
 * division-free quotient of the dequantize kernel. stride 1 is the exhaustive check. */
int64_t fos_oracle_check_div_const(float d, uint32_t start, uint32_t stride, float min_abs) {
    const float y = 1.0f / d;
    int64_t bad = 0;
    if (stride == 0) stride = 1;
    const int64_t n = ((1LL << 32) - start + stride - 1) / stride;
#ifdef _OPENMP
#pragma omp parallel for reduction(+ : bad) schedule(static)
#endif
    for (int64_t i = 0; i < n; ++i) {
        const uint32_t bits = (uint32_t)(start + i * stride);
        float a;
        memcpy(&a, &bits, 4);
        if (!isfinite(a) || fabsf(a) < min_abs) continue;
        const float q0 = a * y;
        const float q1 = fmaf(fmaf(-d, q0, a), y, q0);
        const float ref = a / d;
        if (q1 != ref && !(q1 == 0.0f && ref == 0.0f)) ++bad;
    }
    return bad;
}

int fos_oracle_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* Threads for the following calls (launchers such as torchrun export OMP_NUM_THREADS=1). */
void fos_oracle_set_num_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}
