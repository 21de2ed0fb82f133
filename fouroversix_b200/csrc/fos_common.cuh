// Shared device helpers for the fouroversix_b200 kernels (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/fouroversix_b200.h"

#if defined(__CUDA_ARCH__) && !(defined(__CUDA_ARCH_FEAT_SM100_ALL) || defined(__CUDA_ARCH_FEAT_SM103_ALL))
#error "fouroversix_b200 kernels must be compiled for sm_100a"
#endif

namespace fos {

// Records a failed runtime call for fos_last_cuda_error() and maps it to FOS_ERR_CUDA.
int note_cuda_error(cudaError_t e);
// FOS_OK when the current device is compute capability 10.x, else FOS_ERR_ARCH / FOS_ERR_CUDA.
int check_device();
// The sticky wait-failure word of each group of kernels on the current device (0: no bounded wait ever gave up).
cudaError_t quantize_wait_failures(int32_t *host_value);
cudaError_t gemm_wait_failures(int32_t *host_value);
cudaError_t gemm_if4_wait_failures(int32_t *host_value);
cudaError_t quantize_wait_roles(uint32_t *host_value);
cudaError_t gemm_wait_roles(uint32_t *host_value);
cudaError_t gemm_if4_wait_roles(uint32_t *host_value);

// MXFP4 branches of fos_quantize / fos_dequantize (fos_mxfp4.cu); arguments validated by the callers.
int quantize_mxfp4(const void *x, int x_dtype, int64_t rows, int64_t cols, int64_t ld, int scale_rule, int block_2d,
                   int transpose, int sf_layout, uint8_t *codes, uint8_t *sf, float *amax_out, cudaStream_t stream);
int dequantize_mxfp4(const uint8_t *codes, const uint8_t *sf, int sf_layout, int64_t rows_p, int64_t cols_p, int64_t rows,
                     int64_t cols, void *out, int out_dtype, int64_t ld_out, cudaStream_t stream);

#define FOS_CUDA_TRY(expr)                                         \
    do {                                                           \
        cudaError_t fos_e_ = (expr);                               \
        if (fos_e_ != cudaSuccess) return fos::note_cuda_error(fos_e_); \
    } while (0)

static inline int64_t round_up64(int64_t v, int64_t m) { return (v + m - 1) / m * m; }

// (max representable value) * (largest scale) used to undo the two-level scaling.
__host__ __device__ inline float dequant_divisor(int format, int rule) {
    if (format == FOS_IF4) return 2688.0f;
    if (rule == FOS_RULE_STATIC_6) return 2688.0f;
    if (rule == FOS_RULE_STATIC_4) return 1792.0f;
    return 1536.0f;
}

#ifdef __CUDACC__

// Offset of the scale of (row r, block column cb) when scales are stored as 128x4 tiles
// of 512 bytes: 32 groups of 16 bytes, group g = r % 32, inside it four quarters of
// 4 bytes (r / 32 within the tile), inside a quarter the four block columns.
__device__ __forceinline__ int64_t sf_offset(int64_t r, int64_t cb, int64_t n_cb, bool tiled) {
    if (!tiled) return r * n_cb + cb;
    int64_t tile = (r >> 7) * (n_cb >> 2) + (cb >> 2);
    return tile * 512 + (r & 31) * 16 + ((r >> 5) & 3) * 4 + (cb & 3);
}

// ---- format conversions (all round-to-nearest-even, saturating) ----

// Two floats -> one byte of two E2M1 codes; `hi` lands in the upper nibble.
__device__ __forceinline__ uint32_t cvt_e2m1x2(float hi, float lo) {
    uint32_t r;
    asm("{ .reg .b8 b; cvt.rn.satfinite.e2m1x2.f32 b, %1, %2; cvt.u32.u8 %0, b; }" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}

// Eight floats (x[0] = lowest nibble) -> 32 bits of E2M1 codes.
__device__ __forceinline__ uint32_t cvt_e2m1x8(const float *x) {
    uint32_t r;
    asm("{ .reg .b8 b0, b1, b2, b3;\n"
        "cvt.rn.satfinite.e2m1x2.f32 b0, %2, %1;\n"
        "cvt.rn.satfinite.e2m1x2.f32 b1, %4, %3;\n"
        "cvt.rn.satfinite.e2m1x2.f32 b2, %6, %5;\n"
        "cvt.rn.satfinite.e2m1x2.f32 b3, %8, %7;\n"
        "mov.b32 %0, {b0, b1, b2, b3}; }"
        : "=r"(r)
        : "f"(x[0]), "f"(x[1]), "f"(x[2]), "f"(x[3]), "f"(x[4]), "f"(x[5]), "f"(x[6]), "f"(x[7]));
    return r;
}

// One byte of two E2M1 codes -> the two values as floats (lo = low nibble).
__device__ __forceinline__ float2 e2m1x2_to_float2(uint32_t byte) {
    uint32_t h2;
    asm("{ .reg .b8 b; cvt.u8.u32 b, %1; cvt.rn.f16x2.e2m1x2 %0, b; }" : "=r"(h2) : "r"(byte));
    return __half22float2(*reinterpret_cast<__half2 *>(&h2));
}

__device__ __forceinline__ uint32_t cvt_e4m3(float x) {
    uint16_t r;
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(0.0f), "f"(x));
    return r & 0xffu;
}

// Two floats -> two E4M3 bytes, `hi` in bits 8..15.
__device__ __forceinline__ uint32_t cvt_e4m3x2(float hi, float lo) {
    uint16_t r;
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(hi), "f"(lo));
    return r;
}

__device__ __forceinline__ float e4m3_to_float(uint32_t byte) {
    uint32_t h2;
    uint16_t b = static_cast<uint16_t>(byte & 0xffu);
    asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h2) : "h"(b));
    return __half2float(__ushort_as_half(static_cast<unsigned short>(h2 & 0xffffu)));
}

// ---- packed binary32 pairs (sm_100: one instruction, two IEEE operations) ----

__device__ __forceinline__ uint64_t pack2(float lo, float hi) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void unpack2f(uint64_t v, float &lo, float &hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
// Element-wise fma.rn on two binary32 lanes; each lane rounds exactly like fmaf().
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t r;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
    return r;
}

// a / 6 correctly rounded for every finite bf16 or fp16 value a (checked exhaustively on the
// host, see tests): quotient estimate, exact remainder, one correction.
__device__ __forceinline__ float div6_exact(float a) {
    const float y = 1.0f / 6.0f;
    const float q0 = __fmul_rn(a, y);
    return __fmaf_rn(__fmaf_rn(-6.0f, q0, a), y, q0);
}

// E2M1 codes of v[i] * r. The reference multiplies the rounded magnitude by sign(x_scaled),
// which is 0 for a zero of either sign, so a scaled value of -0.0 must encode as +0 (code
// 0x0, not 0x8). fma(v, r, +0.0) rounds exactly like v * r and turns (-0.0) * r into +0.0;
// `guard` adds +0.0 once more for a NEGATIVE product that underflows to -0.0.
__device__ __forceinline__ void encode_e2m1(const float (&v)[16], float r, bool guard, uint32_t &lo, uint32_t &hi) {
    float xs[16];
    const uint64_t r2 = pack2(r, r), zero2 = pack2(0.0f, 0.0f);
#pragma unroll
    for (int k = 0; k < 8; ++k) unpack2f(fma2(pack2(v[2 * k], v[2 * k + 1]), r2, zero2), xs[2 * k], xs[2 * k + 1]);
    if (guard) {
#pragma unroll
        for (int i = 0; i < 16; ++i) xs[i] = __fadd_rn(xs[i], 0.0f);
    }
    lo = cvt_e2m1x8(xs);
    hi = cvt_e2m1x8(xs + 8);
}

// ---- NVFP4 with a static scale rule, one block of 16 values ----
//
// The reference's sequence for scale_rule static_6 / static_4 (src/fouroversix/quantize/pytorch/
// reference.py:184-241, 555-679), as the quantize kernels run it: per tensor encode = (maxq * 448) / amax
// and decode = 1 / encode; per block the scale byte E4M3(bmax / maxq * encode) and the codes of
// x * (1 / (decode * scale)). `lut` maps a scale byte to {scale, 1 / (decode * scale)}.
struct StaticQuantConsts {
    float encode0;   // encode, or 0 when amax is 0 (every scale is then 0)
    float decode;
    bool six;        // static_6 (else static_4)
};
__device__ __forceinline__ StaticQuantConsts static_quant_consts(float amax, int rule) {
    StaticQuantConsts c;
    c.six = rule != FOS_RULE_STATIC_4;
    const float encode = __fdiv_rn((c.six ? 6.0f : 4.0f) * 448.0f, amax);
    c.decode = __frcp_rn(encode);
    c.encode0 = amax == 0.0f ? 0.0f : encode;
    return c;
}
__device__ __forceinline__ float2 static_scale_entry(uint32_t sfb, float decode) {
    const float s = e4m3_to_float(sfb);
    return make_float2(s, __frcp_rn(__fmul_rn(decode, s)));
}
__device__ __forceinline__ void quantize_block_static(const float (&v)[16], const StaticQuantConsts &c, const float2 *lut,
                                                      uint32_t &lo, uint32_t &hi, uint32_t &sf_byte) {
    float bmax = 0.0f;
#pragma unroll
    for (int i = 0; i < 16; ++i) bmax = fmaxf(bmax, fabsf(v[i]));
    const float q = c.six ? div6_exact(bmax) : __fmul_rn(bmax, 0.25f);
    sf_byte = cvt_e4m3(__fmul_rn(q, c.encode0));
    const float2 e = lut[sf_byte];
    lo = hi = 0u;
    if (e.x != 0.0f) encode_e2m1(v, e.y, e.y < 0x1p-16f, lo, hi);
}

// ---- memory ----

__device__ __forceinline__ uint4 ldg_nc_16(const void *p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.b32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

// 32-byte load (sm_100 and later); `p` must be 32-byte aligned.
__device__ __forceinline__ void ldg_nc_32(const void *p, uint32_t (&v)[8]) {
    asm volatile("ld.global.nc.L1::no_allocate.v8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7])
                 : "l"(p));
}

// 32-byte store (sm_100 and later); `p` must be 32-byte aligned.
__device__ __forceinline__ void stg_32(void *p, const uint32_t *v) {
    asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
                 ::"l"(p), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]) : "memory");
}

// The same store for data that will not be read again soon (a GEMM's output): marked evict-first in L2, so that
// it does not push the operand tiles, which every CTA of a band re-reads, out of the cache, and not allocated in L1
// (8192^3: 215 -> 212.5 us, 8192 x 4096 x 4096: 61.7 -> 59.6 us; evict-first alone and .cs measured the same as plain).
#ifndef FOS_ST_STREAM_HINT
#define FOS_ST_STREAM_HINT ".L1::no_allocate.L2::evict_first"
#endif
__device__ __forceinline__ void stg_32_stream(void *p, const uint32_t *v) {
    asm volatile("st.global" FOS_ST_STREAM_HINT ".v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
                 ::"l"(p), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]) : "memory");
}

template <typename T> __device__ __forceinline__ float elem_to_float(T v);
template <> __device__ __forceinline__ float elem_to_float<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <> __device__ __forceinline__ float elem_to_float<__half>(__half v) { return __half2float(v); }

// Two packed 16-bit elements -> floats (x = low half).
template <typename T> __device__ __forceinline__ float2 unpack2(uint32_t w);
template <> __device__ __forceinline__ float2 unpack2<__nv_bfloat16>(uint32_t w) {
    return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u));
}
template <> __device__ __forceinline__ float2 unpack2<__half>(uint32_t w) {
    return __half22float2(*reinterpret_cast<__half2 *>(&w));
}

#endif  // __CUDACC__

}  // namespace fos
