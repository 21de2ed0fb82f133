// Dequantization arithmetic shared by the dequantize kernel and the fused fake-quantization
// path of the quantize kernel (sm_100a only).
//
// Arithmetic of the reference (src/fouroversix/quantize/backend.py:88-160,
// src/fouroversix/quantize/dequantize_utils.py:15-86): value and scale are first
// represented in fp16 and multiplied in fp16 (IF4 integer blocks multiply the integer
// by 6/7 in fp16 first), then (fp32(product) * amax) / divisor in fp32, then the cast.
#pragma once

#include "fos_common.cuh"

namespace fos {
namespace {

template <typename OUT> __device__ __forceinline__ OUT to_out(float v);
template <> __device__ __forceinline__ float to_out<float>(float v) { return v; }
template <> __device__ __forceinline__ __half to_out<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 to_out<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float as_fp16(float v) { return __half2float(__float2half_rn(v)); }

// a / d for d in {1536, 1792, 2688}, correctly rounded, without a division: quotient estimate,
// exact remainder, one correction (y = fl(1 / d)). Checked against a / d for EVERY finite binary32
// a on the host: equal for all |a| >= 2^-100 (the mismatches lie below 2^-117, where the remainder
// underflows), up to the sign of a zero result, which is copied from a here.
__device__ __forceinline__ uint64_t div_const2(uint64_t a, uint64_t d_neg, uint64_t y) {
    const uint64_t q0 = fma2(a, y, pack2(0.0f, 0.0f) /* a * y rounds the same; -0 handled below */);
    const uint64_t q1 = fma2(fma2(d_neg, q0, a), y, q0);
    return (q1 & 0x7fffffff7fffffffull) | (a & 0x8000000080000000ull);
}

struct DequantConsts {
    float amax, divisor, y;
    bool fast;          // every non-zero product is at least 2^-100 in magnitude
};

__device__ __forceinline__ DequantConsts dequant_consts(float amax, float divisor) {
    DequantConsts c;
    c.amax = amax;
    c.divisor = divisor;
    c.y = __frcp_rn(divisor);
    // the smallest non-zero fp16(value * scale) is 2^-10 (0.5 times the smallest E4M3 number)
    c.fast = amax >= 0x1p-90f && amax < 0x1p100f;   // no underflow of the remainder, no overflow of the product
    return c;
}

// The 16 values of one block: fp16(value) * fp16(scale) in fp16, then (fp32 * amax) / divisor.
__device__ __forceinline__ void dequantize_block(uint2 c, uint32_t sfb, bool is_if4, const DequantConsts &k, float (&v)[16]) {
    const bool is_int = is_if4 && (sfb & 0x80u);
    if (is_if4) sfb &= 0x7fu;
    const float s16 = e4m3_to_float(sfb);   // every E4M3 value is an fp16 value
    if (k.fast) {
        const __half2 s2 = __float2half2_rn(s16);
        const uint64_t amax2 = pack2(k.amax, k.amax), y2 = pack2(k.y, k.y), dneg2 = pack2(-k.divisor, -k.divisor);
        const float six_sevenths = static_cast<float>(6.0 / 7.0);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const uint32_t byte = ((j < 4 ? c.x : c.y) >> ((j & 3) * 8)) & 0xffu;
            __half2 val;
            if (is_int) {
                // two's-complement nibble n -> float: (n ^ 8) is n + 8 as an unsigned number, put
                // into the mantissa of 2^23 and shifted back by 2^23 + 8; then fp16(int * fl(6/7))
                const float lo = __uint_as_float(0x4b000000u | ((byte & 0xfu) ^ 8u)) - 8388616.0f;
                const float hi = __uint_as_float(0x4b000000u | ((byte >> 4) ^ 8u)) - 8388616.0f;
                val = __floats2half2_rn(__fmul_rn(lo, six_sevenths), __fmul_rn(hi, six_sevenths));
            } else {
                uint32_t h2;
                asm("{ .reg .b8 b; cvt.u8.u32 b, %1; cvt.rn.f16x2.e2m1x2 %0, b; }" : "=r"(h2) : "r"(byte));
                val = *reinterpret_cast<__half2 *>(&h2);
            }
            const float2 p = __half22float2(__hmul2(val, s2));                                  // one fp16 rounding
            const uint64_t a = fma2(pack2(p.x, p.y), amax2, pack2(0.0f, 0.0f));
            // fma(x, amax, +0) rounds like x * amax but turns -0 into +0: restore the sign
            const uint64_t a_signed = (a & 0x7fffffff7fffffffull) | (pack2(p.x, p.y) & 0x8000000080000000ull);
            unpack2f(div_const2(a_signed, dneg2, y2), v[2 * j], v[2 * j + 1]);
        }
        return;
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const uint32_t byte = ((j < 4 ? c.x : c.y) >> ((j & 3) * 8)) & 0xffu;
        float2 q;
        if (is_int) {
            const float six_sevenths = static_cast<float>(6.0 / 7.0);
            q.x = as_fp16(__fmul_rn(static_cast<float>(static_cast<int>(byte << 28) >> 28), six_sevenths));
            q.y = as_fp16(__fmul_rn(static_cast<float>(static_cast<int>(byte << 24) >> 28), six_sevenths));
        } else {
            q = e2m1x2_to_float2(byte);
        }
        v[2 * j] = __fdiv_rn(__fmul_rn(as_fp16(__fmul_rn(q.x, s16)), k.amax), k.divisor);
        v[2 * j + 1] = __fdiv_rn(__fmul_rn(as_fp16(__fmul_rn(q.y, s16)), k.amax), k.divisor);
    }
}

}  // namespace
}  // namespace fos
