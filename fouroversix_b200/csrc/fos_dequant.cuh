// Dequantization arithmetic shared by the dequantize kernel and the fused fake-quantization
// path of the quantize kernel (sm_100a only).
//
// Arithmetic of the reference (src/fouroversix/quantize/backend.py:88-160,
// src/fouroversix/quantize/dequantize_utils.py:15-86): value and scale are first
// represented in fp16 and multiplied in fp16 (IF4 integer blocks multiply the integer
// by 6/7 in fp16 first), then (fp32(product) * amax) / divisor in fp32, then the cast.
#pragma once

#include <type_traits>

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

// Two floats -> one word of two 16-bit outputs (`lo` in the lower half), round to nearest even.
template <typename OUT>
__device__ __forceinline__ uint32_t pack16x2(float lo, float hi) {
    if constexpr (std::is_same<OUT, __half>::value) {
        const __half2 h = __floats2half2_rn(lo, hi);
        return *reinterpret_cast<const uint32_t *>(&h);
    } else {
        const __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
        return *reinterpret_cast<const uint32_t *>(&h);
    }
}

// One NVFP4 block straight to sixteen 16-bit outputs (o[i] = values 2i, 2i + 1), with two multiplications, two
// divisions and two conversions per BLOCK instead of per value. An E2M1 magnitude is 2^k or 1.5 * 2^k, the product
// with the E4M3 scale s is exact in fp16 (at most 6 significant bits), and scaling by a power of two commutes with
// every rounding on the way as long as nothing leaves the normal range:
//     out(+-2^k)       = +-2^k * OUT(fl32(fl32(s * amax) / divisor))        = +-2^k * Q1
//     out(+-1.5 * 2^k) = +-2^k * OUT(fl32(fl32(1.5 s * amax) / divisor))    = +-2^k * Q3
// so the eight magnitudes are Q1 / 2, Q1, Q3, 2 Q1, 2 Q3, 4 Q1, 4 Q3 (exponent-field additions on the 16-bit
// patterns) and zero; a byte permute looks them up by code, another one supplies the sign bit. The same bits as
// dequantize_block followed by the cast (compared over whole tensors against the reference's fixtures and the
// host-side restatement). Returns false, leaving o alone, for a block it does not take: amax outside the range
// that keeps every step normal (k.fast), a scale byte with the sign bit set or NaN, or - fp16 outputs - a
// magnitude that would leave fp16's normal range.
template <typename OUT>
__device__ __forceinline__ bool dequantize_block_packed(uint2 c, uint32_t sfb, const DequantConsts &k, uint32_t (&o)[8],
                                                        bool is_if4 = false) {
    static_assert(sizeof(OUT) == 2, "16-bit outputs");
    constexpr bool HALF = std::is_same<OUT, __half>::value;
    constexpr uint32_t E = HALF ? 0x0400u : 0x0080u, E2 = E | (E << 16);       // one step of the exponent field
    const bool is_int = is_if4 && (sfb & 0x80u);
    if (is_if4) sfb &= 0x7fu;
    if (!k.fast || (sfb & 0x80u) || sfb == 0x7fu) return false;
    const float s = e4m3_to_float(sfb);
    const uint64_t amax2 = pack2(k.amax, k.amax), dneg2 = pack2(-k.divisor, -k.divisor), y2 = pack2(k.y, k.y);
    uint32_t t01, t23, t45, t67, mag[2], sgn[2];
    sgn[0] = (c.x >> 3) & 0x11111111u;
    sgn[1] = (c.y >> 3) & 0x11111111u;
    if (is_int) {
        // IF4 integer block: the seven magnitudes fp16(fp16(i * 6/7) * s), i = 1 .. 7, each through (x * amax) / divisor
        // and the cast (no power-of-two structure to exploit: four packed products, quotients and conversions per
        // block instead of sixteen); the magnitude of a two's-complement nibble is (n ^ m) + sign, m = 15 where the
        // sign bit is set (-8 does not occur: the quantizer clamps to +-7)
        const __half2 s2 = __float2half2_rn(s);
        auto entry = [&](uint32_t consts) {                                  // consts: fp16(i * fl32(6/7)) for two i
            const float2 p = __half22float2(__hmul2(*reinterpret_cast<const __half2 *>(&consts), s2));
            float q0, q1;
            unpack2f(div_const2(fma2(pack2(p.x, p.y), amax2, pack2(0.0f, 0.0f)), dneg2, y2), q0, q1);
            return pack16x2<OUT>(q0, q1);
        };
        t01 = entry(0x3adb0000u);
        t23 = entry(0x41253edbu);
        t45 = entry(0x444942dbu);
        t67 = entry(0x46004525u);
        mag[0] = ((c.x ^ (sgn[0] * 15u)) + sgn[0]) & 0x77777777u;
        mag[1] = ((c.y ^ (sgn[1] * 15u)) + sgn[1]) & 0x77777777u;
    } else {
        const uint64_t a = fma2(pack2(s, __fmul_rn(s, 1.5f)), amax2, pack2(0.0f, 0.0f));
        float q1, q3;
        unpack2f(div_const2(a, dneg2, y2), q1, q3);
        if (HALF && q1 != 0.0f && !(q1 >= 0x1p-13f && q3 < 16376.0f)) return false;
        t23 = pack16x2<OUT>(q1, q3);                         // [Q1, Q3]
        t01 = (t23 << 16) - (E << 16);                       // [0, Q1 / 2]
        t45 = t23 + E2;                                      // [2 Q1, 2 Q3]
        t67 = t45 + E2;                                      // [4 Q1, 4 Q3]
        if ((t23 & 0xffffu) == 0u) t01 = t23 = t45 = t67 = 0u;   // a zero scale: every magnitude is zero
        mag[0] = c.x & 0x77777777u;
        mag[1] = c.y & 0x77777777u;
    }
    const uint32_t la = __byte_perm(t01, t23, 0x6420), ha = __byte_perm(t01, t23, 0x7531);   // low / high bytes of
    const uint32_t lb = __byte_perm(t45, t67, 0x6420), hb = __byte_perm(t45, t67, 0x7531);   // magnitudes 0-3, 4-7
#pragma unroll
    for (int w = 0; w < 2; ++w) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const uint32_t sel = h ? mag[w] >> 16 : mag[w], ss = h ? sgn[w] >> 16 : sgn[w];
            const uint32_t lo = __byte_perm(la, lb, sel);
            const uint32_t hi = __byte_perm(ha, hb, sel) | __byte_perm(0x00008000u, 0u, ss);
            o[4 * w + 2 * h] = __byte_perm(lo, hi, 0x5140);
            o[4 * w + 2 * h + 1] = __byte_perm(lo, hi, 0x7362);
        }
    }
    return true;
}

}  // namespace
}  // namespace fos
