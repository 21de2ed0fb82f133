// Dequantize packed NVFP4 / IF4 tensors, and the GEMM's alpha.
//
// Arithmetic of the reference (src/fouroversix/quantize/backend.py:88-160,
// src/fouroversix/quantize/dequantize_utils.py:15-86): value and scale are first
// represented in fp16 and multiplied in fp16 (IF4 integer blocks multiply the integer
// by 6/7 in fp16 first), then (fp32(product) * amax) / divisor in fp32, then the cast.
#include "fos_common.cuh"

namespace fos {
namespace {

struct DequantParams {
    const uint8_t *codes;
    const uint8_t *sf;
    const float *amax;
    void *out;
    int64_t rows_p, cols_p, rows, cols, ld_out;
    int format, sf_tiled;
    float divisor;
};

template <typename OUT> __device__ __forceinline__ OUT to_out(float v);
template <> __device__ __forceinline__ float to_out<float>(float v) { return v; }
template <> __device__ __forceinline__ __half to_out<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 to_out<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float as_fp16(float v) { return __half2float(__float2half_rn(v)); }

// One thread per 16-value block: 8 bytes of codes and one scale in, 16 values out.
template <typename OUT>
__global__ void __launch_bounds__(256) dequantize_kernel(const DequantParams p) {
    const int64_t n_cb = p.cols_p >> 4;
    const int64_t cb_used = (p.cols + 15) >> 4;
    const int64_t total = p.rows * cb_used;
    const float amax = __ldg(p.amax);
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total;
         i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = i / cb_used, cb = i - r * cb_used;
        const uint2 c = *reinterpret_cast<const uint2 *>(p.codes + r * (p.cols_p >> 1) + cb * 8);
        uint32_t sfb = p.sf[sf_offset(r, cb, n_cb, p.sf_tiled != 0)];
        const bool is_int = p.format == FOS_IF4 && (sfb & 0x80u);
        if (p.format == FOS_IF4) sfb &= 0x7fu;
        const float s16 = e4m3_to_float(sfb);   // every E4M3 value is an fp16 value
        float v[16];
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
            v[2 * j] = __fdiv_rn(__fmul_rn(as_fp16(__fmul_rn(q.x, s16)), amax), p.divisor);
            v[2 * j + 1] = __fdiv_rn(__fmul_rn(as_fp16(__fmul_rn(q.y, s16)), amax), p.divisor);
        }
        OUT *dst = static_cast<OUT *>(p.out) + r * p.ld_out + cb * 16;
        const int64_t left = p.cols - cb * 16;
        const bool aligned = (reinterpret_cast<uintptr_t>(dst) & 15u) == 0;
        if (left >= 16 && aligned) {
            OUT tmp[16];
#pragma unroll
            for (int k = 0; k < 16; ++k) tmp[k] = to_out<OUT>(v[k]);
            const uint4 *src4 = reinterpret_cast<const uint4 *>(tmp);
#pragma unroll
            for (int k = 0; k < static_cast<int>(sizeof(OUT)); ++k) reinterpret_cast<uint4 *>(dst)[k] = src4[k];
        } else {
#pragma unroll
            for (int k = 0; k < 16; ++k)
                if (k < left) dst[k] = to_out<OUT>(v[k]);
        }
    }
}

__global__ void alpha_kernel(const float *amax_a, const float *amax_b, float denom, float *alpha) {
    alpha[0] = __fdiv_rn(__fmul_rn(amax_a[0], amax_b[0]), denom);
}

}  // namespace
}  // namespace fos

extern "C" int fos_dequantize(const uint8_t *codes, const uint8_t *sf, const float *amax, int format,
                              int scale_rule, int sf_layout, int64_t rows_p, int64_t cols_p, int64_t rows,
                              int64_t cols, void *out, int out_dtype, int64_t ld_out, void *stream_) {
    using namespace fos;
    if (!codes || !sf || !amax || !out) return FOS_ERR_INVALID_ARGUMENT;
    if (format != FOS_NVFP4 && format != FOS_IF4) return FOS_ERR_INVALID_ARGUMENT;
    if (scale_rule < FOS_RULE_STATIC_6 || scale_rule > FOS_RULE_ABS_MAX) return FOS_ERR_INVALID_ARGUMENT;
    if (sf_layout != FOS_SF_ROWMAJOR && sf_layout != FOS_SF_TILED) return FOS_ERR_INVALID_ARGUMENT;
    if (rows_p <= 0 || cols_p <= 0 || rows_p % 128 != 0 || cols_p % 64 != 0) return FOS_ERR_INVALID_ARGUMENT;
    if (rows <= 0 || cols <= 0 || rows > rows_p || cols > cols_p || ld_out < cols) return FOS_ERR_INVALID_ARGUMENT;
    if (out_dtype != FOS_BF16 && out_dtype != FOS_FP16 && out_dtype != FOS_FP32) return FOS_ERR_INVALID_ARGUMENT;
    if (reinterpret_cast<uintptr_t>(codes) % 8 != 0) return FOS_ERR_MISALIGNED;
    int st = check_device();
    if (st != FOS_OK) return st;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);

    DequantParams p{codes, sf, amax, out, rows_p, cols_p, rows, cols, ld_out, format,
                    sf_layout == FOS_SF_TILED, dequant_divisor(format, scale_rule)};
    const int64_t total = rows * ((cols + 15) / 16);
    int64_t blocks = (total + 255) / 256;
    if (blocks > 148 * 32) blocks = 148 * 32;
    const unsigned g = static_cast<unsigned>(blocks);
    if (out_dtype == FOS_BF16) dequantize_kernel<__nv_bfloat16><<<g, 256, 0, stream>>>(p);
    else if (out_dtype == FOS_FP16) dequantize_kernel<__half><<<g, 256, 0, stream>>>(p);
    else dequantize_kernel<float><<<g, 256, 0, stream>>>(p);
    FOS_CUDA_TRY(cudaGetLastError());
    return FOS_OK;
}

extern "C" int fos_gemm_alpha(const float *amax_a, int format_a, int rule_a, const float *amax_b, int format_b,
                              int rule_b, float *alpha, void *stream_) {
    using namespace fos;
    if (!amax_a || !amax_b || !alpha) return FOS_ERR_INVALID_ARGUMENT;
    int st = check_device();
    if (st != FOS_OK) return st;
    // the reference multiplies the integer constants exactly before the one division
    const float denom = static_cast<float>(static_cast<double>(dequant_divisor(format_a, rule_a)) *
                                           static_cast<double>(dequant_divisor(format_b, rule_b)));
    alpha_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream_)>>>(amax_a, amax_b, denom, alpha);
    FOS_CUDA_TRY(cudaGetLastError());
    return FOS_OK;
}
