// Dequantize packed NVFP4 / IF4 tensors, and the GEMM's alpha.
//
// Arithmetic of the reference (src/fouroversix/quantize/backend.py:88-160,
// src/fouroversix/quantize/dequantize_utils.py:15-86): value and scale are first
// represented in fp16 and multiplied in fp16 (IF4 integer blocks multiply the integer
// by 6/7 in fp16 first), then (fp32(product) * amax) / divisor in fp32, then the cast.
#include "fos_dequant.cuh"

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

// One thread per 16-value block: 8 bytes of codes and one scale in, 16 values out. A CTA takes
// runs of 256 blocks of one row at a time (contiguous codes in, contiguous values out).
template <typename OUT>
__global__ void __launch_bounds__(256) dequantize_kernel(const DequantParams p) {
    const int64_t n_cb = p.cols_p >> 4;
    const int cb_used = static_cast<int>((p.cols + 15) >> 4);
    const int chunks = (cb_used + 255) >> 8;
    const int64_t units = p.rows * chunks;
    const DequantConsts k = dequant_consts(__ldg(p.amax), p.divisor);
    for (int64_t u = blockIdx.x; u < units; u += gridDim.x) {
        const int64_t r = u / chunks;
        const int cb = static_cast<int>(u - r * chunks) * 256 + static_cast<int>(threadIdx.x);
        if (cb >= cb_used) continue;
        const uint2 c = *reinterpret_cast<const uint2 *>(p.codes + r * (p.cols_p >> 1) + cb * 8);
        const uint32_t sfb = p.sf[sf_offset(r, cb, n_cb, p.sf_tiled != 0)];
        float v[16];
        dequantize_block(c, sfb, p.format == FOS_IF4, k, v);
        OUT *dst = static_cast<OUT *>(p.out) + r * p.ld_out + cb * 16;
        const int64_t left = p.cols - static_cast<int64_t>(cb) * 16;
        if (left >= 16 && (reinterpret_cast<uintptr_t>(dst) & 15u) == 0) {
            __align__(16) OUT tmp[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) tmp[i] = to_out<OUT>(v[i]);
            const uint4 *src4 = reinterpret_cast<const uint4 *>(tmp);
#pragma unroll
            for (int i = 0; i < static_cast<int>(sizeof(OUT)); ++i) reinterpret_cast<uint4 *>(dst)[i] = src4[i];
        } else {
#pragma unroll
            for (int i = 0; i < 16; ++i)
                if (i < left) dst[i] = to_out<OUT>(v[i]);
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
    if (!codes || !sf || !out || (!amax && format != FOS_MXFP4)) return FOS_ERR_INVALID_ARGUMENT;
    if (format == FOS_MXFP4) {
        if (sf_layout != FOS_SF_ROWMAJOR && sf_layout != FOS_SF_TILED) return FOS_ERR_INVALID_ARGUMENT;
        if (rows_p <= 0 || cols_p <= 0 || rows_p % 128 != 0 || cols_p % 128 != 0) return FOS_ERR_INVALID_ARGUMENT;
        if (rows <= 0 || cols <= 0 || rows > rows_p || cols > cols_p || ld_out < cols) return FOS_ERR_INVALID_ARGUMENT;
        if (out_dtype != FOS_BF16 && out_dtype != FOS_FP16 && out_dtype != FOS_FP32) return FOS_ERR_INVALID_ARGUMENT;
        if (reinterpret_cast<uintptr_t>(codes) % 8 != 0) return FOS_ERR_MISALIGNED;
        const int st_mx = check_device();
        if (st_mx != FOS_OK) return st_mx;
        return dequantize_mxfp4(codes, sf, sf_layout, rows_p, cols_p, rows, cols, out, out_dtype, ld_out,
                                static_cast<cudaStream_t>(stream_));
    }
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
    const int64_t units = rows * ((((cols + 15) / 16) + 255) / 256);     // runs of 256 blocks of one row
    int64_t blocks = units;
    if (blocks > 148 * 8) blocks = 148 * 8;
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
