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
// runs of 256 blocks of one row (contiguous codes in, contiguous values out), DEPTH runs at a time: the
// loads of all of them are issued before the first block is decoded, so a thread has DEPTH loads in
// flight instead of one (with one, the kernel waited a memory latency per run: 29 us for 8192 x 4096).
constexpr int DEQUANT_DEPTH = 4;

// SMALL: every offset (bytes of codes and scales, elements of the output) fits 32 bits, so the address arithmetic
// of a block is 32-bit (a third of the kernel's instructions were 64-bit multiplies and compares).
template <typename OUT, bool SMALL>
__global__ void __launch_bounds__(256) dequantize_kernel(const DequantParams p) {
    using idx_t = typename std::conditional<SMALL, uint32_t, int64_t>::type;
    const int n_cb = static_cast<int>(p.cols_p >> 4);
    const int cb_used = static_cast<int>((p.cols + 15) >> 4);
    const int chunks = (cb_used + 255) >> 8;
    const idx_t units = static_cast<idx_t>(p.rows * chunks);
    const DequantConsts k = dequant_consts(__ldg(p.amax), p.divisor);
    // a unit is (row, chunk of 256 blocks); this CTA's units are blockIdx.x, + gridDim.x, ...: the pair is advanced
    // by additions (a division per unit cost more than decoding it)
    const int step_r = static_cast<int>(gridDim.x) / chunks, step_c = static_cast<int>(gridDim.x) % chunks;
    idx_t row0 = static_cast<idx_t>(blockIdx.x) / static_cast<idx_t>(chunks);
    int ch0 = static_cast<int>(blockIdx.x - row0 * chunks);
    const idx_t code_ld = static_cast<idx_t>(p.cols_p >> 1), ld_out = static_cast<idx_t>(p.ld_out);
    for (idx_t u0 = blockIdx.x; u0 < units; u0 += static_cast<idx_t>(gridDim.x) * DEQUANT_DEPTH) {
        uint2 c[DEQUANT_DEPTH];
        uint32_t sfb[DEQUANT_DEPTH];
        idx_t row[DEQUANT_DEPTH];
        int col_block[DEQUANT_DEPTH];
#pragma unroll
        for (int d = 0; d < DEQUANT_DEPTH; ++d) {
            const idx_t r = row0;
            const int cb = ch0 * 256 + static_cast<int>(threadIdx.x);
            row[d] = r;
            col_block[d] = (u0 + static_cast<idx_t>(d) * gridDim.x < units && cb < cb_used) ? cb : -1;
            c[d] = make_uint2(0u, 0u);
            sfb[d] = 0u;
            if (col_block[d] >= 0) {
                c[d] = *reinterpret_cast<const uint2 *>(p.codes + r * code_ld + cb * 8);
                const idx_t sf_off = p.sf_tiled
                    ? ((r >> 7) * static_cast<idx_t>(n_cb >> 2) + static_cast<idx_t>(cb >> 2)) * 512 +
                          static_cast<idx_t>((static_cast<int>(r) & 31) * 16 + ((static_cast<int>(r) >> 5) & 3) * 4 + (cb & 3))
                    : r * static_cast<idx_t>(n_cb) + static_cast<idx_t>(cb);
                sfb[d] = p.sf[sf_off];
            }
            row0 += step_r;                      // the next unit of this CTA
            ch0 += step_c;
            if (ch0 >= chunks) { ch0 -= chunks; ++row0; }
        }
#pragma unroll
        for (int d = 0; d < DEQUANT_DEPTH; ++d) {
            const int cb = col_block[d];
            if (cb < 0) continue;
            OUT *dst = static_cast<OUT *>(p.out) + (row[d] * ld_out + static_cast<idx_t>(cb * 16));
            const int64_t left = p.cols - static_cast<int64_t>(cb) * 16;
            if constexpr (sizeof(OUT) == 2) {
                // bf16 / fp16 outputs: the whole block from a table of its eight magnitudes
                uint32_t o[8];
                if (dequantize_block_packed<OUT>(c[d], sfb[d], k, o, p.format == FOS_IF4)) {
                    if (left >= 16 && (reinterpret_cast<uintptr_t>(dst) & 31u) == 0) {
                        stg_32(dst, o);                       // one 32-byte store: whole sectors per instruction
                    } else if (left >= 16 && (reinterpret_cast<uintptr_t>(dst) & 15u) == 0) {
                        reinterpret_cast<uint4 *>(dst)[0] = make_uint4(o[0], o[1], o[2], o[3]);
                        reinterpret_cast<uint4 *>(dst)[1] = make_uint4(o[4], o[5], o[6], o[7]);
                    } else {
                        uint16_t *d16 = reinterpret_cast<uint16_t *>(dst);
#pragma unroll
                        for (int i = 0; i < 16; ++i)
                            if (i < left) d16[i] = static_cast<uint16_t>(o[i >> 1] >> ((i & 1) * 16));
                    }
                    continue;
                }
            }
            float v[16];
            dequantize_block(c[d], sfb[d], p.format == FOS_IF4, k, v);
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
}

// The general form, for what the fast kernels above do not cover: a float32 intermediate
// (QuantizeBackendBase.dequantize(..., intermediate_dtype=torch.float32), src/fouroversix/quantize/backend.py:
// 88-160) and the raw values alone (dequantize_values, :164-189). One thread per block of 16 values, every
// step one IEEE operation in the reference's order:
//   value  E2M1 code as a number (exact in any type), or for an IF4 integer block I(int * fl32(6/7))
//   scale  E4M3 / E8M0 byte converted to I
//   I(value * scale), then for NVFP4 / IF4 (fp32 * amax) / divisor, then the cast to the output type
// with I = fp16 or fp32. `values_only` stops after the first line (and writes the padded tensor).
struct GeneralDequantParams {
    const uint8_t *codes;
    const uint8_t *sf;
    const float *amax;
    void *out;
    int64_t rows_p, cols_p, rows, cols, ld_out;
    int format, sf_tiled, intermediate_fp32, values_only;
    float divisor;
};

__device__ __forceinline__ float round_to_intermediate(float v, bool fp32) { return fp32 ? v : as_fp16(v); }

template <typename OUT>
__global__ void __launch_bounds__(256) dequantize_general_kernel(const GeneralDequantParams p) {
    const int block = p.format == FOS_MXFP4 ? 32 : 16;
    const int64_t n_cb = p.cols_p / block;                      // scale bytes per row
    const int64_t runs_per_row = (p.cols + 15) / 16, total = p.rows * runs_per_row;
    const float amax = (p.amax != nullptr && !p.values_only) ? __ldg(p.amax) : 1.0f;
    const float six_sevenths = static_cast<float>(6.0 / 7.0);
    const bool f32 = p.intermediate_fp32 != 0;
    OUT *out = static_cast<OUT *>(p.out);
    for (int64_t u = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; u < total;
         u += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int64_t r = total < (int64_t(1) << 31) ? static_cast<int64_t>(static_cast<uint32_t>(u) / static_cast<uint32_t>(runs_per_row))
                                                     : u / runs_per_row;
        const int64_t col = (u - r * runs_per_row) * 16;
        const uint2 c = *reinterpret_cast<const uint2 *>(p.codes + r * (p.cols_p >> 1) + (col >> 1));
        uint32_t sfb = p.sf[sf_offset(r, col / block, n_cb, p.sf_tiled != 0)];
        const bool is_int = p.format == FOS_IF4 && (sfb & 0x80u);
        if (p.format == FOS_IF4) sfb &= 0x7fu;
        float scale;
        if (p.format == FOS_MXFP4) {
            scale = sfb == 255u ? __uint_as_float(0x7fc00000u) : (sfb == 0u ? 0x1p-127f : __uint_as_float(sfb << 23));
        } else {
            scale = e4m3_to_float(sfb);
        }
        scale = round_to_intermediate(scale, f32);              // (E8M0 -> fp16 overflows / underflows like the reference's cast)
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const uint32_t byte = ((j < 4 ? c.x : c.y) >> ((j & 3) * 8)) & 0xffu;
            float2 q;
            if (is_int) {
                q.x = __fmul_rn(static_cast<float>(static_cast<int>(byte << 28) >> 28), six_sevenths);
                q.y = __fmul_rn(static_cast<float>(static_cast<int>(byte << 24) >> 28), six_sevenths);
            } else {
                q = e2m1x2_to_float2(byte);
            }
            float v[2] = {q.x, q.y};
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                float y;
                if (p.values_only) {
                    y = v[h];                                    // rounded once, to the output type, below
                } else {
                    y = round_to_intermediate(__fmul_rn(round_to_intermediate(v[h], f32), scale), f32);
                    if (p.format != FOS_MXFP4) y = __fdiv_rn(__fmul_rn(y, amax), p.divisor);
                }
                if (col + 2 * j + h < p.cols) out[r * p.ld_out + col + 2 * j + h] = to_out<OUT>(y);
            }
        }
    }
}

__global__ void alpha_kernel(const float *amax_a, const float *amax_b, float denom, float *alpha, int count) {
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < count; i += gridDim.x * blockDim.x)
        alpha[i] = __fdiv_rn(__fmul_rn(amax_a[i], amax_b[i]), denom);
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
    // 32-bit offsets when the padded tensor has fewer than 2^31 elements and the output fits the same bound
    const bool small = rows_p * cols_p < (int64_t(1) << 31) && rows * ld_out < (int64_t(1) << 31) && units + 4 * blocks < (int64_t(1) << 31);
    if (small) {
        if (out_dtype == FOS_BF16) dequantize_kernel<__nv_bfloat16, true><<<g, 256, 0, stream>>>(p);
        else if (out_dtype == FOS_FP16) dequantize_kernel<__half, true><<<g, 256, 0, stream>>>(p);
        else dequantize_kernel<float, true><<<g, 256, 0, stream>>>(p);
    } else {
        if (out_dtype == FOS_BF16) dequantize_kernel<__nv_bfloat16, false><<<g, 256, 0, stream>>>(p);
        else if (out_dtype == FOS_FP16) dequantize_kernel<__half, false><<<g, 256, 0, stream>>>(p);
        else dequantize_kernel<float, false><<<g, 256, 0, stream>>>(p);
    }
    FOS_CUDA_TRY(cudaGetLastError());
    return FOS_OK;
}

extern "C" int fos_dequantize_ex(const uint8_t *codes, const uint8_t *sf, const float *amax, int format,
                                 int scale_rule, int sf_layout, int64_t rows_p, int64_t cols_p, int64_t rows,
                                 int64_t cols, void *out, int out_dtype, int64_t ld_out, int intermediate_dtype,
                                 int flags, void *stream_) {
    using namespace fos;
    const int values_only = flags & FOS_DEQUANT_VALUES_ONLY;
    const bool unbiased = (flags & FOS_DEQUANT_UNBIASED) != 0;
    if (intermediate_dtype != FOS_FP16 && intermediate_dtype != FOS_FP32) return FOS_ERR_UNSUPPORTED;
    if (intermediate_dtype == FOS_FP16 && !values_only && !unbiased)
        return fos_dequantize(codes, sf, amax, format, scale_rule, sf_layout, rows_p, cols_p, rows, cols, out, out_dtype,
                              ld_out, stream_);
    if (!codes || !sf || !out) return FOS_ERR_INVALID_ARGUMENT;
    if (format != FOS_NVFP4 && format != FOS_IF4 && format != FOS_MXFP4) return FOS_ERR_INVALID_ARGUMENT;
    if (!values_only && format != FOS_MXFP4 && !amax) return FOS_ERR_INVALID_ARGUMENT;
    if (scale_rule < FOS_RULE_STATIC_6 || scale_rule > FOS_RULE_ABS_MAX) return FOS_ERR_INVALID_ARGUMENT;
    if (sf_layout != FOS_SF_ROWMAJOR && sf_layout != FOS_SF_TILED) return FOS_ERR_INVALID_ARGUMENT;
    if (rows_p <= 0 || cols_p <= 0 || rows_p % 128 != 0 || cols_p % (format == FOS_MXFP4 ? 128 : 64) != 0) return FOS_ERR_INVALID_ARGUMENT;
    if (rows <= 0 || cols <= 0 || rows > rows_p || cols > cols_p || ld_out < cols) return FOS_ERR_INVALID_ARGUMENT;
    if (out_dtype != FOS_BF16 && out_dtype != FOS_FP16 && out_dtype != FOS_FP32) return FOS_ERR_INVALID_ARGUMENT;
    if (reinterpret_cast<uintptr_t>(codes) % 8 != 0) return FOS_ERR_MISALIGNED;
    const int st = check_device();
    if (st != FOS_OK) return st;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    GeneralDequantParams p{codes, sf, amax, out, rows_p, cols_p, rows, cols, ld_out, format, sf_layout == FOS_SF_TILED,
                           intermediate_dtype == FOS_FP32, values_only != 0,
                           format == FOS_MXFP4 ? 1.0f : dequant_divisor(format, scale_rule)};
    // stochastic_unbiased tensors carry maxima scaled by 16/17: the product is formed in double, as the reference
    // forms it as a Python float, and rounded to binary32 once
    if (unbiased && format != FOS_MXFP4) p.divisor = static_cast<float>(static_cast<double>(p.divisor) * (16.0 / 17.0));
    int64_t blocks = (rows * ((cols + 15) / 16) + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    const unsigned g = static_cast<unsigned>(blocks);
    if (out_dtype == FOS_BF16) dequantize_general_kernel<__nv_bfloat16><<<g, 256, 0, stream>>>(p);
    else if (out_dtype == FOS_FP16) dequantize_general_kernel<__half><<<g, 256, 0, stream>>>(p);
    else dequantize_general_kernel<float><<<g, 256, 0, stream>>>(p);
    FOS_CUDA_TRY(cudaGetLastError());
    return FOS_OK;
}

extern "C" int fos_gemm_alpha(const float *amax_a, int format_a, int rule_a, const float *amax_b, int format_b,
                              int rule_b, float *alpha, void *stream_) {
    return fos_gemm_alpha_ex(amax_a, format_a, rule_a, 0, amax_b, format_b, rule_b, 0, alpha, stream_);
}

extern "C" int fos_gemm_alpha_ex(const float *amax_a, int format_a, int rule_a, int unbiased_a, const float *amax_b,
                                 int format_b, int rule_b, int unbiased_b, float *alpha, void *stream_) {
    return fos_gemm_alpha_grouped(amax_a, format_a, rule_a, unbiased_a, amax_b, format_b, rule_b, unbiased_b, alpha, 1, stream_);
}

extern "C" int fos_gemm_alpha_grouped(const float *amax_a, int format_a, int rule_a, int unbiased_a, const float *amax_b,
                                      int format_b, int rule_b, int unbiased_b, float *alpha, int count, void *stream_) {
    using namespace fos;
    if (!amax_a || !amax_b || !alpha || count <= 0) return FOS_ERR_INVALID_ARGUMENT;
    int st = check_device();
    if (st != FOS_OK) return st;
    // the reference multiplies the constants as Python numbers (exactly, for the integers) before the one division
    double product = static_cast<double>(dequant_divisor(format_a, rule_a)) * static_cast<double>(dequant_divisor(format_b, rule_b));
    if (unbiased_a) product *= 16.0 / 17.0;
    if (unbiased_b) product *= 16.0 / 17.0;
    const float denom = static_cast<float>(product);
    const int threads = count < 256 ? ((count + 31) / 32) * 32 : 256;
    alpha_kernel<<<(count + threads - 1) / threads, threads, 0, static_cast<cudaStream_t>(stream_)>>>(amax_a, amax_b, denom, alpha, count);
    FOS_CUDA_TRY(cudaGetLastError());
    return FOS_OK;
}
