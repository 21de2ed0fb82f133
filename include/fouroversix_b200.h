/*
 * fouroversix_b200 - C ABI of the B200 (sm_100a) kernels for NVFP4 / IF4 block-scaled
 * quantization with Four-Over-Six adaptive block scaling, and for the FP4 GEMM that
 * consumes the result.
 *
 * Conventions
 *   - Every pointer is a DEVICE pointer unless stated otherwise. The caller owns every
 *     buffer; the library never allocates, frees or keeps a pointer after the call.
 *   - `stream` is a cudaStream_t passed as void* (NULL = the default stream). Work is
 *     enqueued on it and the call returns without synchronising.
 *   - Return value: FOS_OK (0) or a negative FOS_ERR_* code; fos_status_string() names it.
 *   - A quantized tensor "Y" is described by three buffers:
 *       codes  [rows_p, cols_p / 2] bytes, row-major, low nibble = even column
 *       sf     rows_p * cols_p / 16 bytes of E4M3 block scales, either in the
 *              128-row x 4-block tile order that tcgen05 block-scaled MMA consumes
 *              (FOS_SF_TILED) or row-major [rows_p, cols_p / 16] (FOS_SF_ROWMAJOR)
 *       amax   one float, max |x| of the source tensor
 *     with rows_p = rows rounded up to 128 and cols_p = cols rounded up to 64.
 *   - The entry points are re-entrant and the library has no settings: what varies per call is an
 *     argument. Calls on different streams or host threads may overlap.
 *
 * The "replaces" notes cite the reference project (mit-han-lab/fouroversix) by path.
 */
#ifndef FOUROVERSIX_B200_H
#define FOUROVERSIX_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FOS_OK 0
#define FOS_ERR_INVALID_ARGUMENT (-1)  /* bad enum value, negative size, NULL pointer */
#define FOS_ERR_UNSUPPORTED (-2)       /* combination this library does not implement */
#define FOS_ERR_MISALIGNED (-3)        /* pointer or stride breaks a stated alignment rule */
#define FOS_ERR_CUDA (-4)              /* a CUDA runtime call failed; see fos_last_cuda_error */
#define FOS_ERR_ARCH (-5)              /* the current device is not compute capability 10.x */
#define FOS_ERR_TIMEOUT (-6)           /* a bounded device-side wait gave up (status word) */
#define FOS_ERR_TOO_LARGE (-7)         /* size beyond a documented maximum */

/* element type of a high-precision tensor */
#define FOS_BF16 0
#define FOS_FP16 1
#define FOS_FP32 2                     /* outputs only */

/* 4-bit format */
#define FOS_NVFP4 0                    /* E2M1 values, E4M3 scale per 16 */
#define FOS_IF4 1                      /* per block E2M1 or INT4*(6/7); scale sign bit = int */
#define FOS_MXFP4 2                    /* E2M1 values, E8M0 scale per 32, no per-tensor scale */

/* scale rule; same numbers as ScaleRule.cuda_id, src/fouroversix/utils.py:271-280 */
#define FOS_RULE_STATIC_6 0
#define FOS_RULE_STATIC_4 1
#define FOS_RULE_MAE 2
#define FOS_RULE_MSE 3
#define FOS_RULE_ABS_MAX 4

#define FOS_SF_ROWMAJOR 0
#define FOS_SF_TILED 1

/* fos_quantize flags */
#define FOS_QUANTIZE_EXACT_ONLY 1      /* skip the fast 4-vs-6 pre-filter (testing aid) */
#define FOS_QUANTIZE_RHT 2             /* rotate every block of 16 along the quantized axis with the reference's
                                          16-point random Hadamard transform (QuantizationConfig.rht,
                                          src/fouroversix/quantize/utils.py:19-85) before quantizing; the length of
                                          that axis (cols, or rows when transposing) must be a multiple of 16 */
#define FOS_QUANTIZE_NO_TMA 4          /* kernel choice (testing aid; every kernel writes the same bytes): never a kernel
                                          fed by the TMA unit, i.e. treat x as if it were not 16-byte aligned */
#define FOS_QUANTIZE_UNBIASED 16        /* fos_quantize_stochastic only: RoundStyle.stochastic_unbiased, every maximum scaled by 16/17
                                          (src/fouroversix/utils.py:223-247); the same factor then belongs into
                                          fos_dequantize_ex (FOS_DEQUANT_UNBIASED) and fos_gemm_alpha_ex */
#define FOS_QUANTIZE_GENERAL_KERNEL 8  /* kernel choice (testing aid): the general TMA-fed kernel also for the
                                          configuration that has a kernel of its own (NVFP4 4/6 MSE, 1-D blocks) */

int fos_version(void);
const char *fos_status_string(int status);
/* cudaError_t of the most recent FOS_ERR_CUDA on the calling host thread, as an int. */
int fos_last_cuda_error(void);

/*
 * Quantize a row-major 2-D tensor x[rows, cols] (bf16 or fp16, row stride `ld`
 * elements, unit column stride) to Y = x, or to Y = x^T when `transpose` is set.
 * Writes all of codes / sf (padding included, no pre-zeroing needed) and amax_out.
 *
 *   format      FOS_NVFP4 (all five rules), FOS_IF4 (mae / mse / abs_max) or FOS_MXFP4 (static_6 /
 *               static_4; blocks of 32, cols padded to 128, one scale byte per 32 values, amax_out = 1,
 *               amax_in ignored; src/fouroversix/quantize/pytorch/reference.py:149-181)
 *   block_2d    0: one scale per 1x16 block of Y; 1: one scale per 16x16 block of Y
 *   sf_layout   FOS_SF_TILED or FOS_SF_ROWMAJOR
 *   amax_in     NULL: the library computes max|x| itself (one extra pass over x);
 *               else a device float holding it (skips that pass)
 *   amax_out    device float; receives the amax that was used (may equal amax_in)
 *
 * Results are bit-identical to the reference's PyTorch backend
 * (src/fouroversix/quantize/pytorch/reference.py:555-679 behind
 * src/fouroversix/quantize/pytorch/backend.py:40-121) for finite inputs whose scaled
 * magnitudes stay below 7 (always, unless a block's scale underflows E4M3).
 *
 * Replaces: torch.ops.fouroversix.quantize, src/fouroversix/csrc/bindings.cpp:28 and
 * src/fouroversix/csrc/quantize/fp4_quant.cu:99-239 (which supports only untransposed
 * 1-D NVFP4); for transposed / 2-D / IF4 it replaces the Triton entry
 * src/fouroversix/kernels/triton/ops.py:17-209.
 */
int fos_quantize(const void *x, int x_dtype, int64_t rows, int64_t cols, int64_t ld,
                 int format, int scale_rule, int block_2d, int transpose, int sf_layout,
                 const float *amax_in, uint8_t *codes, uint8_t *sf, float *amax_out,
                 int flags, void *stream);

/*
 * amax_out[0] = max |x| over x[rows, cols] (bf16 or fp16, row stride `ld` elements): the pass that
 * fos_quantize runs when it is given no amax, on its own. For callers that quantize one tensor in
 * pieces (row slabs on different GPUs): take the maximum of the pieces' values, pass it to every
 * fos_quantize call as amax_in, and the pieces carry the bytes the whole tensor would.
 *
 * Replaces: x.abs().max() of src/fouroversix/quantize/pytorch/reference.py:573-578 and the first pass
 * of the reference's CUDA kernel, src/fouroversix/csrc/include/fp4_quant_kernel.h:133-215.
 */
int fos_amax(const void *x, int x_dtype, int64_t rows, int64_t cols, int64_t ld, float *amax_out, void *stream);

/*
 * Dequantize Y (padded shape rows_p x cols_p) into out[rows, cols] (row stride
 * ld_out elements), cropping the padding: fp16(value) * fp16(|scale|) in fp16, then
 * (fp32 * amax) / (max value * max scale) and a cast to out_dtype.
 *
 * Replaces: QuantizeBackendBase.dequantize, src/fouroversix/quantize/backend.py:88-160
 * with src/fouroversix/quantize/dequantize_utils.py:4-86; the Triton kernel
 * src/fouroversix/kernels/triton/dequantize.py:110-154 for IF4.
 */
int fos_dequantize(const uint8_t *codes, const uint8_t *sf, const float *amax, int format,
                   int scale_rule, int sf_layout, int64_t rows_p, int64_t cols_p,
                   int64_t rows, int64_t cols, void *out, int out_dtype, int64_t ld_out,
                   void *stream);

/*
 * fos_dequantize with the two options of the reference's back-end interface it leaves out:
 *   intermediate_dtype  FOS_FP16 (what fos_dequantize does) or FOS_FP32: the type in which value and scale are
 *                       represented and multiplied (QuantizeBackendBase.dequantize(..., intermediate_dtype=...),
 *                       src/fouroversix/quantize/backend.py:88-160; the reference's tests use float32,
 *                       tests/test_quantize.py:442)
 *   flags               FOS_DEQUANT_VALUES_ONLY: only the raw values (E2M1 codes as numbers, IF4 integer blocks times
 *                       6/7), no scale, no amax (QuantizeBackendBase.dequantize_values,
 *                       src/fouroversix/quantize/backend.py:164-189); pass rows = rows_p and cols = cols_p for the
 *                       padded tensor the reference returns.
 *                       FOS_DEQUANT_UNBIASED: the tensor was quantized with FOS_QUANTIZE_UNBIASED, so the divisor
 *                       carries the factor 16/17 (round_style.adjustment_factor, backend.py:146-154)
 * amax may be NULL for FOS_MXFP4 or with FOS_DEQUANT_VALUES_ONLY.
 */
#define FOS_DEQUANT_VALUES_ONLY 1
#define FOS_DEQUANT_UNBIASED 2
int fos_dequantize_ex(const uint8_t *codes, const uint8_t *sf, const float *amax, int format,
                      int scale_rule, int sf_layout, int64_t rows_p, int64_t cols_p,
                      int64_t rows, int64_t cols, void *out, int out_dtype, int64_t ld_out,
                      int intermediate_dtype, int flags, void *stream);

/*
 * alpha[0] = amax_a[0] * amax_b[0] / (divisor(format_a, rule_a) * divisor(format_b, rule_b))
 * computed on the device (no host synchronisation).
 *
 * Replaces: the tensor expression in src/fouroversix/matmul/cutlass/backend.py:85-98.
 */
int fos_gemm_alpha(const float *amax_a, int format_a, int rule_a, const float *amax_b,
                   int format_b, int rule_b, float *alpha, void *stream);
/* The same with the factor 16/17 per operand that was quantized with FOS_QUANTIZE_UNBIASED
 * (src/fouroversix/matmul/cutlass/backend.py:95-96). */
int fos_gemm_alpha_ex(const float *amax_a, int format_a, int rule_a, int unbiased_a, const float *amax_b,
                      int format_b, int rule_b, int unbiased_b, float *alpha, void *stream);
/* The same for `count` pairs: alpha[i] from amax_a[i] and amax_b[i] (the groups of fos_gemm_nvfp4_grouped). */
int fos_gemm_alpha_grouped(const float *amax_a, int format_a, int rule_a, int unbiased_a, const float *amax_b,
                           int format_b, int rule_b, int unbiased_b, float *alpha, int count, void *stream);

/*
 * D[m, n] = alpha[0] * sum_k A[m, k] * B[n, k]   ("TN": both operands K-major)
 * A: codes [m_p, k_p/2] + tiled scales, B: codes [n_p, k_p/2] + tiled scales, both NVFP4
 * as written by fos_quantize(FOS_SF_TILED). m_p / n_p multiples of 128, k_p a multiple
 * of 64 (>= 64). Block-scaled tcgen05 MMA (kind::mxf4nvf4, UE4M3 scales per 16), fp32
 * accumulation in tensor memory, bf16 / fp16 / fp32 output. Only rows < m and columns
 * < n of D are written (row stride ldd elements; ldd * sizeof(out) a multiple of 16).
 * `status` is an optional device int32: it stays 0 unless a bounded wait timed out.
 *
 * Replaces: gemm_nvfp4nvfp4_accum_fp32_out_{bf16,fp16}_tnt,
 * src/fouroversix/csrc/bindings.cpp:31-33 and src/fouroversix/csrc/fp4_gemm.cu:40-186.
 */
int fos_gemm_nvfp4(const uint8_t *a_codes, const uint8_t *a_sf, const uint8_t *b_codes,
                   const uint8_t *b_sf, const float *alpha, void *d, int out_dtype,
                   int64_t m_p, int64_t n_p, int64_t k_p, int64_t m, int64_t n, int64_t ldd,
                   int32_t *status, void *stream);

/*
 * Per-call options of the FP4 GEMMs (the library keeps no process-wide settings). NULL = all zero.
 *   variant   0 = choose the kernel per problem; 128 / 256 = single-CTA kernel with 128 x 128 /
 *             128 x 256 tiles; 2 = CTA-pair kernel (256 x 256 tiles, cta_group::2) where the padded
 *             M and N are multiples of 256, else the single-CTA kernel. Every variant computes the
 *             same product (fp32 sums in a different order).
 *   max_ctas  0 = one persistent CTA per SM; n > 0 = at most n CTAs, which leaves SMs free for a
 *             kernel that must run beside the GEMM (a collective on another stream: a persistent
 *             grid over every SM would keep it waiting until the GEMM has finished).
 * No counterpart in the reference (its CUTLASS kernel has one tile shape and takes the whole GPU,
 * src/fouroversix/csrc/fp4_gemm.cu:166-172).
 */
typedef struct fos_gemm_opts {
    int32_t variant;
    int32_t max_ctas;
} fos_gemm_opts;
int fos_gemm_nvfp4_ex(const uint8_t *a_codes, const uint8_t *a_sf, const uint8_t *b_codes,
                      const uint8_t *b_sf, const float *alpha, void *d, int out_dtype,
                      int64_t m_p, int64_t n_p, int64_t k_p, int64_t m, int64_t n, int64_t ldd,
                      const fos_gemm_opts *opts, int32_t *status, void *stream);

/*
 * Activation quantization fused into the GEMM: D[m, n] = alpha[0] * sum_k q(x)[m, k] * B[n, k], where q is the
 * NVFP4 quantization of x[m, k] (bf16 / fp16, row stride x_ld elements) with scale rule static_6 or static_4 and
 * the per-tensor amax at x_amax (a device float: fos_amax, or a value the caller knows). The warps that would
 * wait for the tile's epilogue build the packed A tile and its scale tiles in shared memory, so the codes and
 * scales of x are never written to memory. Bit-identical to fos_quantize(x, static rule, amax_in = x_amax)
 * followed by fos_gemm_nvfp4. alpha as for fos_gemm_nvfp4 (fos_gemm_alpha with x_amax and the rule).
 * k must be a multiple of 64, x 32-byte aligned (base and row stride); the rows of A are padded to 128 in the
 * kernel. Every CTA that shares rows of x quantizes them again (n_p / 256 times), so this pays for narrow outputs
 * and costs time for wide ones; the 4/6 rules (two candidates per block) are not offered fused:
 * FOS_ERR_UNSUPPORTED, quantize first.
 *
 * Replaces: the un-fused pair quantize(input) -> quantized_matmul of
 * src/fouroversix/matmul/frontend.py:95-102 for static-rule activations.
 */
int fos_gemm_nvfp4_fused_a(const void *x, int x_dtype, int64_t x_ld, const float *x_amax, int x_rule,
                           const uint8_t *b_codes, const uint8_t *b_sf, const float *alpha, void *d,
                           int out_dtype, int64_t m, int64_t n_p, int64_t k, int64_t n, int64_t ldd,
                           int32_t *status, void *stream);

/*
 * A linear layer's forward pass on a packed weight as ONE host call: out[rows, out_features] = Q(x) @ W^T with x
 * [rows, in_features] (bf16 / fp16, row stride ld_x) quantized here (NVFP4, 1-D blocks, `activation_rule`, its amax
 * computed by the library) and W packed beforehand by fos_quantize (NVFP4, tiled scales, `weight_rule`, padded to
 * 128 rows and 64 columns). Enqueues what fos_quantize, fos_gemm_alpha and fos_gemm_nvfp4_ex enqueue, with the
 * packed activation, its amax and alpha in `workspace` (fos_linear_workspace_bytes(rows, in_features) bytes of
 * device memory, 256-byte aligned): same bits as the three calls. opts may be NULL; status as for fos_gemm_nvfp4.
 *
 * Replaces: FourOverSixLinearFunction.forward of src/fouroversix/model/modules/linear.py:40-110 for packed weights
 * (quantize the input, quantized_matmul), without its bias addition.
 */
int64_t fos_linear_workspace_bytes(int64_t rows, int64_t in_features);
int fos_linear_forward(const void *x, int x_dtype, int64_t rows, int64_t in_features, int64_t ld_x, int activation_rule,
                       const uint8_t *w_codes, const uint8_t *w_sf, const float *w_amax, int weight_rule,
                       int64_t out_features, void *out, int out_dtype, int64_t ld_out, void *workspace,
                       int64_t workspace_bytes, const fos_gemm_opts *opts, int32_t *status, void *stream);

/*
 * Grouped problems in one launch: num_groups GEMMs that share n, k and the output type, each with its own A rows,
 * its own B and its own alpha - what a mixture-of-experts layer does after routing, where the reference loops over
 * the experts on the host (one quantize + one GEMM per expert, the row counts read back from the device).
 *
 * Layout. The rows of all groups lie one after the other in one padded buffer of rows_capacity rows (a multiple of
 * 128): group g occupies rows group_start[g] .. group_start[g + 1] (num_groups + 1 int32 values in DEVICE memory,
 * multiples of 128, non-decreasing), of which the first group_rows[g] (device int32) are real and the rest padding.
 * The host never needs to know how the rows are spread: it sizes the buffers for the worst case
 * (sum of rows + 127 * num_groups, rounded up to 128). a_codes / a_sf / d are [rows_capacity, ...] as for
 * fos_gemm_nvfp4 (scales in 128 x 4 tiles; a group starts on a tile boundary); b_codes is
 * [num_groups][n_p][k_p / 2] and b_sf the groups' tiled scales one after the other; alpha has num_groups entries.
 * Only rows group_start[g] .. + group_rows[g] of d are written. An empty group costs nothing. num_groups <= 256.
 *
 * fos_quantize_grouped quantizes such a buffer of bf16 / fp16 rows: every group as a tensor of its own with its
 * own amax (amax_out[g]; computed here unless amax_in gives num_groups values), 1-D blocks, untransposed, tiled
 * scales, NVFP4 or IF4, any scale rule the format has - the bits fos_quantize gives for the group's rows alone.
 * Padding rows inside a group's range must be zero in x (they quantize to zero codes). cols must be a multiple of
 * 64 and x 16-byte aligned (base and row stride): FOS_ERR_UNSUPPORTED otherwise.
 *
 * Replaces: the per-expert loop of quantized_matmul calls in
 * src/fouroversix/model/modules/gpt_oss.py:297-335.
 */
int fos_quantize_grouped(const void *x, int x_dtype, int64_t rows_capacity, int64_t cols, int64_t ld, int format,
                         int scale_rule, const int32_t *group_start, const int32_t *group_rows, int num_groups,
                         const float *amax_in, uint8_t *codes, uint8_t *sf, float *amax_out, int flags,
                         void *stream);
int fos_gemm_nvfp4_grouped(const uint8_t *a_codes, const uint8_t *a_sf, const uint8_t *b_codes,
                           const uint8_t *b_sf, const float *alpha, void *d, int out_dtype,
                           const int32_t *group_start, const int32_t *group_rows, int num_groups,
                           int64_t rows_capacity, int64_t n_p, int64_t k_p, int64_t n, int64_t ldd,
                           const fos_gemm_opts *opts, int32_t *status, void *stream);

/*
 * The element-wise steps of a mixture-of-experts layer around the two grouped GEMMs, one launch each, on 16-bit
 * tensors (dtype FOS_BF16 or FOS_FP16 for every tensor of a call). The reference runs them as a chain of
 * element-wise tensor operations, each rounding its result to the tensors' type; these kernels keep every one of
 * those roundings, so the bits are the chain's. Row counts and leading dimensions in elements; widths must be
 * multiples of 8 and all tensors 16-byte aligned (base and row stride): FOS_ERR_UNSUPPORTED / FOS_ERR_MISALIGNED.
 *
 * fos_experts_gather_rows: out[r][0..cols) = x[row_token[r]][0..cols), zeros where row_token[r] < 0
 *   (row_token: rows_capacity int32 values in device memory). Fills the padded row buffer fos_quantize_grouped
 *   reads, padding rows included.
 * Both of the calls above and below that write such a buffer can also leave its per-expert maxima: with amax != NULL
 *   (num_experts floats, ZEROED by the caller in the stream before the call; gather_rows then also needs
 *   row_expert) amax[e] is raised to the largest |value| written for expert e - the words fos_quantize_grouped
 *   computes in a pass of its own unless they are handed to it as amax_in.
 * fos_experts_glu: gate_up [rows_capacity][2 * intermediate] with gate in the even and up in the odd columns,
 *   bias [experts][2 * intermediate], row_expert[r] the expert of row r or < 0 for a padding row (whose output row
 *   is zeros and whose input is not read):
 *     g = gate + bias; u = up + bias; g = min(g, limit); u = min(max(u, -limit), limit);
 *     out = (u + 1) * (g * sigmoid(g * alpha))                       out [rows_capacity][intermediate]
 * fos_experts_combine: for token t with slots k < top_k (top_k <= 8): pair_row[t * top_k + k] the row of y that
 *   holds the slot's result, pair_expert[...] its expert, pair_weight[...] its routing weight (16-bit, same type):
 *     out[t] = sum over the slots, in ascending order of the expert index, of (y[row] + bias[expert]) * weight
 *   with the running sum rounded to the 16-bit type after every addition - the order and the roundings of the
 *   reference's host loop over the experts, whatever order the slots are listed in.
 *
 * fos_experts_route: the tables the three calls above and the grouped calls take, from the layer's routing
 *   indices [tokens][top_k] (int32 or int64: index_bytes 4 or 8; device memory), in two launches and without a
 *   read-back: a stable counting sort of the (token, slot) pairs by expert. Writes group_rows[e] (pairs routed to
 *   expert e), group_start[e] (num_experts + 1 values: every expert starts on a multiple of 128 rows),
 *   pair_row[p] (the row of pair p = token * top_k + slot; ascending in p within an expert), pair_expert[p] (the
 *   index as int32), and row_token[r] / row_expert[r] for all rows_capacity rows (-1 for padding rows).
 *   rows_capacity must be a multiple of 128 and at least tokens * top_k + 127 * num_experts rounded up to 128 (the
 *   worst case, known without the counts). An index outside [0, num_experts) gives its pair the row -1, which
 *   fos_experts_combine skips. num_experts <= 256: FOS_ERR_UNSUPPORTED above. workspace: FOS_EXPERTS_ROUTE_WORKSPACE_INTS
 *   * num_experts int32 values of device memory that the call may overwrite (per-segment counts).
 *
 * Replaces: the element-wise tensor operations of src/fouroversix/model/modules/gpt_oss.py:310-333 and the
 * routing mask and its per-expert read-back of lines 286-303.
 */
/*
 * fos_experts_forward: the whole layer in one host call - the four calls above around two fos_quantize_grouped /
 * fos_gemm_alpha_grouped / fos_gemm_nvfp4_grouped chains, eleven kernels enqueued on `stream` without a read-back:
 *   out[t] = sum over the token's experts e (ascending) of
 *            (glu(x[t] @ gate_up[e]^T + gate_up_bias[e]) @ down[e]^T + down_bias[e]) * routing_weights[t][slot]
 * with both products in NVFP4 (activations quantized per expert with `activation_rule`, the weights packed
 * beforehand with `weight_rule`: codes [num_experts][n rounded up to 128][k / 2], tiled scales and one amax per
 * expert, as fos_quantize writes them for each expert's matrix) and every element-wise step as described above.
 * x, out, the biases and routing_weights are 16-bit tensors of type `dtype`; hidden and intermediate must be
 * multiples of 64, top_k <= 8, num_experts <= 256 (FOS_ERR_UNSUPPORTED otherwise). workspace: device memory of
 * fos_experts_workspace_bytes(...) bytes, 256-byte aligned, the call's only scratch (the library does not
 * allocate). status as for fos_gemm_nvfp4.
 *
 * Replaces: GptOssExperts.forward of src/fouroversix/model/modules/gpt_oss.py:270-335 after weight packing.
 */
int64_t fos_experts_workspace_bytes(int64_t tokens, int top_k, int num_experts, int64_t hidden, int64_t intermediate);
int fos_experts_forward(const void *x, int dtype, int64_t tokens, int64_t hidden, int64_t ld_x,
                        const void *routing_indices, int index_bytes, const void *routing_weights, int top_k,
                        int num_experts, const uint8_t *gate_up_codes, const uint8_t *gate_up_sf,
                        const float *gate_up_amax, const void *gate_up_bias, const uint8_t *down_codes,
                        const uint8_t *down_sf, const float *down_amax, const void *down_bias, int64_t intermediate,
                        int weight_rule, int activation_rule, float alpha, float limit, void *out, int64_t ld_out,
                        void *workspace, int64_t workspace_bytes, int32_t *status, void *stream);

#define FOS_EXPERTS_ROUTE_WORKSPACE_INTS 128
int fos_experts_route(const void *routing_indices, int index_bytes, int64_t tokens, int top_k, int num_experts,
                      int64_t rows_capacity, int32_t *group_start, int32_t *group_rows, int32_t *row_token,
                      int32_t *row_expert, int32_t *pair_row, int32_t *pair_expert, int32_t *workspace, void *stream);
int fos_experts_gather_rows(const void *x, int dtype, int64_t ld_x, const int32_t *row_token, void *out,
                            int64_t ld_out, int64_t rows_capacity, int64_t cols, const int32_t *row_expert, float *amax,
                            void *stream);
int fos_experts_glu(const void *gate_up, int dtype, int64_t ld_gate_up, const void *bias, const int32_t *row_expert,
                    void *out, int64_t ld_out, int64_t rows_capacity, int64_t intermediate, float alpha, float limit,
                    float *amax, void *stream);
int fos_experts_combine(const void *y, int dtype, int64_t ld_y, const void *bias, const int32_t *pair_row,
                        const int32_t *pair_expert, const void *pair_weight, int top_k, void *out, int64_t ld_out,
                        int64_t tokens, int64_t hidden, void *stream);

/*
 * The same GEMM for two MXFP4 operands (E8M0 scale per 32 values, scales in the 128 x 4 tile
 * order as fos_quantize(FOS_MXFP4, FOS_SF_TILED) writes them): tcgen05.mma kind::mxf4 with
 * scale_vec::2X. k_p must be a multiple of 128; everything else as for fos_gemm_nvfp4. The
 * reference passes alpha = 1 (src/fouroversix/matmul/cutlass/backend.py:79-84).
 *
 * Replaces: torch.ops.fouroversix.gemm_mxfp4mxfp4_accum_fp32_out_bf16_tnt,
 * src/fouroversix/csrc/bindings.cpp:29, Python caller src/fouroversix/matmul/cutlass/ops.py:6-20.
 */
int fos_gemm_mxfp4(const uint8_t *a_codes, const uint8_t *a_sf, const uint8_t *b_codes,
                   const uint8_t *b_sf, const float *alpha, void *d, int out_dtype, int64_t m_p,
                   int64_t n_p, int64_t k_p, int64_t m, int64_t n, int64_t ldd, int32_t *status,
                   void *stream);
int fos_gemm_mxfp4_ex(const uint8_t *a_codes, const uint8_t *a_sf, const uint8_t *b_codes,
                      const uint8_t *b_sf, const float *alpha, void *d, int out_dtype, int64_t m_p,
                      int64_t n_p, int64_t k_p, int64_t m, int64_t n, int64_t ldd,
                      const fos_gemm_opts *opts, int32_t *status, void *stream);

/*
 * Row-parallel layers over `world` GPUs of one node (2..8), in two kernels with a barrier between the ranks
 * after each (in stream order; the caller provides it):
 *
 * fos_gemm_nvfp4_scatter: the NVFP4 GEMM of fos_gemm_nvfp4, but the partial product of this rank is not
 *   stored to one buffer: row block mb (128 rows) belongs to rank mb % world (interleaved, so that the
 *   peer traffic is spread over the whole run) and is block mb / world of that rank's slab of m_p / world
 *   rows (m_p must be a multiple of 128 * world); every tile is stored, as it completes, into plane `rank`
 *   of its owner's staging buffer: d_peers[o] is rank o's buffer [world][m_p / world][ldd] of out_dtype
 *   (bf16 or fp16), mapped into this process (peer memory over NVLink, e.g. torch symmetric memory;
 *   d_peers[rank] is local). d_peers is a HOST array of `world` device pointers, each 32-byte aligned.
 * fos_reduce_gather: rank `rank` adds the `world` planes of its own staging buffer in binary32 (rank
 *   order), rounds once to `dtype` and stores the rows of its slab (row blocks mb % world == rank) of the
 *   result into out_peers[t] for every t (each [world * slab_rows][ld_out], 16-byte aligned; slab_rows a
 *   multiple of 128; n, ld_staging and ld_out multiples of 8).
 *
 * Together they are an all-reduce of the partial products whose first half rides on the GEMM's epilogue.
 * They stand where the reference relies on vLLM's tensor-parallel all-reduce after a row-parallel layer
 * (src/fouroversix/integrations/vllm_quantization.py:100-124); nothing in the reference's own package
 * corresponds to them.
 */
int fos_gemm_nvfp4_scatter(const uint8_t *a_codes, const uint8_t *a_sf, const uint8_t *b_codes,
                           const uint8_t *b_sf, const float *alpha, void *const *d_peers, int world, int rank,
                           int out_dtype, int64_t m_p, int64_t n_p, int64_t k_p, int64_t m, int64_t n,
                           int64_t ldd, int32_t *status, void *stream);
int fos_reduce_gather(const void *staging, void *const *out_peers, int world, int rank, int64_t slab_rows,
                      int64_t n, int64_t ld_staging, int64_t ld_out, int dtype, void *stream);

/*
 * The same exchange as ONE kernel after a plain GEMM, in place, for layers whose GEMM is too short to hide a
 * scatter behind: every rank has stored its full partial product [rows][ld] (rows a multiple of 128 * world;
 * n and ld multiples of 8; bf16 or fp16) into its own buffer buf_peers[rank]; rank `rank` loads the row blocks
 * mb % world == rank from every rank's buffer (peer loads), adds them in binary32 in rank order, rounds
 * once and stores them back into every rank's buffer (peer stores). Loads and stores use the two directions
 * of the links at once. A barrier between the ranks (in stream order) is needed before and after.
 */
int fos_allreduce_peer(void *const *buf_peers, int world, int rank, int64_t rows, int64_t n, int64_t ld,
                       int dtype, void *stream);

/*
 * Reduce-scatter over peer memory, for a row-parallel layer that hands ROW SLABS on to the next layer instead of
 * the full activation: every rank has stored its partial product into its own buffer buf_peers[rank] ([.][ld],
 * bf16 or fp16); the caller's rank loads rows row0 .. row0 + rows of EVERY rank's buffer (peer loads), adds them
 * in binary32 in rank order, rounds once and stores the sums into its LOCAL buffer out[rows][ld_out]. Nothing is
 * stored to a peer: (world - 1) / world of the slab's bytes cross this GPU's links inbound, once. n, ld, ld_out
 * multiples of 8. max_ctas > 0 caps the grid (the kernel usually runs beside the next chunk's GEMM). A barrier
 * between the ranks (in stream order) is needed after the GEMMs that filled the buffers and before any rank
 * overwrites its buffer. No counterpart in the reference (see fos_gemm_nvfp4_scatter).
 */
int fos_reduce_scatter_peer(void *const *buf_peers, int world, int64_t row0, int64_t rows, int64_t n, int64_t ld,
                            void *out, int64_t ld_out, int dtype, int max_ctas, void *stream);

/*
 * All-gather over peer memory, for the packed row slabs of the hand-off: every rank holds its piece (`bytes` bytes
 * at byte offset src_off of its buffer buf_peers[rank]); the caller's rank copies all pieces in rank order into
 * its LOCAL buffer, dst[r * bytes ..] = buf_peers[r][src_off ..] (peer loads only). bytes and src_off multiples of
 * 16. A barrier between the ranks (in stream order) is needed after the pieces were written and before any rank
 * overwrites its piece. No counterpart in the reference.
 */
int fos_allgather_peer(void *const *buf_peers, int world, int64_t src_off, int64_t bytes, void *dst, int max_ctas,
                       void *stream);

/*
 * D[m, n] = alpha[0] * sum_k A[m, k] * B[n, k] for operands in FOS_IF4 or FOS_NVFP4 (any mix),
 * scales in either layout. Each element is expanded to fp16(value) * fp16(|scale|) (integer
 * blocks: fp16(int * 6/7) first), the fp16 matrices are multiplied on the tensor cores
 * (kind::f16) with fp32 accumulation. `workspace` is device scratch of at least
 * fos_gemm_if4_workspace_bytes(m_p, n_p, k_p) = (m_p + n_p) * k_p * 2 bytes, 128-byte aligned; it
 * holds the expanded operands during the call and nothing afterwards. Other arguments as for
 * fos_gemm_nvfp4.
 *
 * Replaces: the reference's only IF4 matmuls, PyTorchMatmulBackend
 * (src/fouroversix/matmul/pytorch.py:33-52) and the disabled Triton kernel
 * (src/fouroversix/kernels/triton/matmul.py:14-233, src/fouroversix/matmul/triton.py:14-47).
 */
int64_t fos_gemm_if4_workspace_bytes(int64_t m_p, int64_t n_p, int64_t k_p);
int fos_gemm_if4(const uint8_t *a_codes, const uint8_t *a_sf, int a_format, int a_sf_layout,
                 const uint8_t *b_codes, const uint8_t *b_sf, int b_format, int b_sf_layout,
                 const float *alpha, void *d, int out_dtype, int64_t m_p, int64_t n_p, int64_t k_p,
                 int64_t m, int64_t n, int64_t ldd, void *workspace, int64_t workspace_bytes,
                 int32_t *status, void *stream);

/*
 * fos_gemm_if4 without a workspace argument, for callers that have no way to obtain device
 * scratch: code that runs where allocating is forbidden or impossible - in another library's
 * plug-in hook that may launch kernels but must not touch the allocator, under a memory pool that
 * is already fully handed out, or in a process whose allocator belongs to a different runtime.
 * (It still makes CUDA runtime calls - kernel launches - so it is not for cudaLaunchHostFunc
 * callbacks, which may make none.) The expanded fp16 operands are kept
 * in a buffer of FOS_GEMM_IF4_STATIC_WORKSPACE_BYTES that is part of the library image (each GPU
 * that loads the library holds that much memory until the process exits). The caller still passes
 * every input and output; the call performs no cudaMalloc / cudaFree and uses no allocating
 * library routine.
 *   - Limit: (m_p + n_p) * k_p * 2 <= FOS_GEMM_IF4_STATIC_WORKSPACE_BYTES, else FOS_ERR_TOO_LARGE.
 *   - The first call on a device looks up the buffer's device address (a one-time host-side
 *     set-up with that device current); make that first call outside any stream capture.
 *   - All calls on a device share the one buffer. It holds nothing between calls (every byte a
 *     call reads was written by that call), but two calls whose kernels overlap on the GPU, e.g.
 *     on different streams, overwrite each other's operands: serialise them.
 * No counterpart in the reference.
 */
#define FOS_GEMM_IF4_STATIC_WORKSPACE_BYTES (32 * 1024 * 1024)
int fos_gemm_if4_static(const uint8_t *a_codes, const uint8_t *a_sf, int a_format, int a_sf_layout,
                        const uint8_t *b_codes, const uint8_t *b_sf, int b_format, int b_sf_layout,
                        const float *alpha, void *d, int out_dtype, int64_t m_p, int64_t n_p, int64_t k_p,
                        int64_t m, int64_t n, int64_t ldd, int32_t *status, void *stream);

/*
 * fos_quantize with stochastic rounding (RoundStyle.stochastic of the reference: uniform noise of
 * +-half a grid step is added to every scaled magnitude before it is rounded; with a 4/6 rule both
 * candidates get independent noise and the better draw wins). `seed` selects the noise: the same
 * call with the same seed writes the same bytes. NVFP4 (any scale rule) or IF4 with the mse rule (both grids, the
 * E2M1 one and the integer one, draw independent noise and the smaller squared error of the draw wins:
 * src/fouroversix/quantize/pytorch/reference.py:55-63, 328-425), 1-D blocks, x 16-byte aligned (base and row
 * stride; when transposing also codes 16-byte and sf 2-byte aligned); anything else returns
 * FOS_ERR_UNSUPPORTED. With FOS_QUANTIZE_UNBIASED every maximum is scaled by 16/17 (RoundStyle.stochastic_unbiased). The reference draws its noise from torch's generator, so the two agree in
 * distribution, not bit for bit.
 *
 * Replaces: the rbits / is_rtn = false path of torch.ops.fouroversix.quantize
 * (src/fouroversix/csrc/bindings.cpp:28) and fake_quantize_to_e2m1(..., round_style=stochastic)
 * (src/fouroversix/quantize/pytorch/reference.py:30-51).
 */
int fos_quantize_stochastic(const void *x, int x_dtype, int64_t rows, int64_t cols, int64_t ld, int format,
                            int scale_rule, int block_2d, int transpose, int sf_layout, const float *amax_in,
                            uint8_t *codes, uint8_t *sf, float *amax_out, int flags, uint64_t seed, void *stream);

/*
 * Fused fake quantization: out = dequantize(quantize(x)) in x's element type, one pass over x
 * after the amax pass, nothing packed is written. 1-D blocks, untransposed; `out` is
 * [rows][ld_out] elements and only rows x cols of it are written. amax_in / amax_out / flags as
 * in fos_quantize. Returns FOS_ERR_UNSUPPORTED when x is not 16-byte aligned (base and row
 * stride): the caller then runs fos_quantize followed by fos_dequantize, which give the same bits.
 *
 * Replaces: QuantizeBackendBase.pseudo_quantize (src/fouroversix/quantize/backend.py:162-234) and the
 * Triton fake-quantization kernel (src/fouroversix/kernels/triton/quantize.py:1143-1246).
 */
int fos_pseudo_quantize(const void *x, int x_dtype, int64_t rows, int64_t cols, int64_t ld, int format,
                        int scale_rule, const float *amax_in, void *out, int64_t ld_out, float *amax_out,
                        int flags, void *stream);

/*
 * Diagnostics for the quantize kernels, which have no status argument: *site (host memory)
 * receives 0, or a small positive number naming the first bounded device-side wait that ever
 * gave up on the current device. Synchronises the device. No counterpart in the reference.
 */
int fos_wait_failure_site(int32_t *site);
/*
 * Which waits were in progress when a CTA gave up: roles[0] the quantize kernels, roles[1] the FP4 GEMMs, roles[2]
 * the IF4 GEMM; bit s is set for wait site s (the numbering of fos_wait_failure_site within each family) if a wait
 * there timed out or was cut short by its CTA's abort flag. Sticky like the site word; synchronises the device.
 */
int fos_wait_failure_roles(uint32_t roles[3]);

#ifdef __cplusplus
}
#endif
#endif /* FOUROVERSIX_B200_H */
