// NVFP4 / IF4 block-scaled quantization with Four-Over-Six adaptive block scaling.
//
// One CTA of 512 threads produces one 128-row x 64-column tile of the quantized tensor
// Y (= x, or x^T): 512 blocks of 16 values, one per thread, so that every thread keeps
// its 16 inputs, both candidate code sets and both error sums in registers.
//
// The arithmetic follows the reference's eager PyTorch implementation operation by
// operation (src/fouroversix/quantize/pytorch/reference.py:184-325, 328-425, 555-679):
// IEEE binary32, one rounding per step (__fmul_rn / __fadd_rn / __fdiv_rn / __frcp_rn,
// which the compiler never contracts into FMAs), and the summation order of an eager
// last-axis sum. The 4-versus-6 decision of the common case (1-D blocks, mean-squared
// error) is first taken with a cheaper FMA-based estimate; the estimate is only trusted
// when the two error sums differ by more than a proven bound on its own inaccuracy,
// otherwise the block is re-evaluated with the exact sequence. The result is therefore
// identical to always running the exact sequence.
#include "fos_common.cuh"

namespace fos {
namespace {

constexpr int KIND_STATIC = 0;    // NVFP4, one candidate (static_6 / static_4)
constexpr int KIND_ADAPTIVE = 1;  // NVFP4, "6" versus "4" candidate
constexpr int KIND_IF4 = 2;       // IF4, float grid versus integer grid

constexpr int TILE_ROWS = 128;
constexpr int TILE_COLS = 64;
constexpr int CTA_THREADS = 512;
constexpr unsigned FULL = 0xffffffffu;

struct QuantParams {
    const void *x;
    int64_t rows, cols, ld;      // source tensor
    int64_t out_rows, out_cols;  // Y before padding
    int64_t rows_p, cols_p;      // Y after padding
    const float *amax;           // device, already final
    uint8_t *codes;
    uint8_t *sf;
    int rule;
    int sf_tiled;
    int exact_only;
    int vec_bytes;               // 32, 16 or 0: widest aligned load usable on x
};

// ------------------------------------------------------------------------------------
// per-tensor amax
// ------------------------------------------------------------------------------------

template <typename T>
__global__ void __launch_bounds__(256) amax_kernel(const T *__restrict__ x, int64_t rows, int64_t cols,
                                                   int64_t ld, int vec16, float *amax) {
    float m = 0.0f;
    if (vec16) {
        const int64_t chunks_per_row = cols >> 3;
        const int64_t total = rows * chunks_per_row;
        for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total;
             i += (int64_t)gridDim.x * blockDim.x) {
            int64_t r = i / chunks_per_row, c = i - r * chunks_per_row;
            uint4 w = ldg_nc_16(x + r * ld + c * 8);
            uint32_t ws[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                float2 f = unpack2<T>(ws[k]);
                m = fmaxf(m, fmaxf(fabsf(f.x), fabsf(f.y)));
            }
        }
    } else {
        const int64_t total = rows * cols;
        for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total;
             i += (int64_t)gridDim.x * blockDim.x) {
            int64_t r = i / cols, c = i - r * cols;
            m = fmaxf(m, fabsf(elem_to_float<T>(x[r * ld + c])));
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(FULL, m, o));
    __shared__ float warp_max[8];
    if ((threadIdx.x & 31) == 0) warp_max[threadIdx.x >> 5] = m;
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < 8; ++w) m = fmaxf(m, warp_max[w]);
        // non-negative floats order like their bit patterns
        atomicMax(reinterpret_cast<int *>(amax), __float_as_int(m));
    }
}

// ------------------------------------------------------------------------------------
// building blocks
// ------------------------------------------------------------------------------------

// E2M1 codes of v[i] * r; `guard` re-adds +0.0 so that a product that underflows to
// -0.0 encodes as +0 (the reference multiplies by sign(x_scaled), which is 0 there).
__device__ __forceinline__ void encode_e2m1(const float (&v)[16], float r, bool guard, uint32_t &lo, uint32_t &hi) {
    float xs[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) xs[i] = __fmul_rn(v[i], r);
    if (guard) {
#pragma unroll
        for (int i = 0; i < 16; ++i) xs[i] = __fadd_rn(xs[i], 0.0f);
    }
    lo = cvt_e2m1x8(xs);
    hi = cvt_e2m1x8(xs + 8);
}

// Two's-complement INT4 codes of round(clamp(v * r * (7/6), -7, 7)).
__device__ __forceinline__ void encode_int4(const float (&v)[16], float r, uint32_t &lo, uint32_t &hi) {
    const float to_int = 1.16666666f;
    uint32_t w[2] = {0u, 0u};
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        float t = __fmul_rn(__fmul_rn(v[i], r), to_int);
        t = fminf(fmaxf(t, -7.0f), 7.0f);
        int q = __float2int_rn(t);
        w[i >> 3] |= (static_cast<uint32_t>(q) & 0xfu) << ((i & 7) * 4);
    }
    lo = w[0];
    hi = w[1];
}

// Per-element error terms of one candidate, exact reference sequence:
//   deq = ((value * scale) * amax [* 6/7]) / divisor ; d = deq - x ; d*d or |d|.
template <bool IS_INT>
__device__ __forceinline__ void exact_error_terms(const float (&v)[16], uint32_t lo, uint32_t hi, float scale,
                                                  float amax, float divisor, int rule, float (&e)[16]) {
    const float from_int = 0.8571428571f;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        uint32_t byte = ((j < 4 ? lo : hi) >> ((j & 3) * 8)) & 0xffu;
        float2 q;
        if (IS_INT) {
            q.x = static_cast<float>(static_cast<int>(byte << 28) >> 28);
            q.y = static_cast<float>(static_cast<int>(byte << 24) >> 28);
        } else {
            q = e2m1x2_to_float2(byte);
        }
        float qv[2] = {q.x, q.y};
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            float t = __fmul_rn(__fmul_rn(qv[h], scale), amax);
            if (IS_INT) t = __fmul_rn(t, from_int);
            float d = __fsub_rn(__fdiv_rn(t, divisor), v[2 * j + h]);
            e[2 * j + h] = (rule == FOS_RULE_MSE) ? __fmul_rn(d, d) : fabsf(d);
        }
    }
}

// Eager last-axis sum over 16: eight lane partials e[k] + e[k+8], then left to right.
__device__ __forceinline__ float ordered_sum16(const float (&e)[16]) {
    float r = __fadd_rn(e[0], e[8]);
#pragma unroll
    for (int k = 1; k < 8; ++k) r = __fadd_rn(r, __fadd_rn(e[k], e[k + 8]));
    return r;
}

__device__ __forceinline__ float max16(const float (&e)[16]) {
    float m = e[0];
#pragma unroll
    for (int k = 1; k < 16; ++k) m = fmaxf(m, e[k]);
    return m;
}

// How the 32 lanes of a warp map onto blocks of Y, and which lanes share a 16x16 block.
template <bool TWO_D, bool TRANSPOSED>
struct LaneMap {
    // lanes that hold the 16 rows of one 16x16 block differ exactly in these bits
    static constexpr int XOR0 = TRANSPOSED ? 1 : 2;
    __device__ static int row_in_tile(int warp, int lane) {
        if (TRANSPOSED) return (warp & 3) * 32 + lane;
        return TWO_D ? (warp >> 1) * 16 + (lane >> 1) : warp * 8 + (lane >> 2);
    }
    __device__ static int cb_in_tile(int warp, int lane) {
        if (TRANSPOSED) return warp >> 2;
        return TWO_D ? (warp & 1) * 2 + (lane & 1) : lane & 3;
    }
    // 2-D only: which of the warp's two 16x16 blocks the lane belongs to, and its row there
    __device__ static int slot(int lane) { return TRANSPOSED ? lane >> 4 : lane & 1; }
    __device__ static int row16(int lane) { return TRANSPOSED ? lane & 15 : lane >> 1; }
};

template <bool TWO_D, bool TRANSPOSED>
__device__ __forceinline__ float block_max(float m) {
    if (TWO_D) {
#pragma unroll
        for (int s = 0; s < 4; ++s) m = fmaxf(m, __shfl_xor_sync(FULL, m, LaneMap<TWO_D, TRANSPOSED>::XOR0 << s));
    }
    return m;
}

// Error of a whole block from per-element terms. 1-D: the thread's own 16 terms. 2-D: the
// 256 terms of a 16x16 block, reduced in the order of an eager sum over a row of 256
// (32 vectors of 8 lanes, four interleaved accumulators, lanes added left to right);
// `scratch` is this warp's 2 x 256 floats of shared memory.
template <bool TWO_D, bool TRANSPOSED>
__device__ __forceinline__ float block_error(const float (&e)[16], int rule, float *scratch, int lane) {
    if (!TWO_D) return rule == FOS_RULE_ABS_MAX ? max16(e) : ordered_sum16(e);
    using LM = LaneMap<TWO_D, TRANSPOSED>;
    if (rule == FOS_RULE_ABS_MAX) return block_max<TWO_D, TRANSPOSED>(max16(e));
    float4 *row = reinterpret_cast<float4 *>(scratch + LM::slot(lane) * 256 + LM::row16(lane) * 16);
    row[0] = make_float4(e[0], e[1], e[2], e[3]);
    row[1] = make_float4(e[4], e[5], e[6], e[7]);
    row[2] = make_float4(e[8], e[9], e[10], e[11]);
    row[3] = make_float4(e[12], e[13], e[14], e[15]);
    __syncwarp();
    const int s = lane >> 4, k = lane & 15;
    float lane_sum = 0.0f;
    if (k < 8) {
        const float *t = scratch + s * 256;
        float a0 = t[k], a1 = t[k + 8], a2 = t[16 + k], a3 = t[16 + k + 8];
#pragma unroll
        for (int m = 1; m < 8; ++m) {
            a0 = __fadd_rn(a0, t[(2 * m) * 16 + k]);
            a1 = __fadd_rn(a1, t[(2 * m) * 16 + k + 8]);
            a2 = __fadd_rn(a2, t[(2 * m + 1) * 16 + k]);
            a3 = __fadd_rn(a3, t[(2 * m + 1) * 16 + k + 8]);
        }
        lane_sum = __fadd_rn(__fadd_rn(__fadd_rn(a0, a1), a2), a3);
    }
    float total = __shfl_sync(FULL, lane_sum, s * 16);
#pragma unroll
    for (int kk = 1; kk < 8; ++kk) total = __fadd_rn(total, __shfl_sync(FULL, lane_sum, s * 16 + kk));
    __syncwarp();
    return __shfl_sync(FULL, total, LM::slot(lane) * 16);
}

// ------------------------------------------------------------------------------------
// one block of 16 values (one row of a 16x16 block in 2-D mode)
// ------------------------------------------------------------------------------------

template <int KIND, bool TWO_D, bool TRANSPOSED>
__device__ __forceinline__ void quantize_block(const float (&v)[16], float amax, int rule, bool exact_only,
                                               float *scratch, int lane, uint32_t &lo, uint32_t &hi,
                                               uint32_t &sf_byte) {
    float bmax = 0.0f;
#pragma unroll
    for (int i = 0; i < 16; ++i) bmax = fmaxf(bmax, fabsf(v[i]));
    bmax = block_max<TWO_D, TRANSPOSED>(bmax);

    const float maxq = (KIND == KIND_STATIC && rule == FOS_RULE_STATIC_4) ? 4.0f : 6.0f;
    const float maxsf = (KIND == KIND_ADAPTIVE) ? 256.0f : 448.0f;
    const float range = maxq * maxsf;
    const float encode = __fdiv_rn(range, amax);
    const float decode = __frcp_rn(encode);
    float hp = (amax == 0.0f) ? 0.0f : __fmul_rn(__fdiv_rn(bmax, maxq), encode);

    const uint32_t sfb_a = cvt_e4m3(hp);
    const float s_a = e4m3_to_float(sfb_a);
    const float r_a = __frcp_rn(__fmul_rn(decode, s_a));

    if (KIND == KIND_STATIC) {
        lo = hi = 0u;
        if (s_a != 0.0f) encode_e2m1(v, r_a, r_a < 0x1p-16f, lo, hi);
        sf_byte = sfb_a;
        return;
    }

    if (KIND == KIND_ADAPTIVE) {
        const uint32_t sfb_b = cvt_e4m3(__fmul_rn(hp, 1.5f));
        const float s_b = e4m3_to_float(sfb_b);
        const float r_b = __frcp_rn(__fmul_rn(decode, s_b));

        // Fast pre-filter (1-D blocks, mean-squared error, both scales normal E4M3 numbers,
        // no underflow in sight). With g = scale * amax / 1536, the reference's dequantized
        // value is q*g up to 5 ulp, |q*g| <= 6g and |d| <= 1.01g, so each estimated sum is
        // within 1500 * 2^-24 * g^2 of the reference's sum (see the derivation in the design
        // notes); 2^-13 * (g4^2 + g6^2) leaves a 25% margin on top of both.
        if (!TWO_D && rule == FOS_RULE_MSE && !exact_only && sfb_a >= 8u && sfb_b >= 8u &&
            amax > 0x1p-100f && amax < 0x1p100f && r_a >= 0x1p-16f && r_b >= 0x1p-16f) {
            const float inv = 1.0f / 1536.0f;
            const float g_a = s_a * amax * inv, g_b = s_b * amax * inv;
            uint32_t ca[2], cb[2];
            float acc_a = 0.0f, acc_b = 0.0f;
#pragma unroll
            for (int w = 0; w < 2; ++w) {
                float xa[8], xb[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    xa[i] = __fmul_rn(v[8 * w + i], r_a);
                    xb[i] = __fmul_rn(v[8 * w + i], r_b);
                }
                ca[w] = cvt_e2m1x8(xa);
                cb[w] = cvt_e2m1x8(xb);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    float2 qa = e2m1x2_to_float2((ca[w] >> (8 * j)) & 0xffu);
                    float2 qb = e2m1x2_to_float2((cb[w] >> (8 * j)) & 0xffu);
                    float d;
                    d = fmaf(qa.x, g_a, -v[8 * w + 2 * j]);     acc_a = fmaf(d, d, acc_a);
                    d = fmaf(qa.y, g_a, -v[8 * w + 2 * j + 1]); acc_a = fmaf(d, d, acc_a);
                    d = fmaf(qb.x, g_b, -v[8 * w + 2 * j]);     acc_b = fmaf(d, d, acc_b);
                    d = fmaf(qb.y, g_b, -v[8 * w + 2 * j + 1]); acc_b = fmaf(d, d, acc_b);
                }
            }
            const float tau = 0x1p-13f * (g_a * g_a + g_b * g_b);
            const float diff = acc_b - acc_a;
            if (fabsf(diff) > tau) {
                const bool pick_b = diff < 0.0f;
                lo = pick_b ? cb[0] : ca[0];
                hi = pick_b ? cb[1] : ca[1];
                sf_byte = pick_b ? sfb_b : sfb_a;
                return;
            }
        }

        uint32_t lo_a = 0u, hi_a = 0u, lo_b = 0u, hi_b = 0u;
        if (s_a != 0.0f) encode_e2m1(v, r_a, true, lo_a, hi_a);
        if (s_b != 0.0f) encode_e2m1(v, r_b, true, lo_b, hi_b);
        float e[16];
        exact_error_terms<false>(v, lo_b, hi_b, s_b, amax, 1536.0f, rule, e);
        const float err_b = block_error<TWO_D, TRANSPOSED>(e, rule, scratch, lane);
        exact_error_terms<false>(v, lo_a, hi_a, s_a, amax, 1536.0f, rule, e);
        const float err_a = block_error<TWO_D, TRANSPOSED>(e, rule, scratch, lane);
        const bool pick_b = err_b < err_a;
        lo = pick_b ? lo_b : lo_a;
        hi = pick_b ? hi_b : hi_a;
        sf_byte = pick_b ? sfb_b : sfb_a;
        return;
    }

    // IF4: one scale; E2M1 grid versus INT4 grid scaled by 6/7
    uint32_t lo_f = 0u, hi_f = 0u, lo_i = 0u, hi_i = 0u;
    if (s_a != 0.0f) {
        encode_e2m1(v, r_a, true, lo_f, hi_f);
        encode_int4(v, r_a, lo_i, hi_i);
    }
    float e[16];
    exact_error_terms<false>(v, lo_f, hi_f, s_a, amax, 2688.0f, rule, e);
    const float err_f = block_error<TWO_D, TRANSPOSED>(e, rule, scratch, lane);
    exact_error_terms<true>(v, lo_i, hi_i, s_a, amax, 2688.0f, rule, e);
    const float err_i = block_error<TWO_D, TRANSPOSED>(e, rule, scratch, lane);
    const bool pick_int = err_i < err_f;
    lo = pick_int ? lo_i : lo_f;
    hi = pick_int ? hi_i : hi_f;
    sf_byte = sfb_a + (pick_int ? 128u : 0u);
}

// ------------------------------------------------------------------------------------
// the tile kernel
// ------------------------------------------------------------------------------------


template <typename T, int KIND, bool TWO_D, bool TRANSPOSED>
__global__ void __launch_bounds__(CTA_THREADS) quantize_kernel(const QuantParams p) {
    constexpr int SMEM_BYTES = TWO_D ? 32768 : (TRANSPOSED ? 16384 : 16);
    __shared__ __align__(16) unsigned char smem[SMEM_BYTES];
    using LM = LaneMap<TWO_D, TRANSPOSED>;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t tile_r = blockIdx.y, tile_c = blockIdx.x;
    const int64_t row = tile_r * TILE_ROWS + LM::row_in_tile(warp, lane);   // row of Y
    const int64_t cb = tile_c * (TILE_COLS / 16) + LM::cb_in_tile(warp, lane);
    const int64_t col0 = cb * 16;                                            // column of Y
    const T *x = static_cast<const T *>(p.x);

    float v[16];
    if (!TRANSPOSED) {
        const bool row_ok = row < p.out_rows;
        if (row_ok && col0 + 16 <= p.out_cols && p.vec_bytes != 0) {
            uint32_t w[8];
            const T *src = x + row * p.ld + col0;
            if (p.vec_bytes == 32) {
                ldg_nc_32(src, w);
            } else {
                uint4 a = ldg_nc_16(src), b = ldg_nc_16(src + 8);
                w[0] = a.x; w[1] = a.y; w[2] = a.z; w[3] = a.w;
                w[4] = b.x; w[5] = b.y; w[6] = b.z; w[7] = b.w;
            }
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                float2 f = unpack2<T>(w[k]);
                v[2 * k] = f.x;
                v[2 * k + 1] = f.y;
            }
        } else {
#pragma unroll
            for (int i = 0; i < 16; ++i)
                v[i] = (row_ok && col0 + i < p.out_cols) ? elem_to_float<T>(x[row * p.ld + col0 + i]) : 0.0f;
        }
    } else {
        // Y[row, col] = x[col, row]: stage x[tile_c*64 .. +63][tile_r*128 .. +127] in shared memory
        T *stage = reinterpret_cast<T *>(smem);
        const int64_t src_r0 = tile_c * TILE_COLS, src_c0 = tile_r * TILE_ROWS;
        for (int chunk = threadIdx.x; chunk < 64 * 16; chunk += CTA_THREADS) {
            const int sr = chunk >> 4, sc = (chunk & 15) * 8;
            const int64_t gr = src_r0 + sr, gc = src_c0 + sc;
            uint4 w = make_uint4(0u, 0u, 0u, 0u);
            if (gr < p.rows) {
                if (gc + 8 <= p.cols && p.vec_bytes != 0) {
                    w = ldg_nc_16(x + gr * p.ld + gc);
                } else {
                    __align__(16) T tmp[8];
#pragma unroll
                    for (int i = 0; i < 8; ++i) tmp[i] = (gc + i < p.cols) ? x[gr * p.ld + gc + i] : T(0.0f);
                    w = *reinterpret_cast<uint4 *>(tmp);
                }
            }
            *reinterpret_cast<uint4 *>(stage + sr * 128 + sc) = w;
        }
        __syncthreads();
        const int jr = LM::row_in_tile(warp, lane), b = LM::cb_in_tile(warp, lane);
#pragma unroll
        for (int i = 0; i < 16; ++i) v[i] = elem_to_float<T>(stage[(b * 16 + i) * 128 + jr]);
        if (TWO_D) __syncthreads();  // the staging area is reused as reduction scratch
    }
    // -0.0 inputs count as +0.0 (sign() of a zero is zero in the reference)
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = __fadd_rn(v[i], 0.0f);

    float *scratch = TWO_D ? reinterpret_cast<float *>(smem) + warp * 512 : nullptr;
    const float amax = __ldg(p.amax);
    uint32_t lo, hi, sf_byte;
    quantize_block<KIND, TWO_D, TRANSPOSED>(v, amax, p.rule, p.exact_only != 0, scratch, lane, lo, hi, sf_byte);

    // rows_p / cols_p are multiples of the tile, so every thread owns a valid output block
    *reinterpret_cast<uint2 *>(p.codes + row * (p.cols_p >> 1) + cb * 8) = make_uint2(lo, hi);
    p.sf[sf_offset(row, cb, p.cols_p >> 4, p.sf_tiled != 0)] = static_cast<uint8_t>(sf_byte);
}

template <typename T, int KIND>
cudaError_t launch_kind(const QuantParams &p, bool two_d, bool transposed, cudaStream_t stream) {
    dim3 grid(static_cast<unsigned>(p.cols_p / TILE_COLS), static_cast<unsigned>(p.rows_p / TILE_ROWS));
    if (two_d && transposed) quantize_kernel<T, KIND, true, true><<<grid, CTA_THREADS, 0, stream>>>(p);
    else if (two_d) quantize_kernel<T, KIND, true, false><<<grid, CTA_THREADS, 0, stream>>>(p);
    else if (transposed) quantize_kernel<T, KIND, false, true><<<grid, CTA_THREADS, 0, stream>>>(p);
    else quantize_kernel<T, KIND, false, false><<<grid, CTA_THREADS, 0, stream>>>(p);
    return cudaGetLastError();
}

template <typename T>
cudaError_t launch_all(const QuantParams &p, int kind, bool two_d, bool transposed, cudaStream_t stream) {
    if (kind == KIND_STATIC) return launch_kind<T, KIND_STATIC>(p, two_d, transposed, stream);
    if (kind == KIND_ADAPTIVE) return launch_kind<T, KIND_ADAPTIVE>(p, two_d, transposed, stream);
    return launch_kind<T, KIND_IF4>(p, two_d, transposed, stream);
}

template <typename T>
cudaError_t launch_amax(const void *x, int64_t rows, int64_t cols, int64_t ld, bool vec16, float *amax,
                        cudaStream_t stream) {
    const int64_t work = vec16 ? rows * (cols >> 3) : rows * cols;
    int64_t blocks = (work + 255) / 256;
    const int64_t cap = 148 * 8;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    amax_kernel<T><<<static_cast<unsigned>(blocks), 256, 0, stream>>>(static_cast<const T *>(x), rows, cols, ld,
                                                                     vec16 ? 1 : 0, amax);
    return cudaGetLastError();
}

}  // namespace
}  // namespace fos

extern "C" int fos_quantize(const void *x, int x_dtype, int64_t rows, int64_t cols, int64_t ld, int format,
                            int scale_rule, int block_2d, int transpose, int sf_layout, const float *amax_in,
                            uint8_t *codes, uint8_t *sf, float *amax_out, int flags, void *stream_) {
    using namespace fos;
    if (!x || !codes || !sf || !amax_out) return FOS_ERR_INVALID_ARGUMENT;
    if (rows <= 0 || cols <= 0 || ld < cols) return FOS_ERR_INVALID_ARGUMENT;
    if (x_dtype != FOS_BF16 && x_dtype != FOS_FP16) return FOS_ERR_INVALID_ARGUMENT;
    if (format != FOS_NVFP4 && format != FOS_IF4) return FOS_ERR_INVALID_ARGUMENT;
    if (scale_rule < FOS_RULE_STATIC_6 || scale_rule > FOS_RULE_ABS_MAX) return FOS_ERR_INVALID_ARGUMENT;
    if (sf_layout != FOS_SF_ROWMAJOR && sf_layout != FOS_SF_TILED) return FOS_ERR_INVALID_ARGUMENT;
    const bool is_static = scale_rule == FOS_RULE_STATIC_6 || scale_rule == FOS_RULE_STATIC_4;
    if (format == FOS_IF4 && is_static) return FOS_ERR_UNSUPPORTED;
    if (reinterpret_cast<uintptr_t>(codes) % 8 != 0) return FOS_ERR_MISALIGNED;
    int st = check_device();
    if (st != FOS_OK) return st;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);

    QuantParams p{};
    p.x = x;
    p.rows = rows; p.cols = cols; p.ld = ld;
    p.out_rows = transpose ? cols : rows;
    p.out_cols = transpose ? rows : cols;
    p.rows_p = round_up64(p.out_rows, TILE_ROWS);
    p.cols_p = round_up64(p.out_cols, TILE_COLS);
    if (p.rows_p / TILE_ROWS > 65535) return FOS_ERR_TOO_LARGE;
    p.codes = codes; p.sf = sf;
    p.rule = scale_rule;
    p.sf_tiled = sf_layout == FOS_SF_TILED;
    p.exact_only = (flags & FOS_QUANTIZE_EXACT_ONLY) != 0;
    const uintptr_t addr = reinterpret_cast<uintptr_t>(x);
    const int64_t ld_bytes = ld * 2;
    p.vec_bytes = (addr % 32 == 0 && ld_bytes % 32 == 0) ? 32 : ((addr % 16 == 0 && ld_bytes % 16 == 0) ? 16 : 0);
    const bool vec16 = p.vec_bytes != 0 && cols % 8 == 0;

    if (amax_in) {
        if (amax_in != amax_out)
            FOS_CUDA_TRY(cudaMemcpyAsync(amax_out, amax_in, sizeof(float), cudaMemcpyDeviceToDevice, stream));
    } else {
        FOS_CUDA_TRY(cudaMemsetAsync(amax_out, 0, sizeof(float), stream));
        FOS_CUDA_TRY(x_dtype == FOS_BF16
                         ? launch_amax<__nv_bfloat16>(x, rows, cols, ld, vec16, amax_out, stream)
                         : launch_amax<__half>(x, rows, cols, ld, vec16, amax_out, stream));
    }
    p.amax = amax_out;

    const int kind = format == FOS_IF4 ? KIND_IF4 : (is_static ? KIND_STATIC : KIND_ADAPTIVE);
    FOS_CUDA_TRY(x_dtype == FOS_BF16
                     ? launch_all<__nv_bfloat16>(p, kind, block_2d != 0, transpose != 0, stream)
                     : launch_all<__half>(p, kind, block_2d != 0, transpose != 0, stream));
    return FOS_OK;
}
