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
#include "fos_tcgen05.cuh"
#include "fos_dequant.cuh"

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
    const float *amax;           // device, final by the time the quantize kernel reads it
    float *amax_store;           // where the quantize kernel copies amax to, or null
    uint8_t *codes;
    uint8_t *sf;
    int rule;
    int sf_tiled;
    int exact_only;
    int vec_bytes;               // 32, 16 or 0: widest aligned load usable on x
    int variant;                 // 0: kernel chosen by the input; 1: never a TMA-fed kernel (FOS_QUANTIZE_NO_TMA);
                                 // 2: the general TMA-fed kernel where a specialised one exists (FOS_QUANTIZE_GENERAL_KERNEL)
    int x_is_ready;              // x was complete before the previous kernel in the stream started
    int rht;                     // rotate every block of 16 (random Hadamard transform) before quantizing
    int stochastic;              // stochastic rounding (1-D blocks, NVFP4, TMA-fed kernels only)
    int unbiased;                // with it: every maximum is scaled by 16/17 (RoundStyle.stochastic_unbiased)
    uint32_t seed_lo, seed_hi;
    // fused fake quantization (quantize_rows_tma_kernel<.., true>): dequantized values instead of codes
    void *fake_out;              // [rows][fake_ld] elements of x's type
    int64_t fake_ld;
    float fake_divisor;
    // grouped launch (TMA-fed row kernels, grid.y = group): group g is rows group_start[g] .. group_start[g + 1]
    // (device values, multiples of 128) of x and of the outputs, quantized as a tensor of its own with amax[g]
    const int32_t *group_start;
    int num_groups;
};


// ------------------------------------------------------------------------------------
// per-tensor amax
// ------------------------------------------------------------------------------------

template <typename T>
__device__ __forceinline__ float abs_max8(uint4 w) {
    float2 a = unpack2<T>(w.x), b = unpack2<T>(w.y), c = unpack2<T>(w.z), d = unpack2<T>(w.w);
    return fmaxf(fmaxf(fmaxf(fabsf(a.x), fabsf(a.y)), fmaxf(fabsf(b.x), fabsf(b.y))),
                 fmaxf(fmaxf(fabsf(c.x), fabsf(c.y)), fmaxf(fabsf(d.x), fabsf(d.y))));
}

// Sets the amax word to zero. A kernel rather than a memset so that the chain "previous kernel ->
// this -> amax pass -> quantize kernel" consists of kernels only and every link can be a
// programmatic dependent launch: this kernel may be scheduled while the previous one drains, it
// waits for that kernel's completion (amax_out may still be read by it, and x may be written by
// it), and only then lets the amax pass start.
__global__ void zero_amax_kernel(float *amax) {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (threadIdx.x == 0) *amax = 0.0f;
}

// max |x| of the chunks (VB bytes each) that one thread owns: 128 bytes per thread in flight per
// round, every load of a round predicated (a chunk past the end contributes 0), so that there is
// no serial tail of single loads, each of which would cost a full memory latency.
template <typename T, int VB>
__device__ __forceinline__ float amax_chunks(const T *__restrict__ x, int64_t rows, int64_t cols, int64_t ld,
                                             int64_t tid, int64_t stride) {
    constexpr int EL = VB / 2, N = 128 / VB;
    const int64_t chunks_per_row = cols / EL, total = rows * chunks_per_row;
    const bool flat = ld == cols;
    float m = 0.0f;
    for (int64_t i = tid; i < total; i += N * stride) {
        uint32_t w[N][VB / 4];
#pragma unroll
        for (int k = 0; k < N; ++k) {
            const int64_t idx = i + k * stride;
#pragma unroll
            for (int j = 0; j < VB / 4; ++j) w[k][j] = 0u;
            if (idx < total) {
                const int64_t r = flat ? 0 : idx / chunks_per_row;
                const T *ptr = flat ? x + idx * EL : x + r * ld + (idx - r * chunks_per_row) * EL;
                if constexpr (VB == 32) {
                    ldg_nc_32(ptr, w[k]);
                } else {
                    const uint4 v = ldg_nc_16(ptr);
                    w[k][0] = v.x; w[k][1] = v.y; w[k][2] = v.z; w[k][3] = v.w;
                }
            }
        }
#pragma unroll
        for (int k = 0; k < N; ++k)
#pragma unroll
            for (int j = 0; j < VB / 16; ++j)
                m = fmaxf(m, abs_max8<T>(make_uint4(w[k][4 * j], w[k][4 * j + 1], w[k][4 * j + 2], w[k][4 * j + 3])));
    }
    return m;
}

// max |x| with 32-byte (or 16-byte) loads, 128 bytes in flight per thread, then one atomicMax per CTA.
// Launched behind zero_amax_kernel as its programmatic dependent: CTAs of this kernel exist only
// after that kernel has seen its predecessor complete, so x is final; the wait below makes
// the zero visible before the atomics. `vec` = 32 / 16: x's base and row stride are aligned to that
// many bytes and a row holds a whole number of such chunks; 0: element loads.
template <typename T>
__global__ void __launch_bounds__(256) amax_kernel(const T *__restrict__ x, int64_t rows, int64_t cols,
                                                   int64_t ld, int vec, float *amax) {
    float m = 0.0f;
    const int64_t tid = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    if (vec == 32) {
        m = amax_chunks<T, 32>(x, rows, cols, ld, tid, stride);
    } else if (vec == 16) {
        m = amax_chunks<T, 16>(x, rows, cols, ld, tid, stride);
    } else {
        const int64_t total = rows * cols;
        for (int64_t i = tid; i < total; i += stride) {
            int64_t r = i / cols, c = i - r * cols;
            m = fmaxf(m, fabsf(elem_to_float<T>(x[r * ld + c])));
        }
    }
    // the quantize kernel that follows may be scheduled while this grid drains (it waits for this
    // grid's completion with griddepcontrol.wait before it reads amax); signalling here rather
    // than at the top keeps its CTAs from taking SM slots this grid still needs
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
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

// One amax per group of rows: CTA (x, g) takes a share of rows group_start[g] .. + group_rows[g] and ends with an
// atomicMax on amax[g] (zeroed by the caller in the stream before the launch).
template <typename T>
__global__ void __launch_bounds__(256) amax_grouped_kernel(const T *__restrict__ x, int64_t capacity, int64_t cols, int64_t ld,
                                                           int vec, const int32_t *__restrict__ group_start,
                                                           const int32_t *__restrict__ group_rows, float *amax) {
    int64_t r0 = __ldg(group_start + blockIdx.y), rows = __ldg(group_rows + blockIdx.y);
    r0 = r0 < 0 ? 0 : (r0 > capacity ? capacity : r0);
    rows = rows < 0 ? 0 : (rows > capacity - r0 ? capacity - r0 : rows);
    const T *base = x + r0 * ld;
    const int64_t tid = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    float m = 0.0f;
    if (vec == 32) {
        m = amax_chunks<T, 32>(base, rows, cols, ld, tid, stride);
    } else if (vec == 16) {
        m = amax_chunks<T, 16>(base, rows, cols, ld, tid, stride);
    } else {
        const int64_t total = rows * cols;
        for (int64_t i = tid; i < total; i += stride) {
            const int64_t r = i / cols, c = i - r * cols;
            m = fmaxf(m, fabsf(elem_to_float<T>(base[r * ld + c])));
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(FULL, m, o));
    __shared__ float warp_max[8];
    if ((threadIdx.x & 31) == 0) warp_max[threadIdx.x >> 5] = m;
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < 8; ++w) m = fmaxf(m, warp_max[w]);
        if (m > 0.0f) atomicMax(reinterpret_cast<int *>(amax + blockIdx.y), __float_as_int(m));
    }
}

// ------------------------------------------------------------------------------------
// 16-point random Hadamard transform
// ------------------------------------------------------------------------------------

// y = v @ (diag(signs) @ H16 / 4) for the fixed sign vector of the reference
// (src/fouroversix/quantize/utils.py:19-85), as a fast Walsh-Hadamard transform in binary32 (four
// stages of 16 additions / subtractions, the same operations in the same order as the host-side
// restatement), rounded once to T like the reference's matrix product in T.
template <typename T>
__device__ __forceinline__ void rotate16(float (&v)[16]) {
    // signs: + + + - + - - - - - - + - + - -
    v[3] = -v[3]; v[5] = -v[5]; v[6] = -v[6]; v[7] = -v[7]; v[8] = -v[8]; v[9] = -v[9]; v[10] = -v[10];
    v[12] = -v[12]; v[14] = -v[14]; v[15] = -v[15];
#pragma unroll
    for (int h = 1; h < 16; h *= 2) {
#pragma unroll
        for (int base = 0; base < 16; base += 2 * h) {
#pragma unroll
            for (int k = 0; k < h; ++k) {
                const float a = v[base + k], b = v[base + h + k];
                v[base + k] = __fadd_rn(a, b);
                v[base + h + k] = __fsub_rn(a, b);
            }
        }
    }
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        const float y = __fmul_rn(v[i], 0.25f);
        if constexpr (std::is_same<T, __half>::value) v[i] = __half2float(__float2half_rn(y));
        else v[i] = __bfloat162float(__float2bfloat16_rn(y));
    }
}

// max |rotated x|: one thread per block of 16 along the rotated axis (x's rows, or x's columns when
// the tensor is quantized transposed; lanes then walk along a row of x, so loads stay coalesced).
// Same launch chain as amax_kernel.
template <typename T>
__global__ void __launch_bounds__(256) amax_rht_kernel(const T *__restrict__ x, int64_t rows, int64_t cols, int64_t ld,
                                                       int transposed, float *amax) {
    float m = 0.0f;
    const int64_t tid = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    const int64_t units = transposed ? (rows >> 4) * cols : rows * (cols >> 4);
    for (int64_t u = tid; u < units; u += stride) {
        float v[16];
        if (transposed) {
            const int64_t rb = u / cols, c = u - rb * cols;
#pragma unroll
            for (int i = 0; i < 16; ++i) v[i] = elem_to_float<T>(x[(rb * 16 + i) * ld + c]);
        } else {
            const int64_t per_row = cols >> 4, r = u / per_row, cb = u - r * per_row;
#pragma unroll
            for (int i = 0; i < 16; ++i) v[i] = elem_to_float<T>(x[r * ld + cb * 16 + i]);
        }
        rotate16<T>(v);
#pragma unroll
        for (int i = 0; i < 16; ++i) m = fmaxf(m, fabsf(v[i]));
    }
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(FULL, m, o));
    __shared__ float warp_max[8];
    if ((threadIdx.x & 31) == 0) warp_max[threadIdx.x >> 5] = m;
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < 8; ++w) m = fmaxf(m, warp_max[w]);
        atomicMax(reinterpret_cast<int *>(amax), __float_as_int(m));
    }
}

// ------------------------------------------------------------------------------------
// building blocks
// ------------------------------------------------------------------------------------

// E2M1 codes of eight scaled values v[i] * r (as encode_e2m1 without the guard) and the
// rounding residuals t[i] = q[i] - v[i] * r, each one IEEE subtraction of the binary32
// scaled value from the binary16 code value.
__device__ __forceinline__ uint32_t encode8_with_residuals(const float *v, uint64_t r2, float (&t)[8], uint64_t *scaled = nullptr) {
    float x[8];
    const uint64_t zero2 = pack2(0.0f, 0.0f);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const uint64_t xs = fma2(pack2(v[2 * k], v[2 * k + 1]), r2, zero2);
        if (scaled != nullptr) scaled[k] = xs;
        unpack2f(xs, x[2 * k], x[2 * k + 1]);
    }
    uint32_t codes;
    asm("{ .reg .b8 b0, b1, b2, b3;\n"
        ".reg .b32 h;\n"
        ".reg .f16 l, u;\n"
        "cvt.rn.satfinite.e2m1x2.f32 b0, %10, %9;\n"
        "cvt.rn.f16x2.e2m1x2 h, b0;\n"
        "mov.b32 {l, u}, h;\n"
        "sub.rn.f32.f16 %1, l, %9;\n"
        "sub.rn.f32.f16 %2, u, %10;\n"
        "cvt.rn.satfinite.e2m1x2.f32 b1, %12, %11;\n"
        "cvt.rn.f16x2.e2m1x2 h, b1;\n"
        "mov.b32 {l, u}, h;\n"
        "sub.rn.f32.f16 %3, l, %11;\n"
        "sub.rn.f32.f16 %4, u, %12;\n"
        "cvt.rn.satfinite.e2m1x2.f32 b2, %14, %13;\n"
        "cvt.rn.f16x2.e2m1x2 h, b2;\n"
        "mov.b32 {l, u}, h;\n"
        "sub.rn.f32.f16 %5, l, %13;\n"
        "sub.rn.f32.f16 %6, u, %14;\n"
        "cvt.rn.satfinite.e2m1x2.f32 b3, %16, %15;\n"
        "cvt.rn.f16x2.e2m1x2 h, b3;\n"
        "mov.b32 {l, u}, h;\n"
        "sub.rn.f32.f16 %7, l, %15;\n"
        "sub.rn.f32.f16 %8, u, %16;\n"
        "mov.b32 %0, {b0, b1, b2, b3}; }"
        : "=r"(codes), "=f"(t[0]), "=f"(t[1]), "=f"(t[2]), "=f"(t[3]), "=f"(t[4]), "=f"(t[5]), "=f"(t[6]), "=f"(t[7])
        : "f"(x[0]), "f"(x[1]), "f"(x[2]), "f"(x[3]), "f"(x[4]), "f"(x[5]), "f"(x[6]), "f"(x[7]));
    return codes;
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

// The same codes for |v * r * (7/6)| < 7.5 (no clamp needed), without float-to-int conversions:
// adding 1.5 * 2^23 rounds to the nearest integer (ties to even) and leaves it, in two's
// complement, in the low mantissa bits.
__device__ __forceinline__ void encode_int4_small(const float (&v)[16], float r, uint32_t &lo, uint32_t &hi) {
    const uint64_t r2 = pack2(r, r), zero2 = pack2(0.0f, 0.0f), one2 = pack2(1.0f, 1.0f);
    const uint64_t to_int2 = pack2(1.16666666f, 1.16666666f), magic2 = pack2(12582912.0f, 12582912.0f);
    uint32_t w[2] = {0u, 0u};
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        const uint64_t xs = fma2(pack2(v[2 * k], v[2 * k + 1]), r2, zero2);
        const uint64_t qm = fma2(fma2(xs, to_int2, zero2), one2, magic2);
        float a, b;
        unpack2f(qm, a, b);
        const uint32_t pair = (__float_as_uint(a) & 0xfu) | ((__float_as_uint(b) & 0xfu) << 4);
        w[k >> 2] |= pair << ((k & 3) * 8);
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

// Per-tensor constants: encode = (max value * max scale) / amax and decode = 1 / encode.
struct TensorConsts {
    float amax, maxq, encode, decode;
    float encode0;    // encode, or 0 when amax is 0 (every block scale is then 0)
    float block_div;  // 0: the block maximum is divided by maxq with the exact fast forms; else by this (maxq * 16/17)
    bool filter_ok;   // amax is in the range where the fast pre-filter's error bound holds
};

// `unbiased`: RoundStyle.stochastic_unbiased of the reference (src/fouroversix/utils.py:223-247): the largest
// value and the product (largest value * largest scale) are multiplied by 16/17, as Python floats, before they
// become binary32 tensors (src/fouroversix/quantize/pytorch/reference.py:203-218), which leaves the stochastically
// rounded maximum room below the clamp.
template <int KIND>
__device__ __forceinline__ TensorConsts tensor_consts(float amax, int rule, bool unbiased = false) {
    TensorConsts c;
    c.amax = amax;
    c.maxq = (KIND == KIND_STATIC && rule == FOS_RULE_STATIC_4) ? 4.0f : 6.0f;
    c.block_div = 0.0f;
    if (unbiased) {
        const float maxsf_u = (KIND == KIND_ADAPTIVE) ? 256.0f : 448.0f;
        c.block_div = static_cast<float>(static_cast<double>(c.maxq) * (16.0 / 17.0));
        c.encode = __fdiv_rn(static_cast<float>(static_cast<double>(c.maxq) * maxsf_u * (16.0 / 17.0)), amax);
        c.decode = __frcp_rn(c.encode);
        c.encode0 = amax == 0.0f ? 0.0f : c.encode;
        c.filter_ok = false;
        return c;
    }
    const float maxsf = (KIND == KIND_ADAPTIVE) ? 256.0f : 448.0f;
    c.encode = __fdiv_rn(c.maxq * maxsf, amax);
    c.decode = __frcp_rn(c.encode);
    c.encode0 = amax == 0.0f ? 0.0f : c.encode;
    c.filter_ok = amax > 0x1p-100f && amax < 0x1p100f;
    return c;
}

// What a block needs to know about a scale byte b: s = its value, r = 1 / (decode * s) as the
// reference rounds it, g = s * amax / (6 * 256) (approximate, pre-filter only) and g * g, the
// last one replaced by -1 when the fast pre-filter must not be used with this scale: the
// caller rules it out (`filter_allowed`: wrong rule, exact-only run, amax out of range), the
// scale is zero or subnormal, or r is so small that x * r can underflow.
// The 1-D kernels tabulate this once per CTA for all 128 bytes; other callers compute it.
// Which configurations have a fast pre-filter: NVFP4 4/6 with 1-D blocks for all three rules (sums of squares,
// sums of magnitudes, largest magnitude); 2-D blocks and IF4 for the mean-squared error only.
template <int KIND, bool TWO_D>
__device__ __forceinline__ bool rule_has_filter(int rule) {
    if (rule == FOS_RULE_MSE) return true;
    return KIND == KIND_ADAPTIVE && !TWO_D && (rule == FOS_RULE_MAE || rule == FOS_RULE_ABS_MAX);
}

__device__ __forceinline__ float4 scale_entry(uint32_t sfb, const TensorConsts &tc, bool filter_allowed) {
    const float s = e4m3_to_float(sfb);
    const float r = __frcp_rn(__fmul_rn(tc.decode, s));
    const float g = s * tc.amax * (1.0f / 1536.0f);
    const bool usable = filter_allowed && sfb >= 8u && r >= 0x1p-16f;
    // third field: this scale's share of the pre-filter's tolerance, 1.5 * 188u * g^2, or +infinity where the
    // pre-filter must not be used: a tolerance of infinity leaves every block undecided (quantize_rows_mse_kernel)
    return make_float4(s, r, usable ? (0x1p-24f * 1.5f * 188.0f) * (g * g) : __int_as_float(0x7f800000), usable ? g * g : -1.0f);
}

// ---- stochastic rounding (RoundStyle.stochastic) ----
//
// The reference adds uniform noise in [-0.5, 0.5) grid steps to the magnitude and then rounds to
// the nearest point of the local grid (src/fouroversix/quantize/pytorch/reference.py:39-51): step
// 0.5 below 2, 1 below 4, 2 above, the choice made on the magnitude BEFORE the noise, results
// above 6 clamped. Its random numbers come from torch's generator and cannot be reproduced, so
// parity here is in distribution (the reference's own test pins distances, tests/test_quantize.py:
// 317-388). The noise below is a counter-based hash of (seed, block, candidate, element): the
// same call with the same seed gives the same bytes.
struct StochasticArgs {
    uint32_t on;       // 0: round to nearest
    uint32_t key;      // hash of the seed and the high bits of the block number
    uint32_t block;    // low bits of the block number
};

__device__ __forceinline__ uint32_t hash32(uint32_t h) {
    h ^= h >> 16; h *= 0x7feb352du; h ^= h >> 15; h *= 0x846ca68bu; h ^= h >> 16;
    return h;
}

// Codes and quantization residuals t = q - x*r of 16 values rounded stochastically; returns sum t^2.
__device__ __forceinline__ float encode_stochastic(const float (&v)[16], float r, const StochasticArgs &sr, uint32_t candidate,
                                                   uint32_t &lo, uint32_t &hi) {
    float q[16], sum = 0.0f;
#pragma unroll
    for (int i = 0; i < 16; i += 2) {
        // one hash per pair of values: 16 random bits each, centred (the low mantissa bit set)
        const uint32_t h = hash32(sr.key ^ (sr.block * 32u + candidate * 16u + i));
#pragma unroll
        for (int k = 0; k < 2; ++k) {
            const float xs = __fmaf_rn(v[i + k], r, 0.0f);
            const float a = fabsf(xs);
            const float inv = a < 2.0f ? 2.0f : (a < 4.0f ? 1.0f : 0.5f);          // 1 / grid step at |x*r|
            const float step = a < 2.0f ? 0.5f : (a < 4.0f ? 1.0f : 2.0f);
            const uint32_t bits16 = k == 0 ? (h & 0xffffu) : (h >> 16);
            const float noise = __uint_as_float((bits16 << 7) | 0x3f800040u) - 1.5f;    // uniform in (-0.5, 0.5)
            const float steps = (__fmaf_rn(a, inv, noise) + 12582912.0f) - 12582912.0f;   // rint, ties to even
            const float mag = fminf(fmaxf(steps, 0.0f) * step, 6.0f);
            q[i + k] = copysignf(mag, xs);
            const float t = q[i + k] - xs;
            sum = __fmaf_rn(t, t, sum);
        }
    }
    lo = cvt_e2m1x8(q);          // exact: every q is a grid point
    hi = cvt_e2m1x8(q + 8);
    return sum;
}

// The integer grid of IF4 under stochastic rounding (src/fouroversix/quantize/pytorch/reference.py:55-63):
// u = (x * r) * fl(7/6), magnitude rint(|u| + noise) clamped to 7, sign of u. Returns the sum of the squared
// residuals (6/7) * q - x * r, in the same scaled units as encode_stochastic, so that the two candidates of a block
// compare directly (they share the scale).
__device__ __forceinline__ float encode_stochastic_int(const float (&v)[16], float r, const StochasticArgs &sr,
                                                       uint32_t candidate, uint32_t &lo, uint32_t &hi) {
    const float to_int = 1.16666666f, from_int = 0.8571428571f;
    uint32_t w[2] = {0u, 0u};
    float sum = 0.0f;
#pragma unroll
    for (int i = 0; i < 16; i += 2) {
        const uint32_t h = hash32(sr.key ^ (sr.block * 32u + candidate * 16u + i));
#pragma unroll
        for (int k = 0; k < 2; ++k) {
            const float xs = __fmaf_rn(v[i + k], r, 0.0f);
            const float u = __fmul_rn(xs, to_int);
            const uint32_t bits16 = k == 0 ? (h & 0xffffu) : (h >> 16);
            const float noise = __uint_as_float((bits16 << 7) | 0x3f800040u) - 1.5f;    // uniform in (-0.5, 0.5)
            const float steps = ((fabsf(u) + noise) + 12582912.0f) - 12582912.0f;       // rint, ties to even
            const float mag = fminf(fmaxf(steps, 0.0f), 7.0f);
            const float q = copysignf(mag, u);
            const float t = __fmaf_rn(q, from_int, -xs);
            sum = __fmaf_rn(t, t, sum);
            w[(i + k) >> 3] |= (static_cast<uint32_t>(static_cast<int>(q)) & 0xfu) << (((i + k) & 7) * 4);
        }
    }
    lo = w[0];
    hi = w[1];
    return sum;
}

template <int KIND, bool TWO_D, bool TRANSPOSED>
__device__ __forceinline__ void quantize_block(const float (&v)[16], const TensorConsts &tc, int rule,
                                               bool exact_only, float *scratch, int lane, const float4 *lut,
                                               float *coop, uint32_t &lo, uint32_t &hi, uint32_t &sf_byte,
                                               const StochasticArgs sr = StochasticArgs{0u, 0u, 0u}) {
    const float amax = tc.amax;
    float bmax = 0.0f;
#pragma unroll
    for (int i = 0; i < 16; ++i) bmax = fmaxf(bmax, fabsf(v[i]));
    bmax = block_max<TWO_D, TRANSPOSED>(bmax);
    const float q = tc.block_div != 0.0f ? __fdiv_rn(bmax, tc.block_div)
                                         : (tc.maxq == 6.0f ? div6_exact(bmax) : __fmul_rn(bmax, 0.25f));   // bmax / maxq
    const float hp = __fmul_rn(q, tc.encode0);
    const bool filter_allowed = !TWO_D && rule_has_filter<KIND, TWO_D>(rule) && !exact_only && tc.filter_ok;   // unused with a table

    if (KIND == KIND_STATIC) {
        const uint32_t sfb = cvt_e4m3(hp);
        const float4 ea = lut ? lut[sfb] : scale_entry(sfb, tc, false);
        lo = hi = 0u;
        if (sr.on) {
            if (ea.x != 0.0f) encode_stochastic(v, ea.y, sr, 0u, lo, hi);
        } else if (ea.x != 0.0f) {
            encode_e2m1(v, ea.y, ea.y < 0x1p-16f, lo, hi);
        }
        sf_byte = sfb;
        return;
    }

    uint32_t sfb_a, sfb_b = 0u;
    if (KIND == KIND_ADAPTIVE) {
        const uint32_t both = cvt_e4m3x2(__fmul_rn(hp, 1.5f), hp);   // "4" candidate in the upper byte
        sfb_a = both & 0xffu;
        sfb_b = both >> 8;
    } else {
        sfb_a = cvt_e4m3(hp);
    }
    const float4 ea = lut ? lut[sfb_a] : scale_entry(sfb_a, tc, filter_allowed);
    const float s_a = ea.x, r_a = ea.y;

    if (KIND == KIND_ADAPTIVE) {
        const float4 eb = lut ? lut[sfb_b] : scale_entry(sfb_b, tc, filter_allowed);
        const float s_b = eb.x, r_b = eb.y;

        if (sr.on) {
            // both candidates rounded stochastically with independent noise, the one with the smaller
            // error of THIS draw wins (mean-squared error; g = s * amax / 1536 converts to x's units)
            uint32_t lo_a = 0u, hi_a = 0u, lo_b = 0u, hi_b = 0u;
            const float ga = s_a * amax * (1.0f / 1536.0f), gb = s_b * amax * (1.0f / 1536.0f);
            const float err_a = s_a != 0.0f ? encode_stochastic(v, r_a, sr, 0u, lo_a, hi_a) * ga * ga : 0.0f;
            const float err_b = s_b != 0.0f ? encode_stochastic(v, r_b, sr, 1u, lo_b, hi_b) * gb * gb : 0.0f;
            const bool take_b = err_b < err_a;
            lo = take_b ? lo_b : lo_a;
            hi = take_b ? hi_b : hi_a;
            sf_byte = take_b ? sfb_b : sfb_a;
            return;
        }

        // Fast pre-filter: 1-D blocks, mean-squared error, both scales normal E4M3 numbers (so
        // |x*r| <= 6.4 and a rounding residual t = q - x*r is at most 1.01), amax and r in a range
        // without underflow. In units of G = s*amax/1536 the reference's error term is
        // (deq - x)/G = t + eta with |eta| <= 47 ulp(1) (two roundings in deq, five between x*r
        // and x/G, |q| <= 6, |x*r| <= 6.4), so its sum differs from G^2 * sum(t^2) by at most
        // 2 * 47u * sum|t| * G^2 <= 376u * sqrt(sum t^2) * G^2 (Cauchy-Schwarz over 16 terms)
        // <= 188u * (sum t^2 + 1) * G^2 (arithmetic over geometric mean), plus 40u relative for the
        // roundings of the two summations. `tau` is 1.5 times that, for both candidates
        // together; a difference inside tau is re-decided exactly below.
        const bool eligible = fminf(ea.w, eb.w) >= 0.0f;     // (callers without a table rule 2-D blocks out)
        bool decided = false, pick_b = false;
        uint32_t ca[2] = {0u, 0u}, cb[2] = {0u, 0u};
        float row_a = 0.0f, row_b = 0.0f;                    // 2-D: this row's share of the block's sums
        if (eligible && !TWO_D && rule != FOS_RULE_MSE) {
            // Sums of magnitudes (mae) and largest magnitude (abs_max), 1-D blocks. The reference's term is
            // |deq - x| = G * |t + eta| with the same eta as above plus the rounding of the subtraction: |eta| <= 64u
            // generously. Hence sum|t + eta| differs from sum|t| by at most 16 * 64u = 1024u and max|t + eta| from
            // max|t| by at most 64u (absolute, in units of G); the roundings of either summation, of the residuals
            // and of G itself add at most 60u relative (8u for the maximum, which is not summed).
            const uint64_t ra2 = pack2(r_a, r_a), rb2 = pack2(r_b, r_b);
            const bool is_max = rule == FOS_RULE_ABS_MAX;
            float m_a = 0.0f, m_b = 0.0f;
#pragma unroll
            for (int w = 0; w < 2; ++w) {
                float ta[8], tb[8];
                ca[w] = encode8_with_residuals(&v[8 * w], ra2, ta);
                cb[w] = encode8_with_residuals(&v[8 * w], rb2, tb);
                if (is_max) {
#pragma unroll
                    for (int k = 0; k < 8; k += 2) {     // (three-input maxima: half as many instructions on the ALU pipe)
                        m_a = fmaxf(fmaxf(m_a, fabsf(ta[k])), fabsf(ta[k + 1]));
                        m_b = fmaxf(fmaxf(m_b, fabsf(tb[k])), fabsf(tb[k + 1]));
                    }
                } else {
#pragma unroll
                    for (int k = 0; k < 8; ++k) {
                        m_a += fabsf(ta[k]);
                        m_b += fabsf(tb[k]);
                    }
                }
            }
            const float g_a = s_a * amax * (1.0f / 1536.0f), g_b = s_b * amax * (1.0f / 1536.0f);
            const float err_a = m_a * g_a, err_b = m_b * g_b;
            const float tau = is_max ? 0x1p-24f * 1.5f * (8.0f * (err_a + err_b) + 64.0f * (g_a + g_b))
                                     : 0x1p-24f * 1.5f * (60.0f * (err_a + err_b) + 1024.0f * (g_a + g_b));
            const float diff = err_b - err_a;
            decided = fabsf(diff) > tau;
            pick_b = diff < 0.0f;
        } else if (eligible) {
            const uint64_t ra2 = pack2(r_a, r_a), rb2 = pack2(r_b, r_b);
            uint64_t acc_a = pack2(0.0f, 0.0f), acc_b = acc_a;
#pragma unroll
            for (int w = 0; w < 2; ++w) {
                float ta[8], tb[8];
                ca[w] = encode8_with_residuals(&v[8 * w], ra2, ta);
                cb[w] = encode8_with_residuals(&v[8 * w], rb2, tb);
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const uint64_t pa = pack2(ta[2 * k], ta[2 * k + 1]), pb = pack2(tb[2 * k], tb[2 * k + 1]);
                    acc_a = fma2(pa, pa, acc_a);
                    acc_b = fma2(pb, pb, acc_b);
                }
            }
            float a0, a1, b0, b1;
            unpack2f(acc_a, a0, a1);
            unpack2f(acc_b, b0, b1);
            const float sum_a = a0 + a1, sum_b = b0 + b1;                 // sum of t^2, scaled units
            if (!TWO_D) {
                const float err_a = sum_a * ea.w, err_b = sum_b * eb.w;   // times G^2
                const float tau = 0x1p-24f * 1.5f * (228.0f * (err_a + err_b) + 188.0f * (ea.w + eb.w));
                const float diff = err_b - err_a;
                decided = fabsf(diff) > tau;
                pick_b = diff < 0.0f;
            } else {
                row_a = sum_a;
                row_b = sum_b;
            }
        }
        if (TWO_D) {
            // 16 x 16 blocks: the 16 lanes that hold a block's rows add their row sums (any order:
            // this is the estimate). Same per-element bound; over 256 terms Cauchy-Schwarz gives
            // 2 * 47u * 16 * sqrt(S) <= 752u * (S + 1), and 100u covers the roundings of both
            // 256-term summations. The block's lanes share the scales, so `eligible` is uniform
            // over them. The exact path below is collective over the warp (shared scratch), so it
            // is taken by the whole warp as soon as one of its two blocks needs it.
#pragma unroll
            for (int sh = 0; sh < 4; ++sh) {
                row_a += __shfl_xor_sync(FULL, row_a, LaneMap<TWO_D, TRANSPOSED>::XOR0 << sh);
                row_b += __shfl_xor_sync(FULL, row_b, LaneMap<TWO_D, TRANSPOSED>::XOR0 << sh);
            }
            const float err_a = row_a * ea.w, err_b = row_b * eb.w;
            const float tau = 0x1p-24f * 1.5f * (852.0f * (err_a + err_b) + 752.0f * (ea.w + eb.w));
            const float diff = err_b - err_a;
            pick_b = diff < 0.0f;
            decided = __all_sync(FULL, eligible && fabsf(diff) > tau);
        }

        // Undecided blocks are re-decided with the reference's exact sequence. When the caller
        // provides a per-warp exchange buffer (and calls this function from converged code) the
        // whole warp works on one such block at a time: lane 16c+i evaluates element i under
        // candidate c, and the 16 terms are added in the reference's order with shuffles. That
        // costs the warp about 60 instructions per undecided block instead of running the
        // 16-element exact loop on every lane of a diverged warp.
        if (!TWO_D && coop != nullptr) {
            unsigned pending = __ballot_sync(FULL, eligible && !decided);
            while (pending) {
                const int src = __ffs(pending) - 1;
                pending &= pending - 1;
                if (lane == src) {
                    float4 *x4 = reinterpret_cast<float4 *>(coop);
                    x4[0] = make_float4(v[0], v[1], v[2], v[3]);
                    x4[1] = make_float4(v[4], v[5], v[6], v[7]);
                    x4[2] = make_float4(v[8], v[9], v[10], v[11]);
                    x4[3] = make_float4(v[12], v[13], v[14], v[15]);
                    x4[4] = make_float4(s_a, r_a, s_b, r_b);
                }
                __syncwarp();
                const int cand = lane >> 4, i = lane & 15;
                const float x = coop[i];
                const float s = coop[16 + 2 * cand], r = coop[17 + 2 * cand];
                const float2 q = e2m1x2_to_float2(cvt_e2m1x2(0.0f, __fmaf_rn(x, r, 0.0f)));
                const float d = __fsub_rn(__fdiv_rn(__fmul_rn(__fmul_rn(q.x, s), amax), 1536.0f), x);
                const float e = rule == FOS_RULE_MSE ? __fmul_rn(d, d) : fabsf(d);
                float total;
                if (rule == FOS_RULE_ABS_MAX) {
                    total = e;                                                   // maximum over the candidate's 16 lanes
#pragma unroll
                    for (int o = 8; o > 0; o >>= 1) total = fmaxf(total, __shfl_xor_sync(FULL, total, o));
                } else {
                    const float p = __fadd_rn(e, __shfl_down_sync(FULL, e, 8));  // valid in lanes with i < 8
                    total = __shfl_sync(FULL, p, cand * 16);
#pragma unroll
                    for (int k = 1; k < 8; ++k) total = __fadd_rn(total, __shfl_sync(FULL, p, cand * 16 + k));
                }
                const float exact_a = __shfl_sync(FULL, total, 0), exact_b = __shfl_sync(FULL, total, 16);
                if (lane == src) {
                    decided = true;
                    pick_b = exact_b < exact_a;
                }
                __syncwarp();
            }
        }
        if (eligible && decided) {
            lo = pick_b ? cb[0] : ca[0];
            hi = pick_b ? cb[1] : ca[1];
            sf_byte = pick_b ? sfb_b : sfb_a;
            return;
        }

        if (!TWO_D && s_a == 0.0f && s_b == 0.0f) {
            // an all-zero block (or one whose scales underflow to zero): nothing is encoded and both candidates
            // carry a zero scale byte, whichever wins; padding rows of grouped tensors are full of these
            lo = 0u;
            hi = 0u;
            sf_byte = sfb_a;
            return;
        }
        uint32_t lo_a = 0u, hi_a = 0u, lo_b = 0u, hi_b = 0u;
        if (s_a != 0.0f) encode_e2m1(v, r_a, true, lo_a, hi_a);
        if (s_b != 0.0f) encode_e2m1(v, r_b, true, lo_b, hi_b);
        float e[16];
        exact_error_terms<false>(v, lo_b, hi_b, s_b, amax, 1536.0f, rule, e);
        const float err_b = block_error<TWO_D, TRANSPOSED>(e, rule, scratch, lane);
        exact_error_terms<false>(v, lo_a, hi_a, s_a, amax, 1536.0f, rule, e);
        const float err_a = block_error<TWO_D, TRANSPOSED>(e, rule, scratch, lane);
        pick_b = err_b < err_a;
        lo = pick_b ? lo_b : lo_a;
        hi = pick_b ? hi_b : hi_a;
        sf_byte = pick_b ? sfb_b : sfb_a;
        return;
    }

    // IF4: one scale; E2M1 grid versus INT4 grid scaled by 6/7.
    //
    // Fast pre-filter, as for NVFP4 (same conditions, from the same table entry), in units of
    // G = s * amax / 2688. Float grid: the reference's term is t_f + eta, t_f = q_f - x*r,
    // |eta| <= 47u as above. Integer grid: q_i = rint(u), u = (x*r) * fl(7/6), |u| < 7.5 whenever
    // |x*r| <= 6.42 (checked), so no clamp; with d = q_i - u (exact: a multiple of ulp(u) below 1)
    // the reference's term ((q_i * s) * amax * fl(6/7)) / 2688 - x is (6/7) * d + eta_i in units
    // of G with |eta_i| <= 24u (three roundings and the constant, |deq| <= 6 G) + 45u (x*r against
    // x/G: five roundings, the constant 7/6 and one product, |x*r| <= 6.4) + 1u < 80u. Hence
    // err_i differs from (6/7)^2 * sum(d^2) * G^2 by at most 2 * 80u * sum|t| <= 640u * sqrt(S_i)
    // <= 320u * (S_i + 1), plus 40u relative for the summations; likewise 188u * (S_f + 1) + 40u.
    // The two candidates share G, so the comparison is made on S_i and S_f themselves.
    if (KIND == KIND_IF4 && sr.on) {
        // both grids rounded stochastically with independent noise; the grid with the smaller squared error of THIS
        // draw wins (the candidates share the scale, so the sums compare as they are)
        uint32_t lo_f = 0u, hi_f = 0u, lo_i = 0u, hi_i = 0u;
        bool take_int = false;
        if (s_a != 0.0f) {
            const float err_f = encode_stochastic(v, r_a, sr, 0u, lo_f, hi_f);
            const float err_i = encode_stochastic_int(v, r_a, sr, 1u, lo_i, hi_i);
            take_int = err_i < err_f;
        }
        lo = take_int ? lo_i : lo_f;
        hi = take_int ? hi_i : hi_f;
        sf_byte = sfb_a | (take_int ? 0x80u : 0u);
        return;
    }
    const bool if4_eligible = KIND == KIND_IF4 && ea.w >= 0.0f && __fmul_rn(bmax, r_a) <= 6.42f;
    bool if4_decided = false, pick_int_fast = false;
    float row_f = 0.0f, row_i = 0.0f;                  // 2-D: this row's share of the block's sums
    uint32_t cf[2] = {0u, 0u};
    if (if4_eligible) {
        const uint64_t r2 = pack2(r_a, r_a), zero2 = pack2(0.0f, 0.0f), one2 = pack2(1.0f, 1.0f), minus2 = pack2(-1.0f, -1.0f);
        const uint64_t to_int2 = pack2(1.16666666f, 1.16666666f), magic2 = pack2(12582912.0f, 12582912.0f);
        const uint64_t unmagic2 = pack2(-12582912.0f, -12582912.0f);
        uint64_t acc_f = zero2, acc_i = zero2;
#pragma unroll
        for (int w = 0; w < 2; ++w) {
            float tf[8];
            uint64_t xs[4];
            cf[w] = encode8_with_residuals(&v[8 * w], r2, tf, xs);
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const uint64_t pf = pack2(tf[2 * k], tf[2 * k + 1]);
                acc_f = fma2(pf, pf, acc_f);
                const uint64_t u = fma2(xs[k], to_int2, zero2);                    // (x*r) * fl(7/6), as the reference rounds it
                const uint64_t q = fma2(fma2(u, one2, magic2), one2, unmagic2);    // rint(u), ties to even
                const uint64_t d = fma2(u, minus2, q);                            // q - u, exact
                acc_i = fma2(d, d, acc_i);
            }
        }
        float f0, f1, i0, i1;
        unpack2f(acc_f, f0, f1);
        unpack2f(acc_i, i0, i1);
        const float from_int = 0.8571428571f;
        float s_f = f0 + f1, s_i = (i0 + i1) * (from_int * from_int);
        if (!TWO_D) {
            const float tau = 0x1p-24f * 1.5f * (360.0f * s_i + 228.0f * s_f + 508.0f);
            const float diff = s_i - s_f;
            if4_decided = fabsf(diff) > tau;
            pick_int_fast = diff < 0.0f;
        } else {
            row_f = s_f;
            row_i = s_i;
        }
    }
    if (KIND == KIND_IF4 && TWO_D) {
        // 16 x 16 blocks: the 16 lanes that hold a block's rows add their row sums (any order: this is the estimate).
        // Same per-element bounds over 256 terms: 2 * 80u * 16 * sqrt(S_i) <= 1280u * (S_i + 1) and
        // 2 * 47u * 16 * sqrt(S_f) <= 752u * (S_f + 1), plus 100u relative for the roundings of the 256-term
        // summations. The block's lanes share the scale, so eligibility is uniform over them; the exact path below
        // is collective over the warp, so it is taken by the whole warp as soon as one of its two blocks needs it.
#pragma unroll
        for (int sh = 0; sh < 4; ++sh) {
            row_f += __shfl_xor_sync(FULL, row_f, LaneMap<TWO_D, TRANSPOSED>::XOR0 << sh);
            row_i += __shfl_xor_sync(FULL, row_i, LaneMap<TWO_D, TRANSPOSED>::XOR0 << sh);
        }
        const float tau = 0x1p-24f * 1.5f * (1380.0f * row_i + 852.0f * row_f + 2032.0f);
        const float diff = row_i - row_f;
        pick_int_fast = diff < 0.0f;
        if4_decided = __all_sync(FULL, if4_eligible && fabsf(diff) > tau);
    }
    // undecided blocks (ties, mostly): the whole warp evaluates one block at a time exactly, lane
    // 16c + i taking element i under candidate c (0: float grid, 1: integer grid), as for NVFP4
    if (KIND == KIND_IF4 && !TWO_D && coop != nullptr) {
        unsigned pending = __ballot_sync(FULL, if4_eligible && !if4_decided);
        while (pending) {
            const int src = __ffs(pending) - 1;
            pending &= pending - 1;
            if (lane == src) {
                float4 *x4 = reinterpret_cast<float4 *>(coop);
                x4[0] = make_float4(v[0], v[1], v[2], v[3]);
                x4[1] = make_float4(v[4], v[5], v[6], v[7]);
                x4[2] = make_float4(v[8], v[9], v[10], v[11]);
                x4[3] = make_float4(v[12], v[13], v[14], v[15]);
                x4[4] = make_float4(s_a, r_a, 0.0f, 0.0f);
            }
            __syncwarp();
            const int cand = lane >> 4, i = lane & 15;
            const float x = coop[i], s = coop[16], r = coop[17];
            const float xs = __fmaf_rn(x, r, 0.0f);
            float t;
            if (cand == 0) {
                t = __fmul_rn(__fmul_rn(e2m1x2_to_float2(cvt_e2m1x2(0.0f, xs)).x, s), amax);
            } else {
                const float q = rintf(fminf(fmaxf(__fmul_rn(xs, 1.16666666f), -7.0f), 7.0f));
                t = __fmul_rn(__fmul_rn(__fmul_rn(q, s), amax), 0.8571428571f);
            }
            const float d = __fsub_rn(__fdiv_rn(t, 2688.0f), x);
            const float e = __fmul_rn(d, d);
            const float p = __fadd_rn(e, __shfl_down_sync(FULL, e, 8));          // valid in lanes with i < 8
            float total = __shfl_sync(FULL, p, cand * 16);
#pragma unroll
            for (int k = 1; k < 8; ++k) total = __fadd_rn(total, __shfl_sync(FULL, p, cand * 16 + k));
            const float exact_f = __shfl_sync(FULL, total, 0), exact_i = __shfl_sync(FULL, total, 16);
            if (lane == src) {
                if4_decided = true;
                pick_int_fast = exact_i < exact_f;
            }
            __syncwarp();
        }
    }
    if (if4_eligible && if4_decided) {
        if (pick_int_fast) {
            encode_int4_small(v, r_a, lo, hi);
            sf_byte = sfb_a + 128u;
        } else {
            lo = cf[0];
            hi = cf[1];
            sf_byte = sfb_a;
        }
        return;
    }

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

// Noise stream of one block for the stochastic rounding: keyed by the seed and the block's number.
__device__ __forceinline__ StochasticArgs stochastic_args(const QuantParams &p, int64_t block_number) {
    StochasticArgs a;
    a.on = static_cast<uint32_t>(p.stochastic);
    a.key = hash32(hash32(p.seed_hi ^ static_cast<uint32_t>(static_cast<uint64_t>(block_number) >> 27)) ^ p.seed_lo);
    a.block = static_cast<uint32_t>(block_number);
    return a;
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
    float *scratch = TWO_D ? reinterpret_cast<float *>(smem) + warp * 512 : nullptr;
    const TensorConsts tc = tensor_consts<KIND>(__ldg(p.amax), p.rule);
    if (p.amax_store != nullptr && threadIdx.x == 0 && blockIdx.x == 0 && blockIdx.y == 0) *p.amax_store = tc.amax;
    uint32_t lo, hi, sf_byte;
    if (p.rht) rotate16<T>(v);
    quantize_block<KIND, TWO_D, TRANSPOSED>(v, tc, p.rule, p.exact_only != 0, scratch, lane, nullptr, nullptr, lo, hi,
                                            sf_byte);

    // rows_p / cols_p are multiples of the tile, so every thread owns a valid output block
    *reinterpret_cast<uint2 *>(p.codes + row * (p.cols_p >> 1) + cb * 8) = make_uint2(lo, hi);
    p.sf[sf_offset(row, cb, p.cols_p >> 4, p.sf_tiled != 0)] = static_cast<uint8_t>(sf_byte);
}

// ------------------------------------------------------------------------------------
// the common case: 1-D blocks of an untransposed tensor
// ------------------------------------------------------------------------------------
//
// Persistent CTAs of 256 threads walk over 64-row x 64-column tiles (warp w: rows 8w..8w+7;
// lane: row lane/4, block lane%4, so four lanes read one 128-byte line). The 32 bytes of
// the NEXT tile are requested before the current block is processed, which keeps a load in
// flight per thread while the arithmetic runs.

constexpr int ROWS_CTA_THREADS = 256;

// The 16 values of block (row, cb) as eight words of two 16-bit elements; zeros outside x.
template <typename T>
__device__ __forceinline__ void load_block_words(const QuantParams &p, int64_t row, int64_t cb, uint32_t (&w)[8]) {
    const T *x = static_cast<const T *>(p.x);
    const int64_t col0 = cb * 16;
    if (row < p.out_rows && col0 + 16 <= p.out_cols && p.vec_bytes != 0) {
        const T *src = x + row * p.ld + col0;
        if (p.vec_bytes == 32) {
            ldg_nc_32(src, w);
        } else {
            const uint4 a = ldg_nc_16(src), b = ldg_nc_16(src + 8);
            w[0] = a.x; w[1] = a.y; w[2] = a.z; w[3] = a.w;
            w[4] = b.x; w[5] = b.y; w[6] = b.z; w[7] = b.w;
        }
    } else {
        const uint16_t *xs = reinterpret_cast<const uint16_t *>(x);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            uint32_t lo = 0u, hi = 0u;
            if (row < p.out_rows) {
                if (col0 + 2 * k < p.out_cols) lo = xs[row * p.ld + col0 + 2 * k];
                if (col0 + 2 * k + 1 < p.out_cols) hi = xs[row * p.ld + col0 + 2 * k + 1];
            }
            w[k] = lo | (hi << 16);
        }
    }
}

template <typename T, int KIND>
__global__ void __launch_bounds__(ROWS_CTA_THREADS, KIND == KIND_STATIC ? 5 : 4)
quantize_rows_kernel(const QuantParams p) {
    __shared__ float4 lut[128];                  // scale byte -> {s, r, g, g^2}, see scale_entry()
    __shared__ __align__(16) float coop[ROWS_CTA_THREADS / 32][20];   // per warp: one block + its two scales
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tiles_c = static_cast<int>(p.cols_p >> 6), tiles_r = static_cast<int>(p.rows_p >> 6);
    const int r_in_tile = warp * 8 + (lane >> 2), cb_in_tile = lane & 3;
    const int64_t n_cb = p.cols_p >> 4;

    // tile coordinates advance by gridDim.x tiles per step without dividing inside the loop
    const int step_r = static_cast<int>(gridDim.x) / tiles_c, step_c = static_cast<int>(gridDim.x) % tiles_c;
    int tr = static_cast<int>(blockIdx.x) / tiles_c, tc_ = static_cast<int>(blockIdx.x) % tiles_c;
    if (tr >= tiles_r) return;                   // never taken: the grid has at most one CTA per tile

    uint32_t w[8];
    load_block_words<T>(p, static_cast<int64_t>(tr) * 64 + r_in_tile, tc_ * 4 + cb_in_tile, w);
    // amax comes from the previous kernel in the stream; nothing above needed it. With
    // programmatic dependent launch this CTA may be running before that kernel has finished.
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const TensorConsts tc = tensor_consts<KIND>(*reinterpret_cast<const volatile float *>(p.amax), p.rule);
    if (p.amax_store != nullptr && threadIdx.x == 0 && blockIdx.x == 0) *p.amax_store = tc.amax;
    if (threadIdx.x < 128)
        lut[threadIdx.x] = scale_entry(threadIdx.x, tc, rule_has_filter<KIND, false>(p.rule) && !p.exact_only && tc.filter_ok);
    __syncthreads();

    while (true) {
        int nr = tr + step_r, nc = tc_ + step_c;
        if (nc >= tiles_c) { nc -= tiles_c; ++nr; }
        const bool more = nr < tiles_r;
        uint32_t wn[8];
        if (more) load_block_words<T>(p, static_cast<int64_t>(nr) * 64 + r_in_tile, nc * 4 + cb_in_tile, wn);

        float v[16];
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const float2 f = unpack2<T>(w[k]);
            v[2 * k] = f.x;
            v[2 * k + 1] = f.y;
        }
        uint32_t lo, hi, sf_byte;
        if (p.rht) rotate16<T>(v);
        quantize_block<KIND, false, false>(v, tc, p.rule, p.exact_only != 0, nullptr, lane, lut, coop[warp], lo, hi, sf_byte);
        const int64_t row = static_cast<int64_t>(tr) * 64 + r_in_tile, cb = tc_ * 4 + cb_in_tile;
        *reinterpret_cast<uint2 *>(p.codes + row * (p.cols_p >> 1) + cb * 8) = make_uint2(lo, hi);
        p.sf[sf_offset(row, cb, n_cb, p.sf_tiled != 0)] = static_cast<uint8_t>(sf_byte);

        if (!more) break;
#pragma unroll
        for (int k = 0; k < 8; ++k) w[k] = wn[k];
        tr = nr;
        tc_ = nc;
    }
}


// ------------------------------------------------------------------------------------
// the common case, fed by the TMA unit
// ------------------------------------------------------------------------------------
//
// Same arithmetic and thread-to-block assignment as quantize_rows_kernel, but x arrives through a
// ring of shared-memory stages filled by bulk tensor copies: one producer thread keeps
// FEED_STAGES tiles of 128 rows x 64 columns (16 KB each) in flight per CTA whatever the
// occupancy, the copy engine zero-fills what lies outside x (so ragged shapes cost nothing), and
// the 256 consumer threads spend no instructions on global addresses or bounds. Consumer lane
// l of warp w owns rows 8w + l/4 and 64 + 8w + l/4 of the tile and block column l%4; with the
// 128-byte swizzle the two 16-byte pieces of a block sit at chunk (2*(l%4) + h) ^ (l/4) of
// the row, which makes every quarter-warp read 128 distinct bytes (no bank conflicts).
//
// Needs x 16-byte aligned with a row stride that is a multiple of 16 bytes.

constexpr int FEED_TILE_ROWS = 128;
#ifndef FOS_UNPACK_BY_ADD
#define FOS_UNPACK_BY_ADD 1
#endif


#ifndef FOS_FEED_STAGES
#define FOS_FEED_STAGES 4
#endif
#ifndef FOS_FEED_CTAS
#define FOS_FEED_CTAS 3
#endif
constexpr int FEED_STAGES = FOS_FEED_STAGES;
constexpr int FEED_STAGE_BYTES = FEED_TILE_ROWS * 128;
constexpr int FEED_CONSUMERS = 256;
constexpr int FEED_THREADS = FEED_CONSUMERS + 32;
constexpr int FEED_SMEM_BYTES = FEED_STAGES * FEED_STAGE_BYTES + 1024;

// EXTRAS: the instantiation that can rotate blocks (random Hadamard transform) and round
// stochastically; the plain one carries neither code path, which keeps its register count down.
// Grouped launch: the tile rows of group blockIdx.y and its amax word. (The row ranges come from device
// memory that earlier work in the stream wrote; grouped launches are ordinary launches, not programmatic
// dependents, so that work is complete.) Ranges are clipped to the buffers.
__device__ __forceinline__ void group_tiles(const QuantParams &p, int &tile_r0, int &tiles_r, const float *&amax_ptr) {
    const int all = static_cast<int>(p.rows_p >> 7);
    int t0 = __ldg(p.group_start + blockIdx.y) >> 7, t1 = __ldg(p.group_start + blockIdx.y + 1) >> 7;
    t0 = t0 < 0 ? 0 : (t0 > all ? all : t0);
    t1 = t1 < t0 ? t0 : (t1 > all ? all : t1);
    tile_r0 = t0;
    tiles_r = t1 - t0;
    amax_ptr += blockIdx.y;
}

template <typename T, int KIND, bool FAKE = false, bool TWO_D = false, bool EXTRAS = false>
__global__ void __launch_bounds__(FEED_THREADS, FOS_FEED_CTAS)
quantize_rows_tma_kernel(const __grid_constant__ CUtensorMap map_x, const QuantParams p) {
    static_assert(!(FAKE && TWO_D), "the fused fake quantization is built for 1-D blocks");
    extern __shared__ uint8_t feed_smem_raw[];
    __shared__ float4 lut[128];
    __shared__ __align__(16) float coop[FEED_CONSUMERS / 32][20];
    // 2-D blocks: per warp 2 x 256 floats for the exact 256-term sums of its two 16 x 16 blocks
    __shared__ __align__(16) float scratch2d[TWO_D ? (FEED_CONSUMERS / 32) * 512 : 4];
    __shared__ __align__(8) uint64_t full_bar[FEED_STAGES], empty_bar[FEED_STAGES];
    __shared__ int abort_flag;

    const uint32_t stage0 = (smem_u32(feed_smem_raw) + 1023u) & ~1023u;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tiles_c = static_cast<int>(p.cols_p >> 6);
    int tiles_r = static_cast<int>(p.rows_p >> 7), tile_r0 = 0;
    const float *amax_ptr = p.amax;
    if (!FAKE && p.group_start != nullptr) group_tiles(p, tile_r0, tiles_r, amax_ptr);
    const int64_t n_tiles = static_cast<int64_t>(tiles_c) * tiles_r;

    if (threadIdx.x == 0) {
        abort_flag = 0;
#pragma unroll
        for (int s = 0; s < FEED_STAGES; ++s) {
            mbar_init(smem_u32(&full_bar[s]), 1);
            mbar_init(smem_u32(&empty_bar[s]), FEED_CONSUMERS / 32);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    // this CTA's tiles: blockIdx.x, blockIdx.x + gridDim.x, ... in row-major tile order (of its group)
    const int step_r = static_cast<int>(gridDim.x) / tiles_c, step_c = static_cast<int>(gridDim.x) % tiles_c;
    int tr = tile_r0 + static_cast<int>(blockIdx.x) / tiles_c, tc_ = static_cast<int>(blockIdx.x) % tiles_c;
    const int my_tiles = static_cast<int>((n_tiles - blockIdx.x + gridDim.x - 1) / gridDim.x);

    if (warp == FEED_CONSUMERS / 32) {
        // ---------------- producer ----------------
        if (lane != 0) return;
        // x may be the output of the previous kernel in the stream unless the caller knows better
        if (!p.x_is_ready) asm volatile("griddepcontrol.wait;" ::: "memory");
        int issued = 0, s = 0;
        uint32_t parity = 1;   // of the "stage is free" barrier; the first round finds every stage free
        for (; issued < my_tiles; ++issued) {
            if (issued >= FEED_STAGES && !mbar_wait(smem_u32(&empty_bar[s]), parity, &abort_flag, &g_wait_failures, 1))
                break;
            mbar_expect_tx(smem_u32(&full_bar[s]), FEED_STAGE_BYTES);
            tma_load_2d(stage0 + s * FEED_STAGE_BYTES, &map_x, tc_ * 128, tr * FEED_TILE_ROWS, smem_u32(&full_bar[s]));
            if (++s == FEED_STAGES) { s = 0; parity ^= 1u; }
            tr += step_r;
            tc_ += step_c;
            if (tc_ >= tiles_c) { tc_ -= tiles_c; ++tr; }
        }
        // stay until every copy this thread issued has landed: shared memory must outlive them
        for (int j = issued > FEED_STAGES ? issued - FEED_STAGES : 0; j < issued; ++j) {
            const uint32_t bar = smem_u32(&full_bar[j % FEED_STAGES]);
            const uint32_t landed = static_cast<uint32_t>(j / FEED_STAGES) & 1u;
            const unsigned long long t0 = global_timer_ns();
            while (!mbar_try_wait(bar, landed) && global_timer_ns() - t0 < WAIT_LIMIT_NS) {}
        }
        return;
    }

    // ---------------- consumers ----------------
    // amax comes from the previous kernel in the stream; with programmatic dependent launch this
    // CTA may be running before that kernel has finished.
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const TensorConsts tc = tensor_consts<KIND>(*reinterpret_cast<const volatile float *>(amax_ptr), p.rule, EXTRAS && p.unbiased);
    if (p.amax_store != nullptr && threadIdx.x == 0 && blockIdx.x == 0) *p.amax_store = tc.amax;
    if (threadIdx.x < 128)
        lut[threadIdx.x] = scale_entry(threadIdx.x, tc, rule_has_filter<KIND, TWO_D>(p.rule) && !p.exact_only && tc.filter_ok);
    asm volatile("bar.sync 1, %0;" ::"n"(FEED_CONSUMERS) : "memory");

    // What depends on the thread alone is computed here once. The empty asm statements make these
    // values opaque, so that they stay in registers: left alone, the compiler recomputes them
    // for every block (dozens of integer instructions) to save those registers.
    // 1-D blocks: lane l of warp w owns rows 8w + l/4 and 64 + 8w + l/4 of the tile and block column l%4.
    // 2-D blocks: warp w owns rows 16w .. 16w+15 (one row per lane pair), lane l block columns l%2 and
    // 2 + l%2, so that the 16 lanes of equal parity hold the 16 rows of one 16 x 16 block.
    const int q = TWO_D ? lane >> 1 : lane >> 2, cb = TWO_D ? lane & 1 : lane & 3;
    const int row_in_tile = TWO_D ? warp * 16 + q : warp * 8 + q;
    const int64_t code_ld = p.cols_p >> 1, n_cb = p.cols_p >> 4;
    uint32_t piece0 = stage0 + static_cast<uint32_t>(row_in_tile * 128 + ((2 * cb) ^ (row_in_tile & 7)) * 16);
    uint32_t piece1 = stage0 + static_cast<uint32_t>(row_in_tile * 128 + ((2 * cb + 1) ^ (row_in_tile & 7)) * 16);
    uint8_t *code_ptr = p.codes + row_in_tile * code_ld + cb * 8;
    uint8_t *sf_ptr = p.sf + (p.sf_tiled ? (row_in_tile & 31) * 16 + (row_in_tile >> 5) * 4 + cb : row_in_tile * n_cb + cb);
    asm volatile("" : "+r"(piece0), "+r"(piece1), "+l"(code_ptr), "+l"(sf_ptr));

    // offsets of the tile (uniform over the CTA), advanced without multiplications
    // second block of the thread: 64 rows further down (1-D) or two block columns to the right (2-D)
    const int64_t code_half = TWO_D ? 16 : 64 * code_ld, sf_half = TWO_D ? 2 : (p.sf_tiled ? 8 : 64 * n_cb);
    const int64_t code_step = static_cast<int64_t>(step_r) * 128 * code_ld + step_c * 32, code_wrap = 127 * code_ld;
    const int64_t sf_step = p.sf_tiled ? static_cast<int64_t>(gridDim.x) * 512 : static_cast<int64_t>(step_r) * 128 * n_cb + step_c * 4;
    const int64_t sf_wrap = p.sf_tiled ? 0 : 127 * n_cb;
    int64_t code_off = static_cast<int64_t>(tr) * 128 * code_ld + tc_ * 32;
    int64_t sf_off = p.sf_tiled ? (static_cast<int64_t>(tile_r0) * tiles_c + blockIdx.x) * 512
                                : static_cast<int64_t>(tr) * 128 * n_cb + tc_ * 4;

    int fake_tr = tr;                                   // tile row of the current tile
    const DequantConsts dk = dequant_consts(tc.amax, p.fake_divisor);
    int s = 0;
    uint32_t parity = 0;
    for (int k = 0; k < my_tiles; ++k) {
        if (!mbar_wait(smem_u32(&full_bar[s]), parity, &abort_flag, &g_wait_failures, 2)) break;
        uint8_t *codes = code_ptr + code_off;
        uint8_t *sf = sf_ptr + sf_off;
        const uint32_t stage = s * FEED_STAGE_BYTES;
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            // (two block columns to the right = four 16-byte chunks = bit 6 of the swizzled address)
            const uint4 a = lds_16(TWO_D ? (piece0 + stage) ^ (j * 64) : piece0 + stage + j * 64 * 128);
            const uint4 b = lds_16(TWO_D ? (piece1 + stage) ^ (j * 64) : piece1 + stage + j * 64 * 128);
            const uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
            float v[16];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const float2 f = unpack2<T>(w[i]);
                v[2 * i] = f.x;
                v[2 * i + 1] = f.y;
            }
            uint32_t lo, hi, sf_byte;
            if (EXTRAS && p.rht) rotate16<T>(v);
            StochasticArgs sr{0u, 0u, 0u};
            if (EXTRAS && !TWO_D && p.stochastic)
                sr = stochastic_args(p, (static_cast<int64_t>(fake_tr) * 128 + j * 64 + row_in_tile) * n_cb + tc_ * 4 + cb);
            quantize_block<KIND, TWO_D, false>(v, tc, p.rule, p.exact_only != 0, TWO_D ? scratch2d + warp * 512 : nullptr, lane,
                                               lut, TWO_D ? nullptr : coop[warp], lo, hi, sf_byte, sr);
            if (!FAKE) {
                *reinterpret_cast<uint2 *>(codes + j * code_half) = make_uint2(lo, hi);
                sf[j * sf_half] = static_cast<uint8_t>(sf_byte);
            } else {
                // fused fake quantization: what dequantize would make of this block, in x's type,
                // into the un-padded output
                const int64_t row = static_cast<int64_t>(fake_tr) * 128 + j * 64 + warp * 8 + q;
                const int64_t col = (static_cast<int64_t>(tc_) * 4 + cb) * 16;
                if (row < p.rows && col < p.cols) {
                    T *dst = static_cast<T *>(p.fake_out) + row * p.fake_ld + col;
                    {
                        // the block's sixteen outputs from a table of its eight magnitudes
                        uint32_t o[8];
                        if (col + 16 <= p.cols && (reinterpret_cast<uintptr_t>(dst) & 15u) == 0 &&
                            dequantize_block_packed<T>(make_uint2(lo, hi), sf_byte, dk, o, KIND == KIND_IF4)) {
                            reinterpret_cast<uint4 *>(dst)[0] = make_uint4(o[0], o[1], o[2], o[3]);
                            reinterpret_cast<uint4 *>(dst)[1] = make_uint4(o[4], o[5], o[6], o[7]);
                            continue;
                        }
                    }
                    float dq[16];
                    dequantize_block(make_uint2(lo, hi), sf_byte, KIND == KIND_IF4, dk, dq);
                    __align__(16) T tmp[16];
#pragma unroll
                    for (int i = 0; i < 16; ++i) tmp[i] = to_out<T>(dq[i]);
                    if (col + 16 <= p.cols && (reinterpret_cast<uintptr_t>(dst) & 15u) == 0) {
                        reinterpret_cast<uint4 *>(dst)[0] = reinterpret_cast<const uint4 *>(tmp)[0];
                        reinterpret_cast<uint4 *>(dst)[1] = reinterpret_cast<const uint4 *>(tmp)[1];
                    } else {
#pragma unroll
                        for (int i = 0; i < 16; ++i)
                            if (col + i < p.cols) dst[i] = tmp[i];
                    }
                }
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&empty_bar[s]));
        if (++s == FEED_STAGES) { s = 0; parity ^= 1u; }
        fake_tr += step_r;                              // (tile row: used by the fake quantization and the noise stream)
        if (tc_ + step_c >= tiles_c) ++fake_tr;
        code_off += code_step;
        sf_off += sf_step;
        tc_ += step_c;
        if (tc_ >= tiles_c) {
            tc_ -= tiles_c;
            code_off += code_wrap;
            sf_off += sf_wrap;
        }
    }
    // A kernel launched behind this one with programmatic stream serialization (the next quantize
    // call's kernel, for one) may take the SM slots of CTAs that are done while the others finish
    // their last tile; it waits for this grid's completion before it reads anything this grid wrote.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

// ------------------------------------------------------------------------------------
// NVFP4 4/6 with the mean-squared-error rule, 1-D blocks, untransposed: the default configuration
// ------------------------------------------------------------------------------------
//
// The ring, the thread-to-block assignment and the arithmetic of quantize_rows_tma_kernel, with the
// instruction count of the common case cut down:
//   * the producer thread, which computes every tile's coordinates anyway, leaves the byte offsets
//     of the tile's codes and scales next to the stage (16 bytes per stage); the consumers read
//     them with one broadcast load instead of keeping tile coordinates of their own up to date;
//   * the pre-filter runs without a branch: the per-scale table carries each scale's share of the
//     tolerance, and that share is +infinity for scales the pre-filter must not be used with, so
//     "not eligible" is just one more way of being undecided;
//   * one vote per block sends the whole warp through quantize_block (pre-filter again, then the
//     cooperative exact evaluation, then the per-lane exact sequence: same results, block by
//     block) when any of its 32 blocks is undecided.
// Bit-identical to quantize_rows_tma_kernel<T, KIND_ADAPTIVE>: a decided block takes the decision
// that kernel takes from the same sums, an undecided one goes through that kernel's code.

// The reference's exact 4-versus-6 decision for one NVFP4 block held by one lane (any rule): what
// quantize_block does when neither the pre-filter nor the cooperative evaluation applies. Kept out
// of line: it runs for blocks with a zero or subnormal scale (padding, all-zero blocks) and in
// exact-only runs, under divergence, and the hot loop should not carry its code.
struct Block16 { float v[16]; };
__device__ __noinline__ uint4 exact_pick_nvfp4(const Block16 b, float s_a, float r_a, float s_b, float r_b, float amax,
                                               int rule, uint32_t sfb_a, uint32_t sfb_b) {
    uint32_t lo_a = 0u, hi_a = 0u, lo_b = 0u, hi_b = 0u;
    if (s_a != 0.0f) encode_e2m1(b.v, r_a, true, lo_a, hi_a);
    if (s_b != 0.0f) encode_e2m1(b.v, r_b, true, lo_b, hi_b);
    float e[16];
    exact_error_terms<false>(b.v, lo_b, hi_b, s_b, amax, 1536.0f, rule, e);
    const float err_b = rule == FOS_RULE_ABS_MAX ? max16(e) : ordered_sum16(e);
    exact_error_terms<false>(b.v, lo_a, hi_a, s_a, amax, 1536.0f, rule, e);
    const float err_a = rule == FOS_RULE_ABS_MAX ? max16(e) : ordered_sum16(e);
    const bool pick_b = err_b < err_a;
    return make_uint4(pick_b ? lo_b : lo_a, pick_b ? hi_b : hi_a, pick_b ? sfb_b : sfb_a, 0u);
}

// The reference's exact mean-squared errors of one block under both candidates, evaluated by the
// whole warp: lane 16c + i takes element i under candidate c, the 16 terms are added in the
// reference's order with shuffles. `src` is the lane that owns the block; every lane gets the
// decision "the 4 candidate wins". `coop` is this warp's exchange buffer (20 floats).
__device__ __forceinline__ bool coop_pick_nvfp4(const float (&v)[16], float s_a, float r_a, float s_b, float r_b,
                                                float amax, int src, int lane, float *coop) {
    if (lane == src) {
        float4 *x4 = reinterpret_cast<float4 *>(coop);
        x4[0] = make_float4(v[0], v[1], v[2], v[3]);
        x4[1] = make_float4(v[4], v[5], v[6], v[7]);
        x4[2] = make_float4(v[8], v[9], v[10], v[11]);
        x4[3] = make_float4(v[12], v[13], v[14], v[15]);
        x4[4] = make_float4(s_a, r_a, s_b, r_b);
    }
    __syncwarp();
    const int cand = lane >> 4, i = lane & 15;
    const float x = coop[i];
    const float s = coop[16 + 2 * cand], r = coop[17 + 2 * cand];
    const float2 q = e2m1x2_to_float2(cvt_e2m1x2(0.0f, __fmaf_rn(x, r, 0.0f)));
    const float d = __fsub_rn(__fdiv_rn(__fmul_rn(__fmul_rn(q.x, s), amax), 1536.0f), x);
    const float e = __fmul_rn(d, d);
    const float p = __fadd_rn(e, __shfl_down_sync(FULL, e, 8));      // valid in lanes with i < 8
    float total = __shfl_sync(FULL, p, cand * 16);
#pragma unroll
    for (int k = 1; k < 8; ++k) total = __fadd_rn(total, __shfl_sync(FULL, p, cand * 16 + k));
    const float exact_a = __shfl_sync(FULL, total, 0), exact_b = __shfl_sync(FULL, total, 16);
    __syncwarp();
    return exact_b < exact_a;
}

// Two 16-bit elements -> floats. bf16: the mixed-precision add x + (-0.0) is exact for every x,
// keeps the sign of a zero, and runs on the FMA pipe; shifting and masking would run on the ALU
// pipe, which this kernel saturates.
template <typename T> __device__ __forceinline__ void unpack2_fma(uint32_t w, float &lo, float &hi) {
#if FOS_UNPACK_BY_ADD
    if constexpr (std::is_same<T, __nv_bfloat16>::value) {
        asm("{ .reg .b16 l, h;\n"
            "mov.b32 {l, h}, %2;\n"
            "add.rn.f32.bf16 %0, l, 0f80000000;\n"
            "add.rn.f32.bf16 %1, h, 0f80000000; }" : "=f"(lo), "=f"(hi) : "r"(w));
        return;
    }
#endif
    const float2 f = unpack2<T>(w);
    lo = f.x;
    hi = f.y;
}

template <typename T>
__global__ void __launch_bounds__(FEED_THREADS, FOS_FEED_CTAS)
quantize_rows_mse_kernel(const __grid_constant__ CUtensorMap map_x, const QuantParams p) {
    extern __shared__ uint8_t feed_smem_raw[];
    __shared__ float4 lut[128];
    __shared__ __align__(16) float coop[FEED_CONSUMERS / 32][20];
    __shared__ __align__(16) longlong2 tile_meta[FEED_STAGES];     // per stage: byte offsets of the tile's codes and scales
    __shared__ __align__(8) uint64_t full_bar[FEED_STAGES], empty_bar[FEED_STAGES];
    __shared__ int abort_flag;

    const uint32_t stage0 = (smem_u32(feed_smem_raw) + 1023u) & ~1023u;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tiles_c = static_cast<int>(p.cols_p >> 6);
    int tiles_r = static_cast<int>(p.rows_p >> 7), tile_r0 = 0;
    const float *amax_ptr = p.amax;
    if (p.group_start != nullptr) group_tiles(p, tile_r0, tiles_r, amax_ptr);
    const int64_t n_tiles = static_cast<int64_t>(tiles_c) * tiles_r;
    const int64_t code_ld = p.cols_p >> 1, n_cb = p.cols_p >> 4;

    if (threadIdx.x == 0) {
        abort_flag = 0;
#pragma unroll
        for (int s = 0; s < FEED_STAGES; ++s) {
            mbar_init(smem_u32(&full_bar[s]), 1);
            mbar_init(smem_u32(&empty_bar[s]), FEED_CONSUMERS / 32);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    // this CTA's tiles: blockIdx.x, blockIdx.x + gridDim.x, ... in row-major tile order
    const int my_tiles = static_cast<int>((n_tiles - blockIdx.x + gridDim.x - 1) / gridDim.x);

    if (warp == FEED_CONSUMERS / 32) {
        // ---------------- producer ----------------
        if (lane != 0) return;
        const int step_r = static_cast<int>(gridDim.x) / tiles_c, step_c = static_cast<int>(gridDim.x) % tiles_c;
        int tr = tile_r0 + static_cast<int>(blockIdx.x) / tiles_c, tc_ = static_cast<int>(blockIdx.x) % tiles_c;
        int64_t tile = static_cast<int64_t>(tile_r0) * tiles_c + blockIdx.x;
        if (!p.x_is_ready) asm volatile("griddepcontrol.wait;" ::: "memory");
        int issued = 0, s = 0;
        uint32_t parity = 1;   // of the "stage is free" barrier; the first round finds every stage free
        for (; issued < my_tiles; ++issued) {
            if (issued >= FEED_STAGES && !mbar_wait(smem_u32(&empty_bar[s]), parity, &abort_flag, &g_wait_failures, 8))
                break;
            // (the arrive below releases this store to the consumers that acquire the barrier's phase)
            tile_meta[s] = make_longlong2(static_cast<int64_t>(tr) * 128 * code_ld + tc_ * 32,
                                          p.sf_tiled ? tile * 512 : static_cast<int64_t>(tr) * 128 * n_cb + tc_ * 4);
            mbar_expect_tx(smem_u32(&full_bar[s]), FEED_STAGE_BYTES);
            tma_load_2d(stage0 + s * FEED_STAGE_BYTES, &map_x, tc_ * 128, tr * FEED_TILE_ROWS, smem_u32(&full_bar[s]));
            if (++s == FEED_STAGES) { s = 0; parity ^= 1u; }
            tile += gridDim.x;
            tr += step_r;
            tc_ += step_c;
            if (tc_ >= tiles_c) { tc_ -= tiles_c; ++tr; }
        }
        // stay until every copy this thread issued has landed: shared memory must outlive them
        for (int j = issued > FEED_STAGES ? issued - FEED_STAGES : 0; j < issued; ++j) {
            const uint32_t bar = smem_u32(&full_bar[j % FEED_STAGES]);
            const uint32_t landed = static_cast<uint32_t>(j / FEED_STAGES) & 1u;
            const unsigned long long t0 = global_timer_ns();
            while (!mbar_try_wait(bar, landed) && global_timer_ns() - t0 < WAIT_LIMIT_NS) {}
        }
        return;
    }

    // ---------------- consumers ----------------
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const TensorConsts tc = tensor_consts<KIND_ADAPTIVE>(*reinterpret_cast<const volatile float *>(amax_ptr), p.rule);
    if (p.amax_store != nullptr && threadIdx.x == 0 && blockIdx.x == 0) *p.amax_store = tc.amax;
    if (threadIdx.x < 128)
        lut[threadIdx.x] = scale_entry(threadIdx.x, tc, p.rule == FOS_RULE_MSE && !p.exact_only && tc.filter_ok);
    asm volatile("bar.sync 1, %0;" ::"n"(FEED_CONSUMERS) : "memory");

    // lane l of warp w owns rows 8w + l/4 and 64 + 8w + l/4 of the tile and block column l%4
    const int q = lane >> 2, cb = lane & 3;
    const int row_in_tile = warp * 8 + q;
    uint32_t piece0 = stage0 + static_cast<uint32_t>(row_in_tile * 128 + ((2 * cb) ^ (row_in_tile & 7)) * 16);
    uint32_t piece1 = stage0 + static_cast<uint32_t>(row_in_tile * 128 + ((2 * cb + 1) ^ (row_in_tile & 7)) * 16);
    uint8_t *code_ptr = p.codes + row_in_tile * code_ld + cb * 8;
    uint8_t *sf_ptr = p.sf + (p.sf_tiled ? (row_in_tile & 31) * 16 + (row_in_tile >> 5) * 4 + cb : row_in_tile * n_cb + cb);
    uint32_t lut_base = smem_u32(lut), meta_addr = smem_u32(tile_meta), full_addr = smem_u32(full_bar), empty_addr = smem_u32(empty_bar);
    asm volatile("" : "+r"(piece0), "+r"(piece1), "+l"(code_ptr), "+l"(sf_ptr), "+r"(lut_base));
    const int64_t code_half = 64 * code_ld, sf_half = p.sf_tiled ? 8 : 64 * n_cb;
    const float encode0 = tc.encode0;
    const int rule = p.rule;

    uint32_t s_off = 0, s_idx = 0, parity = 0;
    for (int k = 0; k < my_tiles; ++k) {
        if (!mbar_wait(full_addr + 8 * s_idx, parity, &abort_flag, &g_wait_failures, 9)) break;
        int64_t code_off, sf_off;
        asm volatile("ld.shared.v2.b64 {%0, %1}, [%2];" : "=l"(code_off), "=l"(sf_off) : "r"(meta_addr + 16 * s_idx));
        uint8_t *codes = code_ptr + code_off;
        uint8_t *sf = sf_ptr + sf_off;
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const uint4 a = lds_16(piece0 + s_off + j * 64 * 128);
            const uint4 b = lds_16(piece1 + s_off + j * 64 * 128);
            const uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
            float v[16];
#pragma unroll
            for (int i = 0; i < 8; ++i) unpack2_fma<T>(w[i], v[2 * i], v[2 * i + 1]);
            float bmax = fmaxf(fabsf(v[0]), fabsf(v[1]));
#pragma unroll
            for (int i = 2; i < 16; i += 2) bmax = fmaxf(fmaxf(bmax, fabsf(v[i])), fabsf(v[i + 1]));
            const float hp = __fmul_rn(div6_exact(bmax), encode0);
            const uint32_t both = cvt_e4m3x2(__fmul_rn(hp, 1.5f), hp);   // "4" candidate in the upper byte
            float4 ea, eb;
            asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(ea.x), "=f"(ea.y), "=f"(ea.z), "=f"(ea.w)
                         : "r"(lut_base + ((both & 0xffu) << 4)));
            asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(eb.x), "=f"(eb.y), "=f"(eb.z), "=f"(eb.w)
                         : "r"(lut_base + ((both >> 8) << 4)));
            // both candidates: codes, residuals t = q - x*r, sums of t^2 (see quantize_block for the bound)
            const uint64_t ra2 = pack2(ea.y, ea.y), rb2 = pack2(eb.y, eb.y);
            uint64_t acc_a = pack2(0.0f, 0.0f), acc_b = acc_a;
            uint32_t ca[2], cbk[2];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                float ta[8], tb[8];
                ca[h] = encode8_with_residuals(&v[8 * h], ra2, ta);
                cbk[h] = encode8_with_residuals(&v[8 * h], rb2, tb);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const uint64_t pa = pack2(ta[2 * i], ta[2 * i + 1]), pb = pack2(tb[2 * i], tb[2 * i + 1]);
                    acc_a = fma2(pa, pa, acc_a);
                    acc_b = fma2(pb, pb, acc_b);
                }
            }
            float a0, a1, b0, b1;
            unpack2f(acc_a, a0, a1);
            unpack2f(acc_b, b0, b1);
            const float err_a = (a0 + a1) * ea.w, err_b = (b0 + b1) * eb.w;     // times G^2
            const float tau = fmaf(0x1p-24f * 1.5f * 228.0f, err_a + err_b, ea.z + eb.z);
            const float diff = err_b - err_a;
            const bool pick_fast = diff < 0.0f;
            uint32_t lo = pick_fast ? cbk[0] : ca[0], hi = pick_fast ? cbk[1] : ca[1];
            uint32_t sf_byte = pick_fast ? both >> 8 : both & 0xffu;
            const bool undecided = !(fabsf(diff) > tau);
            if (__any_sync(FULL, undecided)) {
                // Undecided blocks whose scales the pre-filter accepts (two normal E4M3 numbers) are
                // re-decided exactly by the whole warp, one block at a time; the others (zero or
                // subnormal scale, exact-only run, amax out of range) take the per-lane exact sequence.
                const bool coop_ok = fminf(ea.w, eb.w) >= 0.0f;
                unsigned pending = __ballot_sync(FULL, undecided && coop_ok);
                while (pending) {
                    const int src = __ffs(pending) - 1;
                    pending &= pending - 1;
                    const bool b_wins = coop_pick_nvfp4(v, ea.x, ea.y, eb.x, eb.y, tc.amax, src, lane, coop[warp]);
                    if (lane == src) {
                        lo = b_wins ? cbk[0] : ca[0];
                        hi = b_wins ? cbk[1] : ca[1];
                        sf_byte = b_wins ? both >> 8 : both & 0xffu;
                    }
                }
                if (undecided && !coop_ok) {
                    if (both == 0u) {
                        // both scales are zero (an all-zero block: the padding rows of grouped tensors are full
                        // of them): the exact sequence encodes nothing and picks between two zero scale bytes
                        lo = 0u;
                        hi = 0u;
                    } else {
                        Block16 blk;
#pragma unroll
                        for (int i = 0; i < 16; ++i) blk.v[i] = v[i];
                        const uint4 r = exact_pick_nvfp4(blk, ea.x, ea.y, eb.x, eb.y, tc.amax, rule, both & 0xffu, both >> 8);
                        lo = r.x;
                        hi = r.y;
                        sf_byte = r.z;
                    }
                }
            }
            *reinterpret_cast<uint2 *>(codes + j * code_half) = make_uint2(lo, hi);
            sf[j * sf_half] = static_cast<uint8_t>(sf_byte);
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(empty_addr + 8 * s_idx);
        s_off += FEED_STAGE_BYTES;
        if (++s_idx == FEED_STAGES) { s_idx = 0; s_off = 0; parity ^= 1u; }
    }
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

// ------------------------------------------------------------------------------------
// transposed input, 1-D blocks, fed by the TMA unit
// ------------------------------------------------------------------------------------
//
// Y = x^T: a block of Y is 16 consecutive ROWS of x at one column. One tile of Y (128 rows x 64
// columns) is 64 rows x 128 columns of x, fetched as one 16 KB box (256-byte rows, no swizzle: a
// warp reads 32 neighbouring 2-byte elements of one x row at a time, which is conflict-free).
// Consumer thread t owns row t % 128 of the tile and the two blocks 2 * (t / 128) and the next:
// 16 bytes of codes and 2 scale bytes per tile, both contiguous. Everything else (ring, table,
// cooperative fallback, launch chain) is as in quantize_rows_tma_kernel.

constexpr int COLS_BOX_ROWS = 64, COLS_BOX_BYTES = 256;

template <typename T, int KIND, bool TWO_D = false, bool EXTRAS = false>
__global__ void __launch_bounds__(FEED_THREADS, FOS_FEED_CTAS)
quantize_cols_tma_kernel(const __grid_constant__ CUtensorMap map_x, const QuantParams p) {
    extern __shared__ uint8_t feed_smem_raw[];
    __shared__ float4 lut[128];
    __shared__ __align__(16) float coop[FEED_CONSUMERS / 32][20];
    // 2-D blocks: lanes 0-15 and 16-31 of a warp hold the rows of two 16 x 16 blocks
    __shared__ __align__(16) float scratch2d[TWO_D ? (FEED_CONSUMERS / 32) * 512 : 4];
    __shared__ __align__(8) uint64_t full_bar[FEED_STAGES], empty_bar[FEED_STAGES];
    __shared__ int abort_flag;

    const uint32_t stage0 = (smem_u32(feed_smem_raw) + 1023u) & ~1023u;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // tiles of Y: tiles_r along its rows (x's columns), tiles_c along its columns (x's rows);
    // neighbours in the order of processing are neighbours along x's rows
    const int tiles_r = static_cast<int>(p.rows_p >> 7), tiles_c = static_cast<int>(p.cols_p >> 6);
    const int64_t n_tiles = static_cast<int64_t>(tiles_c) * tiles_r;

    if (threadIdx.x == 0) {
        abort_flag = 0;
#pragma unroll
        for (int s = 0; s < FEED_STAGES; ++s) {
            mbar_init(smem_u32(&full_bar[s]), 1);
            mbar_init(smem_u32(&empty_bar[s]), FEED_CONSUMERS / 32);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    const int step_c = static_cast<int>(gridDim.x) / tiles_r, step_r = static_cast<int>(gridDim.x) % tiles_r;
    int tc_ = static_cast<int>(blockIdx.x) / tiles_r, tr = static_cast<int>(blockIdx.x) % tiles_r;
    const int my_tiles = static_cast<int>((n_tiles - blockIdx.x + gridDim.x - 1) / gridDim.x);

    if (warp == FEED_CONSUMERS / 32) {
        // ---------------- producer ----------------
        if (lane != 0) return;
        if (!p.x_is_ready) asm volatile("griddepcontrol.wait;" ::: "memory");
        int issued = 0, s = 0;
        uint32_t parity = 1;
        for (; issued < my_tiles; ++issued) {
            if (issued >= FEED_STAGES && !mbar_wait(smem_u32(&empty_bar[s]), parity, &abort_flag, &g_wait_failures, 3))
                break;
            mbar_expect_tx(smem_u32(&full_bar[s]), FEED_STAGE_BYTES);
            tma_load_2d(stage0 + s * FEED_STAGE_BYTES, &map_x, tr * COLS_BOX_BYTES, tc_ * COLS_BOX_ROWS, smem_u32(&full_bar[s]));
            if (++s == FEED_STAGES) { s = 0; parity ^= 1u; }
            tc_ += step_c;
            tr += step_r;
            if (tr >= tiles_r) { tr -= tiles_r; ++tc_; }
        }
        for (int j = issued > FEED_STAGES ? issued - FEED_STAGES : 0; j < issued; ++j) {
            const uint32_t bar = smem_u32(&full_bar[j % FEED_STAGES]);
            const uint32_t landed = static_cast<uint32_t>(j / FEED_STAGES) & 1u;
            const unsigned long long t0 = global_timer_ns();
            while (!mbar_try_wait(bar, landed) && global_timer_ns() - t0 < WAIT_LIMIT_NS) {}
        }
        return;
    }

    // ---------------- consumers ----------------
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const TensorConsts tc = tensor_consts<KIND>(*reinterpret_cast<const volatile float *>(p.amax), p.rule, EXTRAS && p.unbiased);
    if (p.amax_store != nullptr && threadIdx.x == 0 && blockIdx.x == 0) *p.amax_store = tc.amax;
    if (threadIdx.x < 128)
        lut[threadIdx.x] = scale_entry(threadIdx.x, tc, rule_has_filter<KIND, TWO_D>(p.rule) && !p.exact_only && tc.filter_ok);
    asm volatile("bar.sync 1, %0;" ::"n"(FEED_CONSUMERS) : "memory");

    const int jr = threadIdx.x & 127, pair = threadIdx.x >> 7;          // row of the tile, which two of its four blocks
    const int64_t code_ld = p.cols_p >> 1, n_cb = p.cols_p >> 4;
    uint32_t src = stage0 + static_cast<uint32_t>(pair * 32 * COLS_BOX_BYTES + jr * 2);
    uint8_t *code_ptr = p.codes + jr * code_ld + pair * 16;
    uint8_t *sf_ptr = p.sf + (p.sf_tiled ? (jr & 31) * 16 + (jr >> 5) * 4 + pair * 2 : jr * n_cb + pair * 2);
    asm volatile("" : "+r"(src), "+l"(code_ptr), "+l"(sf_ptr));

    int s = 0;
    uint32_t parity = 0;
    for (int k = 0; k < my_tiles; ++k) {
        if (!mbar_wait(smem_u32(&full_bar[s]), parity, &abort_flag, &g_wait_failures, 4)) break;
        uint8_t *codes = code_ptr + static_cast<int64_t>(tr) * 128 * code_ld + tc_ * 32;
        uint8_t *sf = sf_ptr + (p.sf_tiled ? (static_cast<int64_t>(tr) * tiles_c + tc_) * 512
                                           : static_cast<int64_t>(tr) * 128 * n_cb + tc_ * 4);
        const uint32_t stage = src + s * FEED_STAGE_BYTES;
        uint32_t words[4], sf_pair = 0u;
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            float v[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                uint16_t h;
                asm volatile("ld.shared.u16 %0, [%1];" : "=h"(h) : "r"(stage + (j * 16 + i) * COLS_BOX_BYTES));
                v[i] = elem_to_float<T>(reinterpret_cast<const T &>(h));
            }
            uint32_t lo, hi, sf_byte;
            if (EXTRAS && p.rht) rotate16<T>(v);
            StochasticArgs sr{0u, 0u, 0u};
            if (EXTRAS && !TWO_D && p.stochastic)
                sr = stochastic_args(p, (static_cast<int64_t>(tr) * 128 + jr) * n_cb + tc_ * 4 + pair * 2 + j);
            quantize_block<KIND, TWO_D, TWO_D>(v, tc, p.rule, p.exact_only != 0, TWO_D ? scratch2d + warp * 512 : nullptr, lane,
                                               lut, TWO_D ? nullptr : coop[warp], lo, hi, sf_byte, sr);
            words[2 * j] = lo;
            words[2 * j + 1] = hi;
            sf_pair |= sf_byte << (8 * j);
        }
        *reinterpret_cast<uint4 *>(codes) = make_uint4(words[0], words[1], words[2], words[3]);
        *reinterpret_cast<uint16_t *>(sf) = static_cast<uint16_t>(sf_pair);
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&empty_bar[s]));
        if (++s == FEED_STAGES) { s = 0; parity ^= 1u; }
        tc_ += step_c;
        tr += step_r;
        if (tr >= tiles_r) { tr -= tiles_r; ++tc_; }
    }
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

// Tensor map over x as bytes: [rows][cols * 2] with a row pitch of ld * 2, boxes of 128 rows x 128 bytes.
inline bool make_x_map(CUtensorMap *map, const QuantParams &p, bool transposed) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return false;
    cuuint64_t dims[2] = {static_cast<cuuint64_t>(p.cols * 2), static_cast<cuuint64_t>(p.rows)};
    cuuint64_t strides[1] = {static_cast<cuuint64_t>(p.ld * 2)};
    cuuint32_t box[2] = {transposed ? static_cast<cuuint32_t>(COLS_BOX_BYTES) : 128u,
                         static_cast<cuuint32_t>(transposed ? COLS_BOX_ROWS : FEED_TILE_ROWS)};
    cuuint32_t estr[2] = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(p.x), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, transposed ? CU_TENSOR_MAP_SWIZZLE_NONE : CU_TENSOR_MAP_SWIZZLE_128B,
              CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Launches the TMA-fed kernel when x qualifies; *launched tells whether it did.
template <typename T, int KIND, bool TRANSPOSED, bool FAKE, bool TWO_D, bool EXTRAS, bool LEAN = false>
cudaError_t launch_rows_tma_impl(const QuantParams &p, cudaStream_t stream, bool *launched) {
    *launched = false;
    if (reinterpret_cast<uintptr_t>(p.x) % 16 != 0 || (p.ld * 2) % 16 != 0) return cudaSuccess;
    // the transposed kernel stores 16 bytes of codes and 2 scale bytes at a time
    if (TRANSPOSED && (reinterpret_cast<uintptr_t>(p.codes) % 16 != 0 || reinterpret_cast<uintptr_t>(p.sf) % 2 != 0)) return cudaSuccess;
    if (p.cols * 2 >= (int64_t(1) << 31) || p.rows >= (int64_t(1) << 31) || p.ld * 2 >= (int64_t(1) << 40)) return cudaSuccess;
    CUtensorMap map;
    if (!make_x_map(&map, p, TRANSPOSED)) return cudaSuccess;
    auto kernel = LEAN ? quantize_rows_mse_kernel<T>
                       : (TRANSPOSED ? quantize_cols_tma_kernel<T, KIND, TWO_D, EXTRAS> : quantize_rows_tma_kernel<T, KIND, FAKE, TWO_D, EXTRAS>);
    static int ctas_per_sm[64] = {};
    static int sm_count[64] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    const int slot = (dev >= 0 && dev < 64) ? dev : 0;
    if (ctas_per_sm[slot] == 0) {
        int n = 0, sms = 0;
        e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, FEED_SMEM_BYTES);
        if (e != cudaSuccess) return e;
        e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kernel, FEED_THREADS, FEED_SMEM_BYTES);
        if (e != cudaSuccess) return e;
        e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        if (e != cudaSuccess) return e;
        sm_count[slot] = sms;
        ctas_per_sm[slot] = n > 0 ? n : 1;
    }
    const int64_t n_tiles = (p.rows_p >> 7) * (p.cols_p >> 6);
    int64_t grid = static_cast<int64_t>(ctas_per_sm[slot]) * sm_count[slot];
    const bool grouped = p.group_start != nullptr;
    if (grouped) {
        // how the rows are spread over the groups is known on the device only: every group gets twice its even
        // share of the resident CTAs (at least 8), and a CTA whose group has fewer tiles than that leaves at once
        grid = 2 * grid / p.num_groups;
        if (grid < 8) grid = 8;
    }
    if (grid > n_tiles) grid = n_tiles;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(grid), grouped ? static_cast<unsigned>(p.num_groups) : 1u);
    cfg.blockDim = dim3(FEED_THREADS);
    cfg.dynamicSmemBytes = FEED_SMEM_BYTES;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = grouped ? 0 : 1;      // (a grouped launch reads row ranges written by earlier work: a full dependency)
    e = cudaLaunchKernelEx(&cfg, kernel, map, p);
    if (e == cudaSuccess) *launched = true;
    return e;
}

template <typename T, int KIND, bool TRANSPOSED, bool FAKE = false, bool TWO_D = false>
cudaError_t launch_rows_tma(const QuantParams &p, cudaStream_t stream, bool *launched) {
    if constexpr (!FAKE) {
        if (p.rht || p.stochastic) return launch_rows_tma_impl<T, KIND, TRANSPOSED, FAKE, TWO_D, true>(p, stream, launched);
    }
    return launch_rows_tma_impl<T, KIND, TRANSPOSED, FAKE, TWO_D, false>(p, stream, launched);
}

template <typename T, int KIND>
cudaError_t launch_rows(const QuantParams &p, cudaStream_t stream) {
    if (p.variant != 1) {
        bool launched = false;
        if constexpr (KIND == KIND_ADAPTIVE) {
            // the default configuration (mean-squared error, round to nearest, no rotation) has a kernel of its own
            if (p.rule == FOS_RULE_MSE && !p.rht && !p.stochastic && p.variant != 2) {
                const cudaError_t e = launch_rows_tma_impl<T, KIND, false, false, false, false, true>(p, stream, &launched);
                if (e != cudaSuccess || launched) return e;
            }
        }
        const cudaError_t e = launch_rows_tma<T, KIND, false>(p, stream, &launched);
        if (e != cudaSuccess || launched) return e;
    }
    auto kernel = quantize_rows_kernel<T, KIND>;
    static int ctas_per_sm[64] = {};
    static int sm_count[64] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    const int slot = (dev >= 0 && dev < 64) ? dev : 0;
    if (ctas_per_sm[slot] == 0) {
        int n = 0, sms = 0;
        e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kernel, ROWS_CTA_THREADS, 0);
        if (e != cudaSuccess) return e;
        e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        if (e != cudaSuccess) return e;
        ctas_per_sm[slot] = n > 0 ? n : 1;
        sm_count[slot] = sms;
    }
    const int64_t n_tiles = (p.rows_p >> 6) * (p.cols_p >> 6);
    int64_t grid = static_cast<int64_t>(ctas_per_sm[slot]) * sm_count[slot];
    if (grid > n_tiles) grid = n_tiles;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(grid));
    cfg.blockDim = dim3(ROWS_CTA_THREADS);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, p);
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

// The TMA-fed kernel for (2-D blocks or not) x (transposed or not); *launched tells whether x qualified.
template <typename T, int KIND>
cudaError_t launch_fed(const QuantParams &p, bool two_d, bool transposed, cudaStream_t stream, bool *launched) {
    *launched = false;
    if (p.variant == 1) return cudaSuccess;
    if (two_d) {
        return transposed ? launch_rows_tma<T, KIND, true, false, true>(p, stream, launched)
                          : launch_rows_tma<T, KIND, false, false, true>(p, stream, launched);
    }
    return transposed ? launch_rows_tma<T, KIND, true>(p, stream, launched) : cudaSuccess;   // (1-D rows: launch_rows)
}

template <typename T>
cudaError_t launch_all(const QuantParams &p, int kind, bool two_d, bool transposed, cudaStream_t stream) {
    if (two_d || transposed) {
        bool launched = false;
        const cudaError_t e = kind == KIND_STATIC     ? launch_fed<T, KIND_STATIC>(p, two_d, transposed, stream, &launched)
                              : kind == KIND_ADAPTIVE ? launch_fed<T, KIND_ADAPTIVE>(p, two_d, transposed, stream, &launched)
                                                      : launch_fed<T, KIND_IF4>(p, two_d, transposed, stream, &launched);
        if (e != cudaSuccess || launched) return e;
    }
    if (!two_d && !transposed) {
        if (kind == KIND_STATIC) return launch_rows<T, KIND_STATIC>(p, stream);
        if (kind == KIND_ADAPTIVE) return launch_rows<T, KIND_ADAPTIVE>(p, stream);
        return launch_rows<T, KIND_IF4>(p, stream);
    }
    if (kind == KIND_STATIC) return launch_kind<T, KIND_STATIC>(p, two_d, transposed, stream);
    if (kind == KIND_ADAPTIVE) return launch_kind<T, KIND_ADAPTIVE>(p, two_d, transposed, stream);
    return launch_kind<T, KIND_IF4>(p, two_d, transposed, stream);
}

inline cudaLaunchConfig_t dependent_launch_config(unsigned grid, unsigned block, cudaStream_t stream,
                                                  cudaLaunchAttribute *attr) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(block);
    cfg.stream = stream;
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cfg;
}

template <typename T>
cudaError_t launch_amax(const void *x, int64_t rows, int64_t cols, int64_t ld, bool vec16, float *amax,
                        cudaStream_t stream, bool rht = false, bool transposed = false) {
    cudaLaunchAttribute attr[1];
    cudaLaunchConfig_t cfg = dependent_launch_config(1, 32, stream, attr);
    cudaError_t e = cudaLaunchKernelEx(&cfg, zero_amax_kernel, amax);
    if (e != cudaSuccess) return e;
    if (rht) {
        // amax of the ROTATED tensor: 6 resident CTAs per SM is a safe single wave
        const int64_t units = transposed ? (rows >> 4) * cols : rows * (cols >> 4);
        int64_t blocks = (units + 255) / 256;
        if (blocks > 148 * 6) blocks = 148 * 6;
        if (blocks < 1) blocks = 1;
        cfg = dependent_launch_config(static_cast<unsigned>(blocks), 256, stream, attr);
        return cudaLaunchKernelEx(&cfg, amax_rht_kernel<T>, static_cast<const T *>(x), rows, cols, ld, transposed ? 1 : 0, amax);
    }
    // one wave: as many CTAs as can be resident at once (a partial second wave would run alone)
    static int resident[64] = {};
    int dev = 0;
    e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    const int slot = (dev >= 0 && dev < 64) ? dev : 0;
    if (resident[slot] == 0) {
        int per_sm = 0, sms = 0;
        e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, amax_kernel<T>, 256, 0);
        if (e != cudaSuccess) return e;
        e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        if (e != cudaSuccess) return e;
        resident[slot] = (per_sm > 0 ? per_sm : 1) * sms;
    }
    const bool vec32 = vec16 && reinterpret_cast<uintptr_t>(x) % 32 == 0 && (ld * 2) % 32 == 0 && cols % 16 == 0;
    const int vec = vec32 ? 32 : (vec16 ? 16 : 0);
    const int64_t work = vec ? rows * (cols / (vec / 2)) : rows * cols;
    int64_t blocks = (work + 255) / 256;
    if (blocks > resident[slot]) blocks = resident[slot];
#ifndef FOS_AMAX_EVEN_ROUNDS
#define FOS_AMAX_EVEN_ROUNDS 1
#endif
    if (FOS_AMAX_EVEN_ROUNDS && vec) {
        // whole rounds: a thread takes 128 bytes per round, so with a full wave of CTAs the last round is usually
        // ragged (8192 x 4096: 3.46 rounds, the fourth with half of the loads in flight). Fewer CTAs, all of which
        // run the same number of full rounds, keep the memory system equally busy to the end.
        const int64_t per_round = 256 * (128 / vec);                     // chunks one CTA takes per round
        const int64_t rounds = (work + per_round * resident[slot] - 1) / (per_round * resident[slot]);
        const int64_t even = (work + per_round * rounds - 1) / (per_round * rounds);
        if (even >= resident[slot] / 2) blocks = even;                   // (tiny inputs keep one CTA per 256 chunks)
    }
    if (blocks < 1) blocks = 1;
    cfg = dependent_launch_config(static_cast<unsigned>(blocks), 256, stream, attr);
    return cudaLaunchKernelEx(&cfg, amax_kernel<T>, static_cast<const T *>(x), rows, cols, ld, vec, amax);
}

template <typename T>
cudaError_t launch_fake(const QuantParams &p, int kind, cudaStream_t stream, bool *launched) {
    if (kind == KIND_STATIC) return launch_rows_tma<T, KIND_STATIC, false, true>(p, stream, launched);
    if (kind == KIND_ADAPTIVE) return launch_rows_tma<T, KIND_ADAPTIVE, false, true>(p, stream, launched);
    return launch_rows_tma<T, KIND_IF4, false, true>(p, stream, launched);
}

}  // namespace
}  // namespace fos

extern "C" int fos_pseudo_quantize(const void *x, int x_dtype, int64_t rows, int64_t cols, int64_t ld, int format,
                                   int scale_rule, const float *amax_in, void *out, int64_t ld_out, float *amax_out,
                                   int flags, void *stream_) {
    using namespace fos;
    if (!x || !out || !amax_out) return FOS_ERR_INVALID_ARGUMENT;
    if (rows <= 0 || cols <= 0 || ld < cols || ld_out < cols) return FOS_ERR_INVALID_ARGUMENT;
    if (x_dtype != FOS_BF16 && x_dtype != FOS_FP16) return FOS_ERR_INVALID_ARGUMENT;
    if (format == FOS_MXFP4) return FOS_ERR_UNSUPPORTED;          // quantize, then dequantize
    if (format != FOS_NVFP4 && format != FOS_IF4) return FOS_ERR_INVALID_ARGUMENT;
    if (scale_rule < FOS_RULE_STATIC_6 || scale_rule > FOS_RULE_ABS_MAX) return FOS_ERR_INVALID_ARGUMENT;
    const bool is_static = scale_rule == FOS_RULE_STATIC_6 || scale_rule == FOS_RULE_STATIC_4;
    if (format == FOS_IF4 && is_static) return FOS_ERR_UNSUPPORTED;
    if (flags & FOS_QUANTIZE_RHT) return FOS_ERR_UNSUPPORTED;
    // only inputs the TMA-fed kernel takes; the caller runs fos_quantize + fos_dequantize otherwise
    if (reinterpret_cast<uintptr_t>(x) % 16 != 0 || (ld * 2) % 16 != 0) return FOS_ERR_UNSUPPORTED;
    int st = check_device();
    if (st != FOS_OK) return st;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);

    QuantParams p{};
    p.x = x;
    p.rows = rows; p.cols = cols; p.ld = ld;
    p.out_rows = rows; p.out_cols = cols;
    p.rows_p = round_up64(rows, TILE_ROWS);
    p.cols_p = round_up64(cols, TILE_COLS);
    p.rule = scale_rule;
    p.sf_tiled = 1;
    p.exact_only = (flags & FOS_QUANTIZE_EXACT_ONLY) != 0;
    p.fake_out = out;
    p.fake_ld = ld_out;
    p.fake_divisor = dequant_divisor(format, scale_rule);
    const bool vec16 = cols % 8 == 0;
    if (amax_in) {
        p.amax = amax_in;
        p.amax_store = amax_in != amax_out ? amax_out : nullptr;
    } else {
        FOS_CUDA_TRY(x_dtype == FOS_BF16
                         ? launch_amax<__nv_bfloat16>(x, rows, cols, ld, vec16, amax_out, stream)
                         : launch_amax<__half>(x, rows, cols, ld, vec16, amax_out, stream));
        p.amax = amax_out;
    }
    p.x_is_ready = amax_in == nullptr;
    const int kind = format == FOS_IF4 ? KIND_IF4 : (is_static ? KIND_STATIC : KIND_ADAPTIVE);
    bool launched = false;
    FOS_CUDA_TRY(x_dtype == FOS_BF16 ? launch_fake<__nv_bfloat16>(p, kind, stream, &launched)
                                     : launch_fake<__half>(p, kind, stream, &launched));
    // (the amax pass, if any, has been enqueued already: harmless, the caller's fallback repeats it)
    return launched ? FOS_OK : FOS_ERR_UNSUPPORTED;
}

static int quantize_entry(const void *x, int x_dtype, int64_t rows, int64_t cols, int64_t ld, int format,
                          int scale_rule, int block_2d, int transpose, int sf_layout, const float *amax_in,
                          uint8_t *codes, uint8_t *sf, float *amax_out, int flags, void *stream_, int stochastic,
                          uint64_t seed) {
    using namespace fos;
    if (stochastic) {
        // stochastic rounding lives in the TMA-fed kernels only: NVFP4, 1-D blocks, aligned input
        if ((format != FOS_NVFP4 && format != FOS_IF4) || block_2d) return FOS_ERR_UNSUPPORTED;
        if (format == FOS_IF4 && scale_rule != FOS_RULE_MSE) return FOS_ERR_UNSUPPORTED;   // the noisy candidates are compared by squared error
        if ((flags & FOS_QUANTIZE_NO_TMA) || reinterpret_cast<uintptr_t>(x) % 16 != 0 || (ld * 2) % 16 != 0) return FOS_ERR_UNSUPPORTED;
        if (transpose && (reinterpret_cast<uintptr_t>(codes) % 16 != 0 || reinterpret_cast<uintptr_t>(sf) % 2 != 0))
            return FOS_ERR_UNSUPPORTED;
    }
    if (!x || !codes || !sf || !amax_out) return FOS_ERR_INVALID_ARGUMENT;
    if (rows <= 0 || cols <= 0 || ld < cols) return FOS_ERR_INVALID_ARGUMENT;
    if (x_dtype != FOS_BF16 && x_dtype != FOS_FP16) return FOS_ERR_INVALID_ARGUMENT;
    if (format != FOS_NVFP4 && format != FOS_IF4 && format != FOS_MXFP4) return FOS_ERR_INVALID_ARGUMENT;
    if (scale_rule < FOS_RULE_STATIC_6 || scale_rule > FOS_RULE_ABS_MAX) return FOS_ERR_INVALID_ARGUMENT;
    if (sf_layout != FOS_SF_ROWMAJOR && sf_layout != FOS_SF_TILED) return FOS_ERR_INVALID_ARGUMENT;
    if (format == FOS_MXFP4) {
        // power-of-two scales per 32 values: static rules only, no rotation, one kernel, no amax pass
        if ((scale_rule != FOS_RULE_STATIC_6 && scale_rule != FOS_RULE_STATIC_4) || (flags & FOS_QUANTIZE_RHT))
            return FOS_ERR_UNSUPPORTED;
        if (reinterpret_cast<uintptr_t>(codes) % 8 != 0) return FOS_ERR_MISALIGNED;
        const int st_mx = check_device();
        if (st_mx != FOS_OK) return st_mx;
        return quantize_mxfp4(x, x_dtype, rows, cols, ld, scale_rule, block_2d, transpose, sf_layout, codes, sf, amax_out,
                              static_cast<cudaStream_t>(stream_));
    }
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
    p.variant = (flags & FOS_QUANTIZE_NO_TMA) ? 1 : ((flags & FOS_QUANTIZE_GENERAL_KERNEL) ? 2 : 0);
    p.rht = (flags & FOS_QUANTIZE_RHT) != 0;
    if (p.rht && p.out_cols % 16 != 0) return FOS_ERR_INVALID_ARGUMENT;   // blocks of 16 along the quantized axis
    p.stochastic = stochastic;
    p.unbiased = stochastic && (flags & FOS_QUANTIZE_UNBIASED) != 0;
    p.seed_lo = static_cast<uint32_t>(seed);
    p.seed_hi = static_cast<uint32_t>(seed >> 32);
    const uintptr_t addr = reinterpret_cast<uintptr_t>(x);
    const int64_t ld_bytes = ld * 2;
    p.vec_bytes = (addr % 32 == 0 && ld_bytes % 32 == 0) ? 32 : ((addr % 16 == 0 && ld_bytes % 16 == 0) ? 16 : 0);
    const bool vec16 = p.vec_bytes != 0 && cols % 8 == 0;

    if (amax_in) {
        // the quantize kernel copies the value over: no separate copy operation in the stream
        p.amax = amax_in;
        p.amax_store = amax_in != amax_out ? amax_out : nullptr;
    } else {
        FOS_CUDA_TRY(x_dtype == FOS_BF16
                         ? launch_amax<__nv_bfloat16>(x, rows, cols, ld, vec16, amax_out, stream, p.rht != 0, transpose != 0)
                         : launch_amax<__half>(x, rows, cols, ld, vec16, amax_out, stream, p.rht != 0, transpose != 0));
        p.amax = amax_out;
        p.amax_store = nullptr;
    }
    // When this call launched the amax pass itself, the kernel before the quantize kernel is that
    // pass: it does not write x, so x can be fetched while it drains.
    p.x_is_ready = amax_in == nullptr;

    const int kind = format == FOS_IF4 ? KIND_IF4 : (is_static ? KIND_STATIC : KIND_ADAPTIVE);
    FOS_CUDA_TRY(x_dtype == FOS_BF16
                     ? launch_all<__nv_bfloat16>(p, kind, block_2d != 0, transpose != 0, stream)
                     : launch_all<__half>(p, kind, block_2d != 0, transpose != 0, stream));
    return FOS_OK;
}

cudaError_t fos::quantize_wait_failures(int32_t *host_value) { return fos::read_wait_failures(host_value); }
cudaError_t fos::quantize_wait_roles(uint32_t *host_value) { return fos::read_wait_roles(host_value); }

extern "C" int fos_amax(const void *x, int x_dtype, int64_t rows, int64_t cols, int64_t ld, float *amax_out, void *stream_) {
    using namespace fos;
    if (!x || !amax_out) return FOS_ERR_INVALID_ARGUMENT;
    if (rows <= 0 || cols <= 0 || ld < cols) return FOS_ERR_INVALID_ARGUMENT;
    if (x_dtype != FOS_BF16 && x_dtype != FOS_FP16) return FOS_ERR_INVALID_ARGUMENT;
    const int st = check_device();
    if (st != FOS_OK) return st;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    const bool vec16 = reinterpret_cast<uintptr_t>(x) % 16 == 0 && (ld * 2) % 16 == 0 && cols % 8 == 0;
    FOS_CUDA_TRY(x_dtype == FOS_BF16 ? launch_amax<__nv_bfloat16>(x, rows, cols, ld, vec16, amax_out, stream)
                                     : launch_amax<__half>(x, rows, cols, ld, vec16, amax_out, stream));
    return FOS_OK;
}

template <typename T, int KIND>
cudaError_t launch_rows_grouped(const fos::QuantParams &p, cudaStream_t stream, bool *launched) {
    using namespace fos;
    if constexpr (KIND == KIND_ADAPTIVE) {
        if (p.rule == FOS_RULE_MSE && p.variant != 2) return launch_rows_tma_impl<T, KIND, false, false, false, false, true>(p, stream, launched);
    }
    return launch_rows_tma_impl<T, KIND, false, false, false, false>(p, stream, launched);
}

extern "C" int fos_quantize_grouped(const void *x, int x_dtype, int64_t rows_capacity, int64_t cols, int64_t ld, int format,
                                    int scale_rule, const int32_t *group_start, const int32_t *group_rows, int num_groups,
                                    const float *amax_in, uint8_t *codes, uint8_t *sf, float *amax_out, int flags,
                                    void *stream_) {
    using namespace fos;
    if (!x || !codes || !sf || !amax_out || !group_start || !group_rows) return FOS_ERR_INVALID_ARGUMENT;
    if (num_groups <= 0 || num_groups > 65535) return FOS_ERR_INVALID_ARGUMENT;
    if (rows_capacity <= 0 || rows_capacity % 128 || cols <= 0 || ld < cols) return FOS_ERR_INVALID_ARGUMENT;
    if (x_dtype != FOS_BF16 && x_dtype != FOS_FP16) return FOS_ERR_INVALID_ARGUMENT;
    if (scale_rule < FOS_RULE_STATIC_6 || scale_rule > FOS_RULE_ABS_MAX) return FOS_ERR_INVALID_ARGUMENT;
    if (format != FOS_NVFP4 && format != FOS_IF4) return format == FOS_MXFP4 ? FOS_ERR_UNSUPPORTED : FOS_ERR_INVALID_ARGUMENT;
    const bool is_static = scale_rule == FOS_RULE_STATIC_6 || scale_rule == FOS_RULE_STATIC_4;
    if (format == FOS_IF4 && is_static) return FOS_ERR_UNSUPPORTED;
    if (flags & (FOS_QUANTIZE_RHT | FOS_QUANTIZE_NO_TMA | FOS_QUANTIZE_UNBIASED)) return FOS_ERR_UNSUPPORTED;
    // the TMA-fed kernels only: whole 64-value scale tiles per row, 16-byte aligned rows
    if (cols % 64 != 0 || reinterpret_cast<uintptr_t>(x) % 16 != 0 || (ld * 2) % 16 != 0) return FOS_ERR_UNSUPPORTED;
    if (reinterpret_cast<uintptr_t>(codes) % 8 != 0) return FOS_ERR_MISALIGNED;
    if (rows_capacity >= (int64_t(1) << 31)) return FOS_ERR_TOO_LARGE;
    int st = check_device();
    if (st != FOS_OK) return st;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);

    QuantParams p{};
    p.x = x;
    p.rows = rows_capacity; p.cols = cols; p.ld = ld;
    p.out_rows = rows_capacity; p.out_cols = cols;
    p.rows_p = rows_capacity; p.cols_p = cols;
    p.codes = codes; p.sf = sf;
    p.rule = scale_rule;
    p.sf_tiled = 1;
    p.exact_only = (flags & FOS_QUANTIZE_EXACT_ONLY) != 0;
    p.variant = (flags & FOS_QUANTIZE_GENERAL_KERNEL) ? 2 : 0;
    p.vec_bytes = (reinterpret_cast<uintptr_t>(x) % 32 == 0 && (ld * 2) % 32 == 0) ? 32 : 16;
    p.x_is_ready = 1;
    p.group_start = group_start;
    p.num_groups = num_groups;
    if (amax_in) {
        if (amax_in != amax_out)
            FOS_CUDA_TRY(cudaMemcpyAsync(amax_out, amax_in, sizeof(float) * num_groups, cudaMemcpyDeviceToDevice, stream));
    } else {
        FOS_CUDA_TRY(cudaMemsetAsync(amax_out, 0, sizeof(float) * num_groups, stream));
        int dev = 0, sms = 0;
        FOS_CUDA_TRY(cudaGetDevice(&dev));
        FOS_CUDA_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
        int per_group = 8 * sms / num_groups;
        per_group = per_group < 4 ? 4 : per_group;
        const dim3 grid(static_cast<unsigned>(per_group), static_cast<unsigned>(num_groups));
        const int vec = cols % 16 == 0 ? p.vec_bytes : (cols % 8 == 0 ? 16 : 0);
        if (x_dtype == FOS_BF16)
            amax_grouped_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(static_cast<const __nv_bfloat16 *>(x), rows_capacity, cols, ld,
                                                                        vec, group_start, group_rows, amax_out);
        else
            amax_grouped_kernel<__half><<<grid, 256, 0, stream>>>(static_cast<const __half *>(x), rows_capacity, cols, ld, vec,
                                                                 group_start, group_rows, amax_out);
        FOS_CUDA_TRY(cudaGetLastError());
    }
    p.amax = amax_out;
    p.amax_store = nullptr;
    bool launched = false;
    const int kind = format == FOS_IF4 ? KIND_IF4 : (is_static ? KIND_STATIC : KIND_ADAPTIVE);
    cudaError_t e;
    if (x_dtype == FOS_BF16)
        e = kind == KIND_IF4 ? launch_rows_grouped<__nv_bfloat16, KIND_IF4>(p, stream, &launched)
            : kind == KIND_STATIC ? launch_rows_grouped<__nv_bfloat16, KIND_STATIC>(p, stream, &launched)
                                  : launch_rows_grouped<__nv_bfloat16, KIND_ADAPTIVE>(p, stream, &launched);
    else
        e = kind == KIND_IF4 ? launch_rows_grouped<__half, KIND_IF4>(p, stream, &launched)
            : kind == KIND_STATIC ? launch_rows_grouped<__half, KIND_STATIC>(p, stream, &launched)
                                  : launch_rows_grouped<__half, KIND_ADAPTIVE>(p, stream, &launched);
    FOS_CUDA_TRY(e);
    return launched ? FOS_OK : FOS_ERR_UNSUPPORTED;
}

extern "C" int fos_quantize(const void *x, int x_dtype, int64_t rows, int64_t cols, int64_t ld, int format,
                            int scale_rule, int block_2d, int transpose, int sf_layout, const float *amax_in,
                            uint8_t *codes, uint8_t *sf, float *amax_out, int flags, void *stream) {
    return quantize_entry(x, x_dtype, rows, cols, ld, format, scale_rule, block_2d, transpose, sf_layout, amax_in, codes, sf,
                          amax_out, flags, stream, 0, 0);
}

extern "C" int fos_quantize_stochastic(const void *x, int x_dtype, int64_t rows, int64_t cols, int64_t ld, int format,
                                       int scale_rule, int block_2d, int transpose, int sf_layout, const float *amax_in,
                                       uint8_t *codes, uint8_t *sf, float *amax_out, int flags, uint64_t seed, void *stream) {
    return quantize_entry(x, x_dtype, rows, cols, ld, format, scale_rule, block_2d, transpose, sf_layout, amax_in, codes, sf,
                          amax_out, flags, stream, 1, seed);
}
