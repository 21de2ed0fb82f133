// The steps of a mixture-of-experts layer around the two grouped GEMMs:
//
//   fos_experts_route         routing indices -> row ranges per expert and the tables the other kernels take
//   fos_experts_gather_rows   routed tokens -> the padded row buffer the grouped quantization reads
//   fos_experts_glu           gate-up output + bias -> clamped SwiGLU, the input of the down projection
//   fos_experts_combine       down output + bias, times the routing weight, summed per token
//
// The arithmetic follows the reference's GPT-OSS experts module
// (src/fouroversix/model/modules/gpt_oss.py:297-335), which runs it as a chain of element-wise tensor
// operations on 16-bit tensors: every operation computes in binary32 and rounds its result to the
// tensor's type. The kernels keep every one of those roundings, so the results are the bits of that
// chain; what they save is its memory traffic (each operation reads and writes the whole tensor, the
// gathers materialise the bias per row) and its launches. Gather and combine are bound by HBM, the SwiGLU
// by its arithmetic (a sigmoid with an IEEE division and six roundings per output).
#include "fos_common.cuh"

namespace fos {
namespace {

template <typename T> struct Half16;
template <> struct Half16<__nv_bfloat16> {
    using Pair = __nv_bfloat162;
    static __device__ __forceinline__ float lo(uint32_t w) { return __uint_as_float(w << 16); }
    static __device__ __forceinline__ float hi(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }
    static __device__ __forceinline__ float r16(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
    static __device__ __forceinline__ uint32_t pack(float lo_v, float hi_v) {   // round and pack
        Pair p = __floats2bfloat162_rn(lo_v, hi_v);
        return *reinterpret_cast<uint32_t *>(&p);
    }
};
template <> struct Half16<__half> {
    using Pair = __half2;
    static __device__ __forceinline__ float lo(uint32_t w) { return __half2float(__ushort_as_half(static_cast<unsigned short>(w & 0xffffu))); }
    static __device__ __forceinline__ float hi(uint32_t w) { return __half2float(__ushort_as_half(static_cast<unsigned short>(w >> 16))); }
    static __device__ __forceinline__ float r16(float v) { return __half2float(__float2half_rn(v)); }
    static __device__ __forceinline__ uint32_t pack(float lo_v, float hi_v) {
        Pair p = __floats2half2_rn(lo_v, hi_v);
        return *reinterpret_cast<uint32_t *>(&p);
    }
};
template <typename P> __device__ __forceinline__ P as_pair(uint32_t w) { return *reinterpret_cast<P *>(&w); }
template <typename P> __device__ __forceinline__ uint32_t as_word(P p) { return *reinterpret_cast<uint32_t *>(&p); }

__device__ __forceinline__ uint4 ldg_stream(const uint4 *p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.b32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

// max |value| of the eight 16-bit numbers of a 16-byte piece, folded into a running packed maximum
// (NaNs are skipped, as fmaxf skips them in the amax pass of the quantization).
template <typename P> __device__ __forceinline__ P fold_abs_max(P m, uint4 v) {
    m = __hmax2(m, __habs2(as_pair<P>(v.x)));
    m = __hmax2(m, __habs2(as_pair<P>(v.y)));
    m = __hmax2(m, __habs2(as_pair<P>(v.z)));
    return __hmax2(m, __habs2(as_pair<P>(v.w)));
}

// The CTA's maximum of the threads' packed running maxima, raised into amax[0] (a non-negative float, zeroed by the
// caller before the launch, compared as an integer). The words written are the ones the grouped amax pass would
// write: the largest magnitude of the group's values, exactly, as a float. Called by all threads of the CTA.
template <typename T>
__device__ __forceinline__ void raise_amax(typename Half16<T>::Pair m2, float *amax, float *warp_max) {
    using H = Half16<T>;
    float m = fmaxf(H::lo(as_word(m2)), H::hi(as_word(m2)));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    __syncthreads();                                      // the previous row's values have been read
    if ((threadIdx.x & 31) == 0) warp_max[threadIdx.x >> 5] = m;
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < static_cast<int>(blockDim.x >> 5); ++w) m = fmaxf(m, warp_max[w]);
        // (a stale smaller value read here only costs an atomic that changes nothing)
        if (m > 0.0f && m > *reinterpret_cast<volatile float *>(amax)) atomicMax(reinterpret_cast<int *>(amax), __float_as_int(m));
    }
}

// out[r] = x[row_token[r]], or zeros where row_token[r] < 0. One CTA per row at a time, 16 bytes per thread.
// With amax != nullptr also amax[row_expert[r]] = max(amax[..], max |out[r]|): the per-expert maxima the grouped
// quantization of `out` needs, so that it can skip its own pass over the buffer.
template <typename T>
__global__ void __launch_bounds__(256)
gather_rows_kernel(const uint8_t *__restrict__ x, int64_t ld_x_bytes, const int32_t *__restrict__ row_token,
                   uint8_t *__restrict__ out, int64_t ld_out_bytes, int rows, int chunks,
                   const int32_t *__restrict__ row_expert, float *__restrict__ amax) {
    using P = typename Half16<T>::Pair;
    __shared__ float warp_max[8];
    for (int r = blockIdx.x; r < rows; r += gridDim.x) {
        const int t = __ldg(row_token + r);
        const uint4 *src = reinterpret_cast<const uint4 *>(x + static_cast<int64_t>(t < 0 ? 0 : t) * ld_x_bytes);
        uint4 *dst = reinterpret_cast<uint4 *>(out + r * ld_out_bytes);
        P m2 = as_pair<P>(0u);
        for (int c = threadIdx.x; c < chunks; c += blockDim.x) {
            const uint4 v = t < 0 ? make_uint4(0u, 0u, 0u, 0u) : __ldg(src + c);
            dst[c] = v;
            m2 = fold_abs_max<P>(m2, v);
        }
        if (amax != nullptr && t >= 0) raise_amax<T>(m2, amax + __ldg(row_expert + r), warp_max);
    }
}

// The reference's chain on one (gate, up) pair, every intermediate rounded to the 16-bit type:
//   g = gate + bias_g; u = up + bias_u; g = min(g, limit); u = min(max(u, -limit), limit)   (NaN passes through)
//   out = (u + 1) * (g * sigmoid(g * alpha))
// A (gate, up) pair is one 32-bit word, and a packed 16-bit addition, multiplication or fused multiply-add
// rounds once from the exact result, which is what "compute in binary32, round to the type" gives for sums and
// products of 16-bit numbers (their exact value fits binary32, or lies so far from a rounding boundary of the
// 16-bit type that the first rounding cannot move it across). Only g * alpha (alpha is a binary32 number) and
// the sigmoid run in binary32. The _rn forms of the packed operations keep the compiler from contracting a
// multiplication and the addition after it into one fused operation, which would drop a rounding. limit2 = (r, r), floor2 = (-inf, -r) with r the limit rounded to the type:
// comparing with r selects the same values as comparing with the limit itself, because no number of the type
// lies between the two. Returns the output in the low half.
template <typename T>
__device__ __forceinline__ uint32_t glu_word(uint32_t gate_up, uint32_t bias, float alpha,
                                             typename Half16<T>::Pair limit2, typename Half16<T>::Pair floor2,
                                             typename Half16<T>::Pair tail2) {
    using H = Half16<T>;
    using P = typename H::Pair;
    P v = __hadd2_rn(as_pair<P>(gate_up), as_pair<P>(bias));
    v = __hmax2_nan(__hmin2_nan(v, limit2), floor2);
    const float t = H::r16(H::lo(as_word(v)) * alpha);
    const float s = 1.0f / (1.0f + expf(-t));
    // (g, u) * (s, 1) + (-0, 1) = (g * s, u + 1): adding -0 keeps the sign of a zero product
    const uint32_t s1 = (H::pack(s, 0.0f) & 0xffffu) | (as_word(tail2) & 0xffff0000u);
    const P w = __hfma2(v, as_pair<P>(s1), as_pair<P>((as_word(tail2) & 0xffff0000u) | 0x8000u));
    return as_word(__hmul2_rn(w, __lowhigh2highlow(w)));
}

// gate_up [rows][2 * inter] with gate in the even and up in the odd columns; bias [experts][2 * inter];
// out [rows][inter]. A thread makes 8 outputs from 32 bytes of gate_up and 32 bytes of bias.
template <typename T>
__global__ void __launch_bounds__(256)
glu_kernel(const uint8_t *__restrict__ gate_up, int64_t ld_gu_bytes, const uint8_t *__restrict__ bias, int64_t ld_bias_bytes,
           const int32_t *__restrict__ row_expert, uint8_t *__restrict__ out, int64_t ld_out_bytes, int rows, int chunks,
           float alpha, float limit, float *__restrict__ amax) {
    using H = Half16<T>;
    using P = typename H::Pair;
    __shared__ float warp_max[8];
    const float r = H::r16(limit);
    const P limit2 = as_pair<P>(H::pack(r, r)), floor2 = as_pair<P>(H::pack(-INFINITY, -r)), tail2 = as_pair<P>(H::pack(1.0f, 1.0f));
    for (int row = blockIdx.x; row < rows; row += gridDim.x) {
        const int e = __ldg(row_expert + row);
        uint4 *dst = reinterpret_cast<uint4 *>(out + row * ld_out_bytes);
        if (e < 0) {
            for (int c = threadIdx.x; c < chunks; c += blockDim.x) dst[c] = make_uint4(0u, 0u, 0u, 0u);
            continue;
        }
        const uint4 *src = reinterpret_cast<const uint4 *>(gate_up + row * ld_gu_bytes);
        const uint4 *b = reinterpret_cast<const uint4 *>(bias + e * ld_bias_bytes);
        P m2 = as_pair<P>(0u);
        for (int c = threadIdx.x; c < chunks; c += blockDim.x) {
            const uint4 v0 = ldg_stream(src + 2 * c), v1 = ldg_stream(src + 2 * c + 1);
            const uint4 b0 = __ldg(b + 2 * c), b1 = __ldg(b + 2 * c + 1);
            const uint32_t v[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
            const uint32_t bb[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
            uint32_t o[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) o[i] = glu_word<T>(v[i], bb[i], alpha, limit2, floor2, tail2);
            const uint4 packed = make_uint4(__byte_perm(o[0], o[1], 0x5410), __byte_perm(o[2], o[3], 0x5410),
                                            __byte_perm(o[4], o[5], 0x5410), __byte_perm(o[6], o[7], 0x5410));
            dst[c] = packed;
            m2 = fold_abs_max<P>(m2, packed);
        }
        if (amax != nullptr) raise_amax<T>(m2, amax + e, warp_max);     // (e is the same for the whole CTA: no divergence)
    }
}

constexpr int MAX_TOP_K = 8;

// out[t] = sum over the token's experts, in ascending order of the expert's index (the order in which the
// reference's host loop adds them into the 16-bit result), of (y[row] + bias[expert]) * weight, every
// operation rounded to the 16-bit type, the running sum too (packed 16-bit arithmetic: see glu_word).
template <typename T>
__global__ void __launch_bounds__(256)
combine_kernel(const uint8_t *__restrict__ y, int64_t ld_y_bytes, const uint8_t *__restrict__ bias, int64_t ld_bias_bytes,
               const int32_t *__restrict__ pair_row, const int32_t *__restrict__ pair_expert,
               const uint16_t *__restrict__ pair_weight, int top_k, uint8_t *__restrict__ out, int64_t ld_out_bytes, int tokens,
               int chunks) {
    using P = typename Half16<T>::Pair;
    __shared__ int s_row[MAX_TOP_K], s_ex[MAX_TOP_K];
    __shared__ uint32_t s_w[MAX_TOP_K];
    for (int t = blockIdx.x; t < tokens; t += gridDim.x) {
        __syncthreads();                                  // the previous token's slots have been read
        if (threadIdx.x == 0) {                           // insertion sort of the token's slots by expert
            for (int k = 0; k < top_k; ++k) {
                const int64_t i = static_cast<int64_t>(t) * top_k + k;
                const int e = __ldg(pair_expert + i), r = __ldg(pair_row + i);
                const uint32_t w = __ldg(pair_weight + i);
                int j = k;
                for (; j > 0 && s_ex[j - 1] > e; --j) { s_ex[j] = s_ex[j - 1]; s_row[j] = s_row[j - 1]; s_w[j] = s_w[j - 1]; }
                s_ex[j] = e; s_row[j] = r; s_w[j] = w | (w << 16);
            }
        }
        __syncthreads();
        uint4 *dst = reinterpret_cast<uint4 *>(out + t * ld_out_bytes);
        for (int c = threadIdx.x; c < chunks; c += blockDim.x) {
            uint32_t acc[4] = {0u, 0u, 0u, 0u};
            for (int k = 0; k < top_k; ++k) {
                if (s_row[k] < 0) continue;               // a slot whose expert index was out of range
                const uint4 v = ldg_stream(reinterpret_cast<const uint4 *>(y + s_row[k] * ld_y_bytes) + c);
                const uint4 b = __ldg(reinterpret_cast<const uint4 *>(bias + s_ex[k] * ld_bias_bytes) + c);
                const P w2 = as_pair<P>(s_w[k]);
                const uint32_t vv[4] = {v.x, v.y, v.z, v.w}, bb[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
                for (int i = 0; i < 4; ++i)
                    acc[i] = as_word(__hadd2_rn(as_pair<P>(acc[i]), __hmul2_rn(__hadd2_rn(as_pair<P>(vv[i]), as_pair<P>(bb[i])), w2)));
            }
            dst[c] = make_uint4(acc[0], acc[1], acc[2], acc[3]);
        }
    }
}

constexpr int ROUTE_THREADS = 256, ROUTE_WARPS = ROUTE_THREADS / 32, ROUTE_MAX_EXPERTS = 256, ROUTE_MAX_SEGMENTS = 128;

// The routing tables of one layer call: a stable counting sort of the (token, slot) pairs by expert, in two
// launches of one CTA per SEGMENT of the pairs (contiguous, `seg` pairs each).
//   group_rows[e]   pairs routed to expert e           group_start[e]  first row of expert e in the padded buffer
//   pair_row[p]     the row pair p was given (ascending in p within an expert), -1 for an index outside [0, experts)
//   row_token[r], row_expert[r]   the token and the expert of row r, -1 for padding rows
// route_count_kernel: every CTA counts its segment per expert into seg_count[segment][expert], and the CTAs
// together fill the row tables with -1. route_place_kernel: every CTA adds up the counts of all segments (totals,
// hence the experts' first rows) and of the segments before its own (hence its own first row per expert), splits
// its segment over its warps the same way (count, running sum), and then each warp walks its pairs 32 at a
// time, ranks the pairs of one expert among themselves with match_any and advances its own counters. Rows
// ascend with the pair index because segments, warps and lanes do.
template <typename IDX>
__device__ __forceinline__ int route_expert_of(const IDX *__restrict__ routing, int p, int end, int experts) {
    if (p >= end) return -1;
    const long long e = static_cast<long long>(routing[p]);
    return (e >= 0 && e < experts) ? static_cast<int>(e) : -1;
}

template <typename IDX>
__global__ void __launch_bounds__(ROUTE_THREADS)
route_count_kernel(const IDX *__restrict__ routing, int pairs, int seg, int experts, int rows_capacity,
                   int32_t *__restrict__ seg_count, int32_t *__restrict__ row_token, int32_t *__restrict__ row_expert) {
    __shared__ int s_count[ROUTE_MAX_EXPERTS];
    const int tid = threadIdx.x;
    s_count[tid] = 0;
    for (int r = blockIdx.x * ROUTE_THREADS + tid; r < rows_capacity; r += gridDim.x * ROUTE_THREADS) {
        row_token[r] = -1;
        row_expert[r] = -1;
    }
    __syncthreads();
    const int p0 = blockIdx.x * seg, p1 = min(pairs, p0 + seg);
    for (int base = p0; base < p1; base += 4 * ROUTE_THREADS) {       // four independent loads in flight per thread
        int e[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) e[u] = route_expert_of(routing, base + u * ROUTE_THREADS + tid, p1, experts);
#pragma unroll
        for (int u = 0; u < 4; ++u)
            if (e[u] >= 0) atomicAdd(&s_count[e[u]], 1);
    }
    __syncthreads();
    if (tid < experts) seg_count[blockIdx.x * experts + tid] = s_count[tid];
}

template <typename IDX>
__global__ void __launch_bounds__(ROUTE_THREADS)
route_place_kernel(const IDX *__restrict__ routing, int pairs, int seg, int top_k, int experts,
                   const int32_t *__restrict__ seg_count, int32_t *__restrict__ group_start,
                   int32_t *__restrict__ group_rows, int32_t *__restrict__ row_token, int32_t *__restrict__ row_expert,
                   int32_t *__restrict__ pair_row, int32_t *__restrict__ pair_expert) {
    __shared__ int s_at[ROUTE_WARPS][ROUTE_MAX_EXPERTS];     // counts, then next rows, per (warp, expert)
    __shared__ int s_total[ROUTE_MAX_EXPERTS], s_first[ROUTE_MAX_EXPERTS];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    for (int w = 0; w < ROUTE_WARPS; ++w) s_at[w][tid] = 0;
    int before = 0;
    if (tid < experts) {
        int total = 0;
        for (int sgm = 0; sgm < static_cast<int>(gridDim.x); ++sgm) {
            const int n = __ldg(seg_count + sgm * experts + tid);
            total += n;
            if (sgm < static_cast<int>(blockIdx.x)) before += n;
        }
        s_total[tid] = total;
    }
    __syncthreads();
    if (tid == 0) {
        int at = 0;
        for (int e = 0; e < experts; ++e) {
            s_first[e] = at;
            if (blockIdx.x == 0) {
                group_start[e] = at;
                group_rows[e] = s_total[e];
            }
            at += (s_total[e] + 127) / 128 * 128;
        }
        if (blockIdx.x == 0) group_start[experts] = at;
    }
    // this CTA's segment over its warps: count ...
    const int p0 = blockIdx.x * seg, p1 = min(pairs, p0 + seg);
    const int wseg = ((p1 > p0 ? p1 - p0 : 0) + ROUTE_WARPS - 1) / ROUTE_WARPS;
    const int w0 = p0 + warp * wseg, w1 = min(p1, w0 + wseg);
    for (int base = w0; base < w1; base += 128) {
        int e[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) e[u] = route_expert_of(routing, base + 32 * u + lane, w1, experts);
#pragma unroll
        for (int u = 0; u < 4; ++u)
            if (e[u] >= 0) atomicAdd(&s_at[warp][e[u]], 1);
    }
    __syncthreads();
    // ... running sum from the expert's first row and the rows of the segments before this one ...
    if (tid < experts) {
        int at = s_first[tid] + before;
        for (int w = 0; w < ROUTE_WARPS; ++w) {
            const int n = s_at[w][tid];
            s_at[w][tid] = at;
            at += n;
        }
    }
    __syncthreads();
    // ... and place
    int e_next = route_expert_of(routing, w0 + lane, w1, experts);
    for (int base = w0; base < w1; base += 32) {
        const int p = base + lane, e = e_next;
        e_next = route_expert_of(routing, p + 32, w1, experts);      // the next round's load overlaps this round's work
        const uint32_t same = __match_any_sync(0xffffffffu, e);
        const int rank = __popc(same & ((1u << lane) - 1u));
        int row = -1;
        if (e >= 0) row = s_at[warp][e] + rank;
        __syncwarp();
        if (e >= 0 && rank == 0) s_at[warp][e] += __popc(same);
        __syncwarp();
        if (p < w1) {
            pair_row[p] = row;
            pair_expert[p] = e;
            if (e >= 0) {
                row_token[row] = p / top_k;
                row_expert[row] = e;
            }
        }
    }
}

// Threads per CTA for rows of `chunks` 16-byte pieces: the multiple of 32 up to 256 that leaves the fewest
// idle threads in a row's last round (the larger on a tie).
inline unsigned threads_for(int chunks) {
    unsigned best = 256;
    double best_eff = 0.0;
    for (unsigned t = 64; t <= 256; t += 32) {
        const double eff = static_cast<double>(chunks) / (static_cast<double>((chunks + t - 1) / t) * t);
        if (eff >= best_eff) { best_eff = eff; best = t; }
    }
    return best;
}

inline bool aligned16(const void *p, int64_t ld_bytes) {
    return reinterpret_cast<uintptr_t>(p) % 16 == 0 && ld_bytes % 16 == 0;
}

inline unsigned grid_for(int64_t rows) {
    const int64_t cap = 148 * 8;
    return static_cast<unsigned>(rows < cap ? rows : cap);
}

}  // namespace
}  // namespace fos

extern "C" int fos_experts_gather_rows(const void *x, int dtype, int64_t ld_x, const int32_t *row_token, void *out,
                                       int64_t ld_out, int64_t rows_capacity, int64_t cols, const int32_t *row_expert,
                                       float *amax, void *stream_) {
    using namespace fos;
    if (!x || !row_token || !out || rows_capacity <= 0 || cols <= 0 || ld_x < cols || ld_out < cols) return FOS_ERR_INVALID_ARGUMENT;
    if ((amax != nullptr) != (row_expert != nullptr)) return FOS_ERR_INVALID_ARGUMENT;
    if (dtype != FOS_BF16 && dtype != FOS_FP16) return FOS_ERR_UNSUPPORTED;
    if (cols % 8 != 0 || rows_capacity >= (int64_t(1) << 31)) return FOS_ERR_UNSUPPORTED;
    if (!aligned16(x, ld_x * 2) || !aligned16(out, ld_out * 2)) return FOS_ERR_MISALIGNED;
    const int st = check_device();
    if (st != FOS_OK) return st;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    const unsigned g = grid_for(rows_capacity), threads = threads_for(static_cast<int>(cols / 8));
    if (dtype == FOS_BF16)
        gather_rows_kernel<__nv_bfloat16><<<g, threads, 0, stream>>>(static_cast<const uint8_t *>(x), ld_x * 2, row_token,
                                                                     static_cast<uint8_t *>(out), ld_out * 2, static_cast<int>(rows_capacity),
                                                                     static_cast<int>(cols / 8), row_expert, amax);
    else
        gather_rows_kernel<__half><<<g, threads, 0, stream>>>(static_cast<const uint8_t *>(x), ld_x * 2, row_token,
                                                              static_cast<uint8_t *>(out), ld_out * 2, static_cast<int>(rows_capacity),
                                                              static_cast<int>(cols / 8), row_expert, amax);
    FOS_CUDA_TRY(cudaGetLastError());
    return FOS_OK;
}

extern "C" int fos_experts_glu(const void *gate_up, int dtype, int64_t ld_gate_up, const void *bias, const int32_t *row_expert,
                               void *out, int64_t ld_out, int64_t rows_capacity, int64_t intermediate, float alpha,
                               float limit, float *amax, void *stream_) {
    using namespace fos;
    if (!gate_up || !bias || !row_expert || !out || rows_capacity <= 0 || intermediate <= 0 ||
        ld_gate_up < 2 * intermediate || ld_out < intermediate)
        return FOS_ERR_INVALID_ARGUMENT;
    if (dtype != FOS_BF16 && dtype != FOS_FP16) return FOS_ERR_UNSUPPORTED;
    if (intermediate % 8 != 0 || rows_capacity >= (int64_t(1) << 31)) return FOS_ERR_UNSUPPORTED;
    if (!aligned16(gate_up, ld_gate_up * 2) || !aligned16(out, ld_out * 2) || !aligned16(bias, 2 * intermediate * 2))
        return FOS_ERR_MISALIGNED;
    const int st = check_device();
    if (st != FOS_OK) return st;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    const unsigned g = grid_for(rows_capacity);
    const int rows = static_cast<int>(rows_capacity), chunks = static_cast<int>(intermediate / 8);
    if (dtype == FOS_BF16)
        glu_kernel<__nv_bfloat16><<<g, threads_for(chunks), 0, stream>>>(static_cast<const uint8_t *>(gate_up), ld_gate_up * 2,
                                                           static_cast<const uint8_t *>(bias), 2 * intermediate * 2, row_expert,
                                                           static_cast<uint8_t *>(out), ld_out * 2, rows, chunks, alpha, limit, amax);
    else
        glu_kernel<__half><<<g, threads_for(chunks), 0, stream>>>(static_cast<const uint8_t *>(gate_up), ld_gate_up * 2,
                                                    static_cast<const uint8_t *>(bias), 2 * intermediate * 2, row_expert,
                                                    static_cast<uint8_t *>(out), ld_out * 2, rows, chunks, alpha, limit, amax);
    FOS_CUDA_TRY(cudaGetLastError());
    return FOS_OK;
}

extern "C" int fos_experts_combine(const void *y, int dtype, int64_t ld_y, const void *bias, const int32_t *pair_row,
                                   const int32_t *pair_expert, const void *pair_weight, int top_k, void *out,
                                   int64_t ld_out, int64_t tokens, int64_t hidden, void *stream_) {
    using namespace fos;
    if (!y || !bias || !pair_row || !pair_expert || !pair_weight || !out || tokens <= 0 || hidden <= 0 || top_k <= 0 ||
        ld_y < hidden || ld_out < hidden)
        return FOS_ERR_INVALID_ARGUMENT;
    if (dtype != FOS_BF16 && dtype != FOS_FP16) return FOS_ERR_UNSUPPORTED;
    if (top_k > MAX_TOP_K || hidden % 8 != 0 || tokens >= (int64_t(1) << 31)) return FOS_ERR_UNSUPPORTED;
    if (!aligned16(y, ld_y * 2) || !aligned16(out, ld_out * 2) || !aligned16(bias, hidden * 2)) return FOS_ERR_MISALIGNED;
    const int st = check_device();
    if (st != FOS_OK) return st;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    const unsigned g = grid_for(tokens);
    const int n = static_cast<int>(tokens), chunks = static_cast<int>(hidden / 8);
    if (dtype == FOS_BF16)
        combine_kernel<__nv_bfloat16><<<g, threads_for(chunks), 0, stream>>>(static_cast<const uint8_t *>(y), ld_y * 2,
                                                               static_cast<const uint8_t *>(bias), hidden * 2, pair_row, pair_expert,
                                                               static_cast<const uint16_t *>(pair_weight), top_k,
                                                               static_cast<uint8_t *>(out), ld_out * 2, n, chunks);
    else
        combine_kernel<__half><<<g, threads_for(chunks), 0, stream>>>(static_cast<const uint8_t *>(y), ld_y * 2,
                                                        static_cast<const uint8_t *>(bias), hidden * 2, pair_row, pair_expert,
                                                        static_cast<const uint16_t *>(pair_weight), top_k,
                                                        static_cast<uint8_t *>(out), ld_out * 2, n, chunks);
    FOS_CUDA_TRY(cudaGetLastError());
    return FOS_OK;
}

extern "C" int fos_experts_route(const void *routing_indices, int index_bytes, int64_t tokens, int top_k, int num_experts,
                                 int64_t rows_capacity, int32_t *group_start, int32_t *group_rows, int32_t *row_token,
                                 int32_t *row_expert, int32_t *pair_row, int32_t *pair_expert, int32_t *workspace,
                                 void *stream_) {
    using namespace fos;
    if (!routing_indices || !group_start || !group_rows || !row_token || !row_expert || !pair_row || !pair_expert ||
        !workspace || tokens <= 0 || top_k <= 0 || num_experts <= 0 || (index_bytes != 4 && index_bytes != 8))
        return FOS_ERR_INVALID_ARGUMENT;
    if (num_experts > ROUTE_MAX_EXPERTS) return FOS_ERR_UNSUPPORTED;
    const int64_t pairs64 = tokens * top_k;
    if (pairs64 >= (int64_t(1) << 30) || rows_capacity >= (int64_t(1) << 31)) return FOS_ERR_TOO_LARGE;
    if (rows_capacity % 128 != 0 || rows_capacity < round_up64(pairs64 + 127 * static_cast<int64_t>(num_experts), 128))
        return FOS_ERR_INVALID_ARGUMENT;
    const int st = check_device();
    if (st != FOS_OK) return st;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    // segments of at least 512 pairs, at most ROUTE_MAX_SEGMENTS of them
    const int pairs = static_cast<int>(pairs64), cap = static_cast<int>(rows_capacity);
    int segments = (pairs + 511) / 512;
    if (segments > ROUTE_MAX_SEGMENTS) segments = ROUTE_MAX_SEGMENTS;
    const int seg = (pairs + segments - 1) / segments;
    segments = (pairs + seg - 1) / seg;
    if (index_bytes == 8) {
        const int64_t *idx = static_cast<const int64_t *>(routing_indices);
        route_count_kernel<int64_t><<<segments, ROUTE_THREADS, 0, stream>>>(idx, pairs, seg, num_experts, cap, workspace, row_token, row_expert);
        route_place_kernel<int64_t><<<segments, ROUTE_THREADS, 0, stream>>>(idx, pairs, seg, top_k, num_experts, workspace, group_start,
                                                                            group_rows, row_token, row_expert, pair_row, pair_expert);
    } else {
        const int32_t *idx = static_cast<const int32_t *>(routing_indices);
        route_count_kernel<int32_t><<<segments, ROUTE_THREADS, 0, stream>>>(idx, pairs, seg, num_experts, cap, workspace, row_token, row_expert);
        route_place_kernel<int32_t><<<segments, ROUTE_THREADS, 0, stream>>>(idx, pairs, seg, top_k, num_experts, workspace, group_start,
                                                                            group_rows, row_token, row_expert, pair_row, pair_expert);
    }
    FOS_CUDA_TRY(cudaGetLastError());
    return FOS_OK;
}

// ---------------------------------------------------------------------------- the whole layer in one call

namespace fos {
namespace {

struct ExpertsWorkspace {
    int64_t capacity, pairs;
    // byte offsets into the workspace, each a multiple of 256
    int64_t group_start, group_rows, row_token, row_expert, pair_row, pair_expert, route_work, amax, alpha;
    int64_t rows_x, codes_x, sf_x, gate_up, gated, codes_g, sf_g, y, total;
};

ExpertsWorkspace experts_workspace(int64_t tokens, int top_k, int num_experts, int64_t hidden, int64_t intermediate) {
    ExpertsWorkspace w{};
    w.pairs = tokens * top_k;
    w.capacity = round_up64(w.pairs + 127 * static_cast<int64_t>(num_experts), 128);
    int64_t at = 0;
    auto take = [&](int64_t bytes) { const int64_t here = at; at += round_up64(bytes, 256); return here; };
    w.group_start = take(4 * (num_experts + 1));
    w.group_rows = take(4 * num_experts);
    w.row_token = take(4 * w.capacity);
    w.row_expert = take(4 * w.capacity);
    w.pair_row = take(4 * w.pairs);
    w.pair_expert = take(4 * w.pairs);
    w.route_work = take(4 * static_cast<int64_t>(FOS_EXPERTS_ROUTE_WORKSPACE_INTS) * num_experts);
    w.amax = take(4 * 2 * num_experts);
    w.alpha = take(4 * 2 * num_experts);
    w.rows_x = take(2 * w.capacity * hidden);
    w.codes_x = take(w.capacity * hidden / 2);
    w.sf_x = take(w.capacity * hidden / 16);
    w.gate_up = take(2 * w.capacity * 2 * intermediate);
    w.gated = take(2 * w.capacity * intermediate);
    w.codes_g = take(w.capacity * intermediate / 2);
    w.sf_g = take(w.capacity * intermediate / 16);
    w.y = take(2 * w.capacity * hidden);
    w.total = at;
    return w;
}

}  // namespace
}  // namespace fos

extern "C" int64_t fos_experts_workspace_bytes(int64_t tokens, int top_k, int num_experts, int64_t hidden, int64_t intermediate) {
    if (tokens <= 0 || top_k <= 0 || num_experts <= 0 || hidden <= 0 || intermediate <= 0) return FOS_ERR_INVALID_ARGUMENT;
    return fos::experts_workspace(tokens, top_k, num_experts, hidden, intermediate).total;
}

extern "C" int fos_experts_forward(const void *x, int dtype, int64_t tokens, int64_t hidden, int64_t ld_x,
                                   const void *routing_indices, int index_bytes, const void *routing_weights, int top_k,
                                   int num_experts, const uint8_t *gate_up_codes, const uint8_t *gate_up_sf,
                                   const float *gate_up_amax, const void *gate_up_bias, const uint8_t *down_codes,
                                   const uint8_t *down_sf, const float *down_amax, const void *down_bias,
                                   int64_t intermediate, int weight_rule, int activation_rule, float alpha, float limit,
                                   void *out, int64_t ld_out, void *workspace, int64_t workspace_bytes, int32_t *status,
                                   void *stream_) {
    using namespace fos;
    if (!x || !routing_indices || !routing_weights || !gate_up_codes || !gate_up_sf || !gate_up_amax || !gate_up_bias ||
        !down_codes || !down_sf || !down_amax || !down_bias || !out || !workspace || tokens <= 0 || hidden <= 0 ||
        intermediate <= 0 || top_k <= 0 || num_experts <= 0)
        return FOS_ERR_INVALID_ARGUMENT;
    if (dtype != FOS_BF16 && dtype != FOS_FP16) return FOS_ERR_UNSUPPORTED;
    // whole 64-value scale tiles along both reduction dimensions (the packed weights are then not padded along K)
    if (hidden % 64 != 0 || intermediate % 64 != 0 || num_experts > 256 || top_k > MAX_TOP_K) return FOS_ERR_UNSUPPORTED;
    if (reinterpret_cast<uintptr_t>(workspace) % 256 != 0) return FOS_ERR_MISALIGNED;
    const ExpertsWorkspace w = experts_workspace(tokens, top_k, num_experts, hidden, intermediate);
    if (workspace_bytes < w.total) return FOS_ERR_INVALID_ARGUMENT;
    uint8_t *base = static_cast<uint8_t *>(workspace);
    auto ints = [&](int64_t off) { return reinterpret_cast<int32_t *>(base + off); };
    float *amax = reinterpret_cast<float *>(base + w.amax), *alphas = reinterpret_cast<float *>(base + w.alpha);
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    const int64_t gate_up_rows = round_up64(2 * intermediate, 128), down_rows = round_up64(hidden, 128);

    int st = fos_experts_route(routing_indices, index_bytes, tokens, top_k, num_experts, w.capacity, ints(w.group_start),
                               ints(w.group_rows), ints(w.row_token), ints(w.row_expert), ints(w.pair_row),
                               ints(w.pair_expert), ints(w.route_work), stream_);
    if (st != FOS_OK) return st;
    FOS_CUDA_TRY(cudaMemsetAsync(amax, 0, sizeof(float) * 2 * num_experts, stream));
    st = fos_experts_gather_rows(x, dtype, ld_x, ints(w.row_token), base + w.rows_x, hidden, w.capacity, hidden,
                                 ints(w.row_expert), amax, stream_);
    if (st != FOS_OK) return st;
    st = fos_quantize_grouped(base + w.rows_x, dtype, w.capacity, hidden, hidden, FOS_NVFP4, activation_rule, ints(w.group_start),
                              ints(w.group_rows), num_experts, amax, base + w.codes_x, base + w.sf_x, amax, 0, stream_);
    if (st != FOS_OK) return st;
    st = fos_gemm_alpha_grouped(amax, FOS_NVFP4, activation_rule, 0, gate_up_amax, FOS_NVFP4, weight_rule, 0, alphas, num_experts, stream_);
    if (st != FOS_OK) return st;
    st = fos_gemm_nvfp4_grouped(base + w.codes_x, base + w.sf_x, gate_up_codes, gate_up_sf, alphas, base + w.gate_up, dtype,
                                ints(w.group_start), ints(w.group_rows), num_experts, w.capacity, gate_up_rows, hidden,
                                2 * intermediate, 2 * intermediate, nullptr, status, stream_);
    if (st != FOS_OK) return st;
    st = fos_experts_glu(base + w.gate_up, dtype, 2 * intermediate, gate_up_bias, ints(w.row_expert), base + w.gated, intermediate,
                         w.capacity, intermediate, alpha, limit, amax + num_experts, stream_);
    if (st != FOS_OK) return st;
    st = fos_quantize_grouped(base + w.gated, dtype, w.capacity, intermediate, intermediate, FOS_NVFP4, activation_rule,
                              ints(w.group_start), ints(w.group_rows), num_experts, amax + num_experts, base + w.codes_g,
                              base + w.sf_g, amax + num_experts, 0, stream_);
    if (st != FOS_OK) return st;
    st = fos_gemm_alpha_grouped(amax + num_experts, FOS_NVFP4, activation_rule, 0, down_amax, FOS_NVFP4, weight_rule, 0,
                                alphas + num_experts, num_experts, stream_);
    if (st != FOS_OK) return st;
    st = fos_gemm_nvfp4_grouped(base + w.codes_g, base + w.sf_g, down_codes, down_sf, alphas + num_experts, base + w.y, dtype,
                                ints(w.group_start), ints(w.group_rows), num_experts, w.capacity, down_rows, intermediate,
                                hidden, hidden, nullptr, status, stream_);
    if (st != FOS_OK) return st;
    return fos_experts_combine(base + w.y, dtype, hidden, down_bias, ints(w.pair_row), ints(w.pair_expert), routing_weights,
                               top_k, out, ld_out, tokens, hidden, stream_);
}
