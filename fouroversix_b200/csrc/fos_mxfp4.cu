// MXFP4 for sm_100a: E2M1 values with one E8M0 (power-of-two) scale per 32 values, no per-tensor
// scale. Follows src/fouroversix/quantize/pytorch/reference.py:149-181 (quantize_to_mxfp4) and
// QuantizeBackendBase.dequantize (src/fouroversix/quantize/backend.py:88-160):
//
//   scale exponent e = biased exponent of (max|x| / maxq), plus one unless that quotient is a power
//                      of two; maxq = 6 (static_6) or 4 (static_4); byte 0 for an all-zero block
//   codes            = E2M1(x / 2^(e-127)), round to nearest even
//   dequantized      = fp16(value) * fp16(2^(e-127)) in fp16, cast to the output type
//
// One pass over x (there is no tensor-wide maximum to wait for), so the kernel's floor is the plain
// HBM time of 2 B read + 0.5 B codes + 1/32 B scale per element.
//
// quantize_mx_kernel: a CTA of 256 threads takes 128 x 128 tiles of the OUTPUT (x transposed when
// asked). A thread owns runs of 16 values; two neighbouring lanes make a block. Untransposed 1-D
// blocks go global -> registers (32 bytes per lane, 256 contiguous bytes per quarter warp, the four
// loads of a thread in flight together, four CTAs per SM);
// transposed input and 32 x 32 blocks go through a shared-memory copy of the tile.
#include "fos_common.cuh"

namespace fos {
namespace {

constexpr int MX_TILE = 128;
constexpr int MX_PITCH = MX_TILE + 2;      // elements; 65 words per row: transposed writes spread over the banks
constexpr int MX_THREADS = 256;

struct MxParams {
    const void *x;
    int64_t rows, cols, ld;          // x as given
    int64_t out_rows, out_cols;      // Y = x or x^T
    int64_t rows_p, cols_p;          // padded to multiples of 128
    uint8_t *codes;
    uint8_t *sf;
    float *amax_out;                 // receives 1.0, the per-tensor scale the reference reports for this format
    float inv_maxq_is_quarter;       // 1 for static_4 (divide by 4), 0 for static_6
    int sf_tiled;
    int vec16;                       // x base and row stride are 16-byte aligned
    int vec32;                       // ... and 32-byte aligned
};

// Scale byte of a block with maximum `bmax` and the factor 2^(127-e) that divides by the scale.
__device__ __forceinline__ uint32_t mx_scale(float bmax, bool quarter, float &inv) {
    const float hp = quarter ? bmax * 0.25f : div6_exact(bmax);
    const uint32_t bits = __float_as_uint(hp);
    uint32_t e = (bits >> 23) & 0xffu;
    if (bits & 0x7fffffu) e = (e + 1u) & 0xffu;
    // 2^(127-e): a normal number up to e = 253, the subnormal 2^-127 for e = 254; an all-zero
    // block (e = 0) quantizes to zeros whatever the factor
    inv = e == 0u ? 0.0f : __uint_as_float(e < 254u ? (254u - e) << 23 : 0x00400000u);
    return e;
}

// Sixteen values times `inv` -> 8 bytes of codes. The reference multiplies the rounded magnitude
// by sign(x / scale), so a quotient that IS zero (from -0, or from a negative value that
// underflows) encodes as +0 while a negative quotient that only ROUNDS to zero keeps its sign:
// round the product first, then add +0.
__device__ __forceinline__ uint2 mx_encode16(const float (&v)[16], float inv) {
    float s[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) s[i] = __fadd_rn(__fmul_rn(v[i], inv), 0.0f);
    return make_uint2(cvt_e2m1x8(s), cvt_e2m1x8(s + 8));
}

template <typename T>
__device__ __forceinline__ float unpack16(const uint32_t (&w)[8], float (&v)[16]) {
    float m = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const float2 f = unpack2<T>(w[i]);
        v[2 * i] = f.x; v[2 * i + 1] = f.y;
        m = fmaxf(m, fmaxf(fabsf(f.x), fabsf(f.y)));
    }
    return m;
}

template <typename T, bool TWO_D, bool TRANSPOSED>
__global__ void __launch_bounds__(MX_THREADS, 4)
quantize_mx_kernel(const MxParams p) {
    constexpr bool STAGED = TWO_D || TRANSPOSED;
    __shared__ __align__(16) T tile[STAGED ? MX_TILE * MX_PITCH : 1];
    __shared__ float piece_max[TWO_D ? MX_TILE * 8 : 1];
    __shared__ float block_max[TWO_D ? 16 : 1];
    const T *x = static_cast<const T *>(p.x);
    const int tid = threadIdx.x;
    const int64_t tiles_c = p.cols_p / MX_TILE, n_tiles = (p.rows_p / MX_TILE) * tiles_c;
    const int64_t n_cb = p.cols_p / 32;
    const bool quarter = p.inv_maxq_is_quarter != 0.0f;
    if (blockIdx.x == 0 && tid == 0) *p.amax_out = 1.0f;

    // run `it` of a thread: row 32 * it + tid / 8 of the tile, columns 16 * (tid % 8) .. + 15. What
    // depends on the thread alone is computed once (and made opaque, or the compiler recomputes it).
    const int r0 = tid >> 3, piece = tid & 7;
    const int64_t code_ld = p.cols_p / 2;
    int64_t x_thr = r0 * p.ld + piece * 16, code_thr = r0 * code_ld + piece * 8;
    int64_t sf_thr = p.sf_tiled ? r0 * 16 + (piece >> 1) : r0 * n_cb + (piece >> 1);
    asm volatile("" : "+l"(x_thr), "+l"(code_thr), "+l"(sf_thr));
    const int64_t x_it = 32 * p.ld, code_it = 32 * code_ld, sf_it = p.sf_tiled ? 4 : 32 * n_cb;

    for (int64_t t = blockIdx.x; t < n_tiles; t += gridDim.x) {
        // tile origin in Y (a 32-bit division when the tile count allows it, which is always in practice: the
        // 64-bit form costs about as much as quantizing one of the thread's four runs)
        const int64_t t_row = n_tiles < (int64_t(1) << 31) ? static_cast<int64_t>(static_cast<uint32_t>(t) / static_cast<uint32_t>(tiles_c))
                                                          : t / tiles_c;
        const int64_t i0 = t_row * MX_TILE, j0 = (t - t_row * tiles_c) * MX_TILE;

        if constexpr (STAGED) {
            // copy the tile of Y into shared memory; global reads run along x's rows either way
            __syncthreads();                               // the previous tile's readers are done
            // x rows a0.., x columns b0..: for Y = x^T the tile of Y is x[j0.., i0..]^T
            const int64_t a0 = TRANSPOSED ? j0 : i0, b0 = TRANSPOSED ? i0 : j0;
            // A warp takes 8 rows of x by 4 chunks of 8 columns at a time: lanes 0-7 the rows, lane / 8
            // the chunk. Global: 64 contiguous bytes per row. Shared, transposed: the 8 lanes of a chunk
            // write 8 neighbouring columns of one tile row and the four chunks land 8 tile rows (8 x 65
            // words) apart, on four different bank groups: no conflicts.
            const int lane = tid & 31, wrp = tid >> 5;
            uint4 raw[8];
#pragma unroll
            for (int q = 0; q < 8; ++q) {
                const int task = q * (MX_THREADS / 32) + wrp;
                const int ar = (task >> 2) * 8 + (lane & 7), bc = ((task & 3) * 4 + (lane >> 3)) * 8;
                const int64_t a = a0 + ar, b = b0 + bc;
                if (a < p.rows && b + 8 <= p.cols && p.vec16) {
                    raw[q] = ldg_nc_16(x + a * p.ld + b);
                } else {
                    const uint16_t *xs = reinterpret_cast<const uint16_t *>(x);
                    uint32_t h[8];
#pragma unroll
                    for (int k = 0; k < 8; ++k) h[k] = (a < p.rows && b + k < p.cols) ? xs[a * p.ld + b + k] : 0u;
                    raw[q] = make_uint4(h[0] | (h[1] << 16), h[2] | (h[3] << 16), h[4] | (h[5] << 16), h[6] | (h[7] << 16));
                }
            }
            uint16_t *tile16 = reinterpret_cast<uint16_t *>(tile);
#pragma unroll
            for (int q = 0; q < 8; ++q) {
                const int task = q * (MX_THREADS / 32) + wrp;
                const int ar = (task >> 2) * 8 + (lane & 7), bc = ((task & 3) * 4 + (lane >> 3)) * 8;
                const uint32_t wv[4] = {raw[q].x, raw[q].y, raw[q].z, raw[q].w};
                if constexpr (TRANSPOSED) {
#pragma unroll
                    for (int k = 0; k < 8; ++k)
                        tile16[(bc + k) * MX_PITCH + ar] = static_cast<uint16_t>(wv[k >> 1] >> ((k & 1) * 16));
                } else {
                    uint32_t *dst = reinterpret_cast<uint32_t *>(tile16 + ar * MX_PITCH + bc);
#pragma unroll
                    for (int k = 0; k < 4; ++k) dst[k] = wv[k];
                }
            }
            __syncthreads();
        }

        // all loads of the tile's four runs first (raw 16-bit pairs: 32 registers), then one run at a time
        uint32_t w[4][8];
#pragma unroll
        for (int it = 0; it < 4; ++it) {
            const int r = it * 32 + r0;                   // row of the tile
            if constexpr (STAGED) {
                const uint32_t *src = reinterpret_cast<const uint32_t *>(tile + r * MX_PITCH + piece * 16);
#pragma unroll
                for (int k = 0; k < 8; ++k) w[it][k] = src[k];
            } else {
                const int64_t i = i0 + r, j = j0 + piece * 16;
                if (p.vec32 && i0 + MX_TILE <= p.rows && j0 + MX_TILE <= p.cols) {       // whole tile inside x
                    ldg_nc_32(x + (i0 * p.ld + j0) + x_thr + it * x_it, w[it]);
                } else if (i < p.rows && j + 16 <= p.cols && p.vec32) {
                    ldg_nc_32(x + i * p.ld + j, w[it]);
                } else if (i < p.rows && j + 16 <= p.cols && p.vec16) {
                    const uint4 lo = ldg_nc_16(x + i * p.ld + j), hi = ldg_nc_16(x + i * p.ld + j + 8);
                    w[it][0] = lo.x; w[it][1] = lo.y; w[it][2] = lo.z; w[it][3] = lo.w;
                    w[it][4] = hi.x; w[it][5] = hi.y; w[it][6] = hi.z; w[it][7] = hi.w;
                } else {
                    const uint16_t *xs = reinterpret_cast<const uint16_t *>(x);
#pragma unroll
                    for (int k = 0; k < 8; ++k) {
                        const uint32_t a = (i < p.rows && j + 2 * k < p.cols) ? xs[i * p.ld + j + 2 * k] : 0u;
                        const uint32_t b = (i < p.rows && j + 2 * k + 1 < p.cols) ? xs[i * p.ld + j + 2 * k + 1] : 0u;
                        w[it][k] = a | (b << 16);
                    }
                }
            }
        }

        if constexpr (TWO_D) {
            // 32 x 32 blocks: sixteen per tile, each the maximum of 32 rows x 2 runs
#pragma unroll
            for (int it = 0; it < 4; ++it) {
                float v[16];
                piece_max[it * MX_THREADS + tid] = unpack16<T>(w[it], v);     // index = row * 8 + run
            }
            __syncthreads();
            if (tid < 16) {
                const int br = tid >> 2, bc = tid & 3;
                float m = 0.0f;
                for (int rr = 0; rr < 32; ++rr)
                    m = fmaxf(m, fmaxf(piece_max[(br * 32 + rr) * 8 + 2 * bc], piece_max[(br * 32 + rr) * 8 + 2 * bc + 1]));
                block_max[tid] = m;
            }
            __syncthreads();
        }

        uint8_t *codes_tile = p.codes + i0 * code_ld + (j0 >> 1);
        uint8_t *sf_tile = p.sf + (p.sf_tiled ? t * 512 : i0 * n_cb + (j0 >> 5));   // tile t of the tiled layout
#pragma unroll
        for (int it = 0; it < 4; ++it) {
            const int r = it * 32 + r0;
            float v[16];
            float bmax = unpack16<T>(w[it], v);
            // the neighbouring lane holds the other half of the 32-value block
            if constexpr (TWO_D) bmax = block_max[(r >> 5) * 4 + (piece >> 1)];
            else bmax = fmaxf(bmax, __shfl_xor_sync(0xffffffffu, bmax, 1));
            float inv;
            const uint32_t e = mx_scale(bmax, quarter, inv);
            const uint2 c = mx_encode16(v, inv);
            *reinterpret_cast<uint2 *>(codes_tile + code_thr + it * code_it) = c;
            if ((piece & 1) == 0) sf_tile[sf_thr + it * sf_it] = static_cast<uint8_t>(e);
        }
    }
}

// ---------------------------------------------------------------------------- dequantize

struct MxDequantParams {
    const uint8_t *codes;
    const uint8_t *sf;
    void *out;
    int64_t rows_p, cols_p, rows, cols, ld_out;
    int sf_tiled;
};

template <typename OUT> __device__ __forceinline__ OUT half_to_out(__half h);
template <> __device__ __forceinline__ __half half_to_out<__half>(__half h) { return h; }
template <> __device__ __forceinline__ __nv_bfloat16 half_to_out<__nv_bfloat16>(__half h) { return __float2bfloat16_rn(__half2float(h)); }
template <> __device__ __forceinline__ float half_to_out<float>(__half h) { return __half2float(h); }

// One thread per run of 16 values: 8 bytes of codes and the block's scale byte in, 16 values out.
template <typename OUT>
__global__ void __launch_bounds__(256)
dequantize_mx_kernel(const MxDequantParams p) {
    const int64_t runs_per_row = (p.cols + 15) / 16, total = p.rows * runs_per_row;
    const int64_t n_cb = p.cols_p / 32;
    OUT *out = static_cast<OUT *>(p.out);
    for (int64_t u = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; u < total;
         u += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        // (32-bit division whenever the run count allows it: the 64-bit form is a large part of this kernel)
        const int64_t i = total < (int64_t(1) << 31) ? static_cast<int64_t>(static_cast<uint32_t>(u) / static_cast<uint32_t>(runs_per_row))
                                                     : u / runs_per_row;
        const int64_t j = (u - i * runs_per_row) * 16;
        const uint2 c = *reinterpret_cast<const uint2 *>(p.codes + i * (p.cols_p / 2) + j / 2);
        const uint32_t e = p.sf[sf_offset(i, j >> 5, n_cb, p.sf_tiled != 0)];
        // E8M0 -> fp16 as a conversion of the binary32 value: inf above 2^15, 0 below 2^-25, NaN for 255
        const float sf32 = e == 255u ? __uint_as_float(0x7fc00000u) : (e == 0u ? 0.0f : __uint_as_float(e << 23));
        const __half2 s2 = __half2half2(__float2half_rn(sf32));
        OUT v[16];
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const uint32_t byte = ((k < 4 ? c.x : c.y) >> (8 * (k & 3))) & 0xffu;
            uint32_t h2;
            asm("{ .reg .b8 b; cvt.u8.u32 b, %1; cvt.rn.f16x2.e2m1x2 %0, b; }" : "=r"(h2) : "r"(byte));
            const __half2 r = __hmul2(*reinterpret_cast<__half2 *>(&h2), s2);
            v[2 * k] = half_to_out<OUT>(__low2half(r));
            v[2 * k + 1] = half_to_out<OUT>(__high2half(r));
        }
        OUT *dst = out + i * p.ld_out + j;
        const bool full = j + 16 <= p.cols;
        if (full && reinterpret_cast<uintptr_t>(dst) % 16 == 0) {
#pragma unroll
            for (int q = 0; q < static_cast<int>(sizeof(OUT)); ++q)
                reinterpret_cast<uint4 *>(dst)[q] = reinterpret_cast<const uint4 *>(v)[q];
        } else {
#pragma unroll
            for (int k = 0; k < 16; ++k)
                if (j + k < p.cols) dst[k] = v[k];
        }
    }
}

template <typename T>
cudaError_t launch_mx(const MxParams &p, bool two_d, bool transposed, cudaStream_t stream) {
    const int64_t tiles = (p.rows_p / MX_TILE) * (p.cols_p / MX_TILE);
    const int64_t cap = 148 * 4;
    const unsigned grid = static_cast<unsigned>(tiles < cap ? tiles : cap);
    if (two_d && transposed) quantize_mx_kernel<T, true, true><<<grid, MX_THREADS, 0, stream>>>(p);
    else if (two_d) quantize_mx_kernel<T, true, false><<<grid, MX_THREADS, 0, stream>>>(p);
    else if (transposed) quantize_mx_kernel<T, false, true><<<grid, MX_THREADS, 0, stream>>>(p);
    else quantize_mx_kernel<T, false, false><<<grid, MX_THREADS, 0, stream>>>(p);
    return cudaGetLastError();
}

}  // namespace

// MXFP4 branch of fos_quantize (arguments already validated there). amax_out receives 1.0, the
// per-tensor scale the reference reports for this format.
int quantize_mxfp4(const void *x, int x_dtype, int64_t rows, int64_t cols, int64_t ld, int scale_rule, int block_2d,
                   int transpose, int sf_layout, uint8_t *codes, uint8_t *sf, float *amax_out, cudaStream_t stream) {
    MxParams p{};
    p.x = x;
    p.rows = rows; p.cols = cols; p.ld = ld;
    p.out_rows = transpose ? cols : rows;
    p.out_cols = transpose ? rows : cols;
    p.rows_p = round_up64(p.out_rows, 128);
    p.cols_p = round_up64(p.out_cols, 128);
    p.codes = codes; p.sf = sf; p.amax_out = amax_out;
    p.inv_maxq_is_quarter = scale_rule == FOS_RULE_STATIC_4 ? 1.0f : 0.0f;
    p.sf_tiled = sf_layout == FOS_SF_TILED;
    p.vec16 = reinterpret_cast<uintptr_t>(x) % 16 == 0 && (ld * 2) % 16 == 0;
    p.vec32 = reinterpret_cast<uintptr_t>(x) % 32 == 0 && (ld * 2) % 32 == 0;
    FOS_CUDA_TRY(x_dtype == FOS_BF16 ? launch_mx<__nv_bfloat16>(p, block_2d != 0, transpose != 0, stream)
                                     : launch_mx<__half>(p, block_2d != 0, transpose != 0, stream));
    return FOS_OK;
}

// MXFP4 branch of fos_dequantize.
int dequantize_mxfp4(const uint8_t *codes, const uint8_t *sf, int sf_layout, int64_t rows_p, int64_t cols_p, int64_t rows,
                     int64_t cols, void *out, int out_dtype, int64_t ld_out, cudaStream_t stream) {
    MxDequantParams p{codes, sf, out, rows_p, cols_p, rows, cols, ld_out, sf_layout == FOS_SF_TILED};
    const int64_t total = rows * ((cols + 15) / 16);
    int64_t blocks = (total + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    const unsigned g = static_cast<unsigned>(blocks);
    if (out_dtype == FOS_BF16) dequantize_mx_kernel<__nv_bfloat16><<<g, 256, 0, stream>>>(p);
    else if (out_dtype == FOS_FP16) dequantize_mx_kernel<__half><<<g, 256, 0, stream>>>(p);
    else dequantize_mx_kernel<float><<<g, 256, 0, stream>>>(p);
    FOS_CUDA_TRY(cudaGetLastError());
    return FOS_OK;
}

}  // namespace fos
