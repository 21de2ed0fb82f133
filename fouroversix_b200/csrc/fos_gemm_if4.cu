// GEMM for IF4 operands (and any mix of IF4 / NVFP4): D[m, n] = alpha * sum_k A[m, k] * B[n, k].
//
// tcgen05 has no block-scaled type whose blocks are "E2M1, or INT4 times 6/7", so the product is
// computed the way the reference defines it (src/fouroversix/quantize/backend.py:88-160 feeding
// src/fouroversix/matmul/pytorch.py:33-52; the same decode as its Triton matmul,
// src/fouroversix/kernels/triton/matmul.py:170-222, and as the MAC model in
// if4_mac/scripts/gen_golden_ref.py:162-187): every element becomes the fp16 number
// fp16(value) * fp16(|scale|) (integer blocks: fp16(int * 6/7) first), and the fp16 numbers are
// multiplied with fp32 accumulation. Two kernels:
//
//   expand_kernel    packed codes + scales -> fp16 [rows_p, k_p] in a caller-provided workspace
//                    (one pass per operand, HBM-bound, 0.5625 B read + 2 B written per element)
//   gemm_f16_kernel  tcgen05.mma kind::f16 (M 128, N 256, K 16) over the two fp16 matrices: the
//                    pipeline of the NVFP4 kernel without scale factors, which leaves room in
//                    tensor memory for two accumulators, so the epilogue of one tile overlaps the
//                    main loop of the next
//
// Expanding once per operand instead of inside the GEMM's producer costs 2 * 2 B per element of
// extra HBM traffic but decodes every element once rather than once per tile that uses it.
#include <mutex>

#include "fos_tcgen05.cuh"

namespace fos {
namespace {

// ---------------------------------------------------------------------------- expand

struct ExpandParams {
    const uint8_t *codes;
    const uint8_t *sf;
    __half *out;
    int64_t rows_p, cols_p;
    int format, sf_tiled;
};

__device__ __forceinline__ float as_fp16_value(float v) { return __half2float(__float2half_rn(v)); }

// The sixteen fp16 outputs of one block (o[i] = values 2i, 2i + 1) from a table of its eight magnitudes.
// E2M1 blocks: value * scale is exact in fp16 (at most 6 significant bits, never subnormal: the smallest
// product is 0.5 * 2^-9), so the magnitudes are s / 2, s, 1.5 s, 2 s, 3 s, 4 s, 6 s: two conversions and
// exponent-field additions. Integer blocks: fp16(fp16(i * 6/7) * s) for i = 1 .. 7, four packed fp16
// multiplications by the constants fp16(i * fl32(6/7)); the magnitude of a two's-complement nibble is
// (n ^ m) + sign with m = 15 where the sign bit is set, all eight nibbles of a word at once (-8 does not occur:
// the quantizer clamps to +-7). A byte permute looks the magnitudes up by code, another one supplies the sign
// bit. Returns false for a scale byte it does not take (NaN; a set sign bit on an NVFP4 scale).
__device__ __forceinline__ bool expand_block_packed(uint2 c, uint32_t sfb, bool if4, uint32_t (&o)[8]) {
    const bool is_int = if4 && (sfb & 0x80u);
    if (if4) sfb &= 0x7fu;
    if (sfb >= 0x7fu) return false;
    const float s = e4m3_to_float(sfb);
    uint32_t t01, t23, t45, t67, mag[2], sgn[2];
    sgn[0] = (c.x >> 3) & 0x11111111u;
    sgn[1] = (c.y >> 3) & 0x11111111u;
    if (!is_int) {
        t23 = pack_pair<__half>(s, __fmul_rn(s, 1.5f));
        t01 = (t23 << 16) - 0x04000000u;
        t45 = t23 + 0x04000400u;
        t67 = t45 + 0x04000400u;
        if ((t23 & 0xffffu) == 0u) t01 = t23 = t45 = t67 = 0u;
        mag[0] = c.x & 0x77777777u;
        mag[1] = c.y & 0x77777777u;
    } else {
        const __half2 s2 = __float2half2_rn(s);
        auto times = [&](uint32_t consts) {
            const __half2 r = __hmul2(*reinterpret_cast<const __half2 *>(&consts), s2);
            return *reinterpret_cast<const uint32_t *>(&r);
        };
        t01 = times(0x3adb0000u);            // fp16(i * fl32(6/7)) for i = 0, 1
        t23 = times(0x41253edbu);            // 2, 3
        t45 = times(0x444942dbu);            // 4, 5
        t67 = times(0x46004525u);            // 6, 7
        mag[0] = ((c.x ^ (sgn[0] * 15u)) + sgn[0]) & 0x77777777u;
        mag[1] = ((c.y ^ (sgn[1] * 15u)) + sgn[1]) & 0x77777777u;
    }
    const uint32_t la = __byte_perm(t01, t23, 0x6420), ha = __byte_perm(t01, t23, 0x7531);
    const uint32_t lb = __byte_perm(t45, t67, 0x6420), hb = __byte_perm(t45, t67, 0x7531);
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

// One thread per 16-value block: 8 bytes of codes + 1 scale byte -> 32 bytes of fp16. Four blocks per thread and
// round, their loads issued before the first is decoded.
constexpr int EXPAND_DEPTH = 4;
__global__ void __launch_bounds__(256) expand_kernel(const ExpandParams p) {
    const int64_t n_cb = p.cols_p >> 4;
    const int64_t total = p.rows_p * n_cb;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    const bool small = total < (int64_t(1) << 31);
    for (int64_t i0 = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i0 < total; i0 += stride * EXPAND_DEPTH) {
        uint2 c[EXPAND_DEPTH];
        uint32_t sfbs[EXPAND_DEPTH];
        int64_t offs[EXPAND_DEPTH];
#pragma unroll
        for (int d = 0; d < EXPAND_DEPTH; ++d) {
            const int64_t i = i0 + d * stride;
            offs[d] = -1;
            c[d] = make_uint2(0u, 0u);
            sfbs[d] = 0u;
            if (i < total) {
                // (a 64-bit division costs about as much as decoding the block)
                const int64_t r = small ? static_cast<int64_t>(static_cast<uint32_t>(i) / static_cast<uint32_t>(n_cb)) : i / n_cb;
                const int64_t cb = i - r * n_cb;
                c[d] = *reinterpret_cast<const uint2 *>(p.codes + r * (p.cols_p >> 1) + cb * 8);
                sfbs[d] = p.sf[sf_offset(r, cb, n_cb, p.sf_tiled != 0)];
                offs[d] = r * p.cols_p + cb * 16;
            }
        }
#pragma unroll
        for (int d = 0; d < EXPAND_DEPTH; ++d) {
            if (offs[d] < 0) continue;
            uint4 *dst = reinterpret_cast<uint4 *>(p.out + offs[d]);
            uint32_t o[8];
            if (expand_block_packed(c[d], sfbs[d], p.format == FOS_IF4, o)) {
                stg_32(dst, o);
                continue;
            }
            uint32_t sfb = sfbs[d];
            const bool is_int = p.format == FOS_IF4 && (sfb & 0x80u);
            if (p.format == FOS_IF4) sfb &= 0x7fu;
            const float s16 = e4m3_to_float(sfb);
            __align__(16) __half h[16];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const uint32_t byte = ((j < 4 ? c[d].x : c[d].y) >> ((j & 3) * 8)) & 0xffu;
                float2 q;
                if (is_int) {
                    const float six_sevenths = static_cast<float>(6.0 / 7.0);
                    q.x = as_fp16_value(__fmul_rn(static_cast<float>(static_cast<int>(byte << 28) >> 28), six_sevenths));
                    q.y = as_fp16_value(__fmul_rn(static_cast<float>(static_cast<int>(byte << 24) >> 28), six_sevenths));
                } else {
                    q = e2m1x2_to_float2(byte);
                }
                h[2 * j] = __float2half_rn(__fmul_rn(q.x, s16));
                h[2 * j + 1] = __float2half_rn(__fmul_rn(q.y, s16));
            }
            dst[0] = reinterpret_cast<const uint4 *>(h)[0];
            dst[1] = reinterpret_cast<const uint4 *>(h)[1];
        }
    }
}

// ---------------------------------------------------------------------------- fp16 GEMM

constexpr int BLOCK_M = 128, BLOCK_N = 256;
constexpr int BLOCK_K_BYTES = 128;                  // 64 fp16 values: one 128-byte swizzle row
constexpr int MMAS_PER_STAGE = 4;                   // K = 16 values = 32 bytes each
constexpr int A_BYTES = BLOCK_M * BLOCK_K_BYTES, B_BYTES = BLOCK_N * BLOCK_K_BYTES;
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;      // 48 KiB
constexpr int STAGES = 4, ACC_STAGES = 2;
constexpr int EPI_WARPS = 8;
constexpr int THREADS = 64 + 32 * EPI_WARPS;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256;

struct F16GemmParams {
    const float *alpha;
    void *d;
    int32_t *status;
    int64_t m_p, n_p, k_p, m, n, ldd;
};

// kind::f16 instruction descriptor: fp32 accumulate (1 in bits [4,6)), A and B fp16 (0 in [7,10) and
// [10,13)), both K-major, N >> 3 in [17,23), M >> 4 in [24,29).
__device__ __forceinline__ uint32_t f16_idesc(int n) {
    return (1u << 4) | (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(BLOCK_M >> 4) << 24);
}
__device__ __forceinline__ void tc_mma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                           uint32_t accumulate) {
    asm volatile(
        "{ .reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p; }\n"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}

template <typename OUT>
__global__ void __launch_bounds__(THREADS, 1)
gemm_f16_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                const F16GemmParams p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem_gen + STAGES * STAGE_BYTES);
    const uint32_t full_bar = smem_u32(bars);
    const uint32_t empty_bar = full_bar + 8 * STAGES;
    const uint32_t acc_full_bar = empty_bar + 8 * STAGES;          // [ACC_STAGES]
    const uint32_t acc_empty_bar = acc_full_bar + 8 * ACC_STAGES;  // [ACC_STAGES]
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 2 * STAGES + 2 * ACC_STAGES);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(full_bar + 8 * s, 1);
            mbar_init(empty_bar + 8 * s, 1);
        }
        for (int a = 0; a < ACC_STAGES; ++a) {
            mbar_init(acc_full_bar + 8 * a, 1);
            mbar_init(acc_empty_bar + 8 * a, EPI_WARPS);
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    const int64_t num_m = p.m_p / BLOCK_M, num_n = (p.n_p + BLOCK_N - 1) / BLOCK_N;
    const int64_t num_tiles = num_m * num_n;
    const int64_t k_tiles = p.k_p / 64;

    // The producer and the MMA issuer run as whole warps with one elected lane issuing: with every value of the
    // loop the same in all lanes the compiler keeps addresses and descriptors in uniform registers, which the
    // TMA and tcgen05 instructions take directly; a lone thread pays for moving every operand over.
    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        const bool issue = elect_one();
        uint32_t it = 0;
        bool ok = true;
        for (int64_t t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
            int64_t mb, nb;
            tile_coords(t, num_m, num_n, mb, nb);
            for (int64_t kt = 0; kt < k_tiles; ++kt, ++it) {
                const uint32_t s = it % STAGES, ph = (it / STAGES) & 1u;
                ok = __all_sync(0xffffffffu, mbar_wait(empty_bar + 8 * s, ph ^ 1u, abort_flag, p.status, 1));
                if (!ok) break;
                const uint32_t stage = smem_base + s * STAGE_BYTES, bar = full_bar + 8 * s;
                if (issue) {
                    mbar_expect_tx(bar, STAGE_BYTES);   // rows past n_p are zero-filled and still counted
                    tma_load_2d(stage, &map_a, static_cast<int>(kt * BLOCK_K_BYTES), static_cast<int>(mb * BLOCK_M), bar);
                    tma_load_2d(stage + A_BYTES, &map_b, static_cast<int>(kt * BLOCK_K_BYTES),
                                static_cast<int>(nb * BLOCK_N), bar);
                }
                __syncwarp();
            }
        }
        if (!ok) {
            const unsigned long long t0 = global_timer_ns();
            while (global_timer_ns() - t0 < 200000ull) __nanosleep(1000);
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        const bool issue = elect_one();
        uint32_t it = 0, tile_i = 0;
        bool ok = true;
        for (int64_t t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++tile_i) {
            int64_t mb, nb;
            tile_coords(t, num_m, num_n, mb, nb);
            const int64_t n0 = nb * BLOCK_N;
            const uint32_t idesc = f16_idesc(static_cast<int>((p.n_p - n0) < BLOCK_N ? (p.n_p - n0) : BLOCK_N));
            const uint32_t acc = tile_i % ACC_STAGES, acc_ph = (tile_i / ACC_STAGES) & 1u;
            ok = __all_sync(0xffffffffu, mbar_wait(acc_empty_bar + 8 * acc, acc_ph ^ 1u, abort_flag, p.status, 3));
            if (!ok) break;
            tc_fence_after();
            const uint32_t d_tmem = tmem_base + acc * BLOCK_N;
            for (int64_t kt = 0; kt < k_tiles; ++kt, ++it) {
                const uint32_t s = it % STAGES, ph = (it / STAGES) & 1u;
                ok = __all_sync(0xffffffffu, mbar_wait(full_bar + 8 * s, ph, abort_flag, p.status, 2));
                if (!ok) break;
                tc_fence_after();
                const uint32_t stage = smem_base + s * STAGE_BYTES;
                const uint64_t a_desc = smem_desc(stage, 16, 1024, 2), b_desc = smem_desc(stage + A_BYTES, 16, 1024, 2);
                if (issue) {
#pragma unroll
                    for (int j = 0; j < MMAS_PER_STAGE; ++j)
                        tc_mma_f16(d_tmem, a_desc + 2 * j, b_desc + 2 * j, idesc, (kt > 0 || j > 0) ? 1u : 0u);
                    tc_commit(empty_bar + 8 * s);
                }
                __syncwarp();
            }
            if (ok && issue) tc_commit(acc_full_bar + 8 * acc);
        }
    } else if (warp >= 2) {
        // ------------------------------------------------------------------ epilogue
        const int quad = warp & 3, half = (warp - 2) >> 2;
        constexpr int COLS = BLOCK_N / 2;
        const float alpha = __ldg(p.alpha);
        OUT *out = static_cast<OUT *>(p.d);
        const bool vec_ok = (reinterpret_cast<uintptr_t>(out) % 16 == 0) && ((p.ldd * sizeof(OUT)) % 16 == 0);
        uint32_t tile_i = 0;
        bool ok = true;
        for (int64_t t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++tile_i) {
            int64_t mb, nb;
            tile_coords(t, num_m, num_n, mb, nb);
            const int64_t row = mb * BLOCK_M + quad * 32 + lane, n0 = nb * BLOCK_N + half * COLS;
            const uint32_t acc = tile_i % ACC_STAGES, acc_ph = (tile_i / ACC_STAGES) & 1u;
            ok = mbar_wait(acc_full_bar + 8 * acc, acc_ph, abort_flag, p.status, 4);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
            const uint32_t t_acc = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + acc * BLOCK_N + half * COLS;
#pragma unroll 1
            for (int c = 0; c < COLS / 32; c += 2) {
                uint32_t v0[32], v1[32];
                tc_load_64cols_sync(t_acc + 32 * c, v0, v1);
                if (c + 2 >= COLS / 32) {
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(acc_empty_bar + 8 * acc);
                }
                const int64_t col = n0 + 32 * c;
                const int64_t left0 = p.n - col, left1 = left0 - 32;
                if (row < p.m && left0 > 0)
                    store_chunk<OUT>(out + row * p.ldd + col, v0, alpha, left0 < 32 ? static_cast<int>(left0) : 32, vec_ok);
                if (row < p.m && left1 > 0)
                    store_chunk<OUT>(out + row * p.ldd + col + 32, v1, alpha, left1 < 32 ? static_cast<int>(left1) : 32, vec_ok);
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

template <typename OUT>
int launch_f16(const CUtensorMap &ma, const CUtensorMap &mb, const F16GemmParams &p, cudaStream_t stream) {
    auto kernel = gemm_f16_kernel<OUT>;
    static OncePerDevice configured;   // per instantiation
    int dev = 0, sms = 0;
    FOS_CUDA_TRY(cudaGetDevice(&dev));
    FOS_CUDA_TRY(configured.run(dev, [&] {
        return cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    }));
    FOS_CUDA_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    const int64_t tiles = (p.m_p / BLOCK_M) * ((p.n_p + BLOCK_N - 1) / BLOCK_N);
    const unsigned grid = static_cast<unsigned>(tiles < sms ? tiles : sms);
    kernel<<<grid, THREADS, SMEM_BYTES, stream>>>(ma, mb, p);
    FOS_CUDA_TRY(cudaGetLastError());
    return FOS_OK;
}

int launch_expand(const uint8_t *codes, const uint8_t *sf, int format, int sf_layout, int64_t rows_p, int64_t cols_p,
                  __half *out, cudaStream_t stream) {
    ExpandParams p{codes, sf, out, rows_p, cols_p, format, sf_layout == FOS_SF_TILED};
    const int64_t total = rows_p * (cols_p / 16);
    int64_t blocks = (total + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    expand_kernel<<<static_cast<unsigned>(blocks), 256, 0, stream>>>(p);
    FOS_CUDA_TRY(cudaGetLastError());
    return FOS_OK;
}

}  // namespace
}  // namespace fos

cudaError_t fos::gemm_if4_wait_failures(int32_t *host_value) { return fos::read_wait_failures(host_value); }
cudaError_t fos::gemm_if4_wait_roles(uint32_t *host_value) { return fos::read_wait_roles(host_value); }

extern "C" int64_t fos_gemm_if4_workspace_bytes(int64_t m_p, int64_t n_p, int64_t k_p) {
    if (m_p <= 0 || n_p <= 0 || k_p <= 0) return 0;
    return (m_p + n_p) * k_p * 2;
}

namespace fos {
namespace {

// Scratch for fos_gemm_if4_static: lives in the library image, one copy per GPU that loads it.
constexpr int64_t STATIC_WORKSPACE_BYTES = int64_t(FOS_GEMM_IF4_STATIC_WORKSPACE_BYTES);
static __device__ __align__(256) unsigned char g_static_workspace[STATIC_WORKSPACE_BYTES];

// Validates the arguments shared by both entry points, expands both operands into `workspace`
// and runs the fp16 GEMM. Allocates nothing.
int gemm_if4_impl(const uint8_t *a_codes, const uint8_t *a_sf, int a_format, int a_sf_layout, const uint8_t *b_codes,
                  const uint8_t *b_sf, int b_format, int b_sf_layout, const float *alpha, void *d, int out_dtype,
                  int64_t m_p, int64_t n_p, int64_t k_p, int64_t m, int64_t n, int64_t ldd, void *workspace,
                  int32_t *status, cudaStream_t stream) {
    __half *a16 = static_cast<__half *>(workspace);
    __half *b16 = a16 + m_p * k_p;
    int st;
    if ((st = launch_expand(a_codes, a_sf, a_format, a_sf_layout, m_p, k_p, a16, stream)) != FOS_OK) return st;
    if ((st = launch_expand(b_codes, b_sf, b_format, b_sf_layout, n_p, k_p, b16, stream)) != FOS_OK) return st;
    CUtensorMap map_a, map_b;
    if ((st = make_operand_map(&map_a, a16, m_p, k_p * 2, BLOCK_M)) != FOS_OK) return st;
    if ((st = make_operand_map(&map_b, b16, n_p, k_p * 2, BLOCK_N)) != FOS_OK) return st;
    if (status) {
        FOS_CUDA_TRY(cudaMemsetAsync(status, 0, sizeof(int32_t), stream));
    } else {
        FOS_CUDA_TRY(wait_failures_ptr(&status));   // the library's sticky word
    }
    F16GemmParams p{alpha, d, status, m_p, n_p, k_p, m, n, ldd};
    if (out_dtype == FOS_BF16) return launch_f16<__nv_bfloat16>(map_a, map_b, p, stream);
    if (out_dtype == FOS_FP16) return launch_f16<__half>(map_a, map_b, p, stream);
    return launch_f16<float>(map_a, map_b, p, stream);
}

int check_gemm_if4_args(const uint8_t *a_codes, const uint8_t *a_sf, int a_format, int a_sf_layout,
                        const uint8_t *b_codes, const uint8_t *b_sf, int b_format, int b_sf_layout, const float *alpha,
                        void *d, int out_dtype, int64_t m_p, int64_t n_p, int64_t k_p, int64_t m, int64_t n,
                        int64_t ldd) {
    if (!a_codes || !a_sf || !b_codes || !b_sf || !alpha || !d) return FOS_ERR_INVALID_ARGUMENT;
    if (m_p <= 0 || n_p <= 0 || k_p < 64 || m_p % 128 || n_p % 128 || k_p % 64) return FOS_ERR_INVALID_ARGUMENT;
    if (m <= 0 || n <= 0 || m > m_p || n > n_p || ldd < n) return FOS_ERR_INVALID_ARGUMENT;
    if (out_dtype != FOS_BF16 && out_dtype != FOS_FP16 && out_dtype != FOS_FP32) return FOS_ERR_INVALID_ARGUMENT;
    for (int f : {a_format, b_format})
        if (f != FOS_NVFP4 && f != FOS_IF4) return FOS_ERR_INVALID_ARGUMENT;
    for (int l : {a_sf_layout, b_sf_layout})
        if (l != FOS_SF_ROWMAJOR && l != FOS_SF_TILED) return FOS_ERR_INVALID_ARGUMENT;
    if (reinterpret_cast<uintptr_t>(a_codes) % 8 || reinterpret_cast<uintptr_t>(b_codes) % 8) return FOS_ERR_MISALIGNED;
    if (m_p > INT32_MAX || n_p > INT32_MAX || k_p * 2 > INT32_MAX) return FOS_ERR_TOO_LARGE;
    return FOS_OK;
}

}  // namespace
}  // namespace fos

extern "C" int fos_gemm_if4(const uint8_t *a_codes, const uint8_t *a_sf, int a_format, int a_sf_layout,
                            const uint8_t *b_codes, const uint8_t *b_sf, int b_format, int b_sf_layout,
                            const float *alpha, void *d, int out_dtype, int64_t m_p, int64_t n_p, int64_t k_p,
                            int64_t m, int64_t n, int64_t ldd, void *workspace, int64_t workspace_bytes,
                            int32_t *status, void *stream_) {
    using namespace fos;
    int st = check_gemm_if4_args(a_codes, a_sf, a_format, a_sf_layout, b_codes, b_sf, b_format, b_sf_layout, alpha, d,
                                 out_dtype, m_p, n_p, k_p, m, n, ldd);
    if (st != FOS_OK) return st;
    if (!workspace || workspace_bytes < fos_gemm_if4_workspace_bytes(m_p, n_p, k_p)) return FOS_ERR_INVALID_ARGUMENT;
    if (reinterpret_cast<uintptr_t>(workspace) % 128) return FOS_ERR_MISALIGNED;
    if ((st = check_device()) != FOS_OK) return st;
    return gemm_if4_impl(a_codes, a_sf, a_format, a_sf_layout, b_codes, b_sf, b_format, b_sf_layout, alpha, d, out_dtype,
                         m_p, n_p, k_p, m, n, ldd, workspace, status, static_cast<cudaStream_t>(stream_));
}

// fos_gemm_if4 for callers that cannot hand over scratch memory: the expanded operands go into
// g_static_workspace. The array's name is a host-side handle, not a device address, so the
// address is asked for once per device (with that device current) and cached; that first call
// is the only set-up and should happen outside any stream capture.
extern "C" int fos_gemm_if4_static(const uint8_t *a_codes, const uint8_t *a_sf, int a_format, int a_sf_layout,
                                   const uint8_t *b_codes, const uint8_t *b_sf, int b_format, int b_sf_layout,
                                   const float *alpha, void *d, int out_dtype, int64_t m_p, int64_t n_p, int64_t k_p,
                                   int64_t m, int64_t n, int64_t ldd, int32_t *status, void *stream_) {
    using namespace fos;
    int st = check_gemm_if4_args(a_codes, a_sf, a_format, a_sf_layout, b_codes, b_sf, b_format, b_sf_layout, alpha, d,
                                 out_dtype, m_p, n_p, k_p, m, n, ldd);
    if (st != FOS_OK) return st;
    if (fos_gemm_if4_workspace_bytes(m_p, n_p, k_p) > STATIC_WORKSPACE_BYTES) return FOS_ERR_TOO_LARGE;
    if ((st = check_device()) != FOS_OK) return st;

    static void *device_address[64] = {};
    static std::mutex setup_lock;
    int dev = 0;
    FOS_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return FOS_ERR_UNSUPPORTED;
    void *workspace = nullptr;
    {
        std::lock_guard<std::mutex> guard(setup_lock);
        if (device_address[dev] == nullptr) {
            void *ptr = nullptr;
            FOS_CUDA_TRY(cudaGetSymbolAddress(&ptr, g_static_workspace));
            device_address[dev] = ptr;
        }
        workspace = device_address[dev];
    }
    return gemm_if4_impl(a_codes, a_sf, a_format, a_sf_layout, b_codes, b_sf, b_format, b_sf_layout, alpha, d, out_dtype,
                         m_p, n_p, k_p, m, n, ldd, workspace, status, static_cast<cudaStream_t>(stream_));
}
