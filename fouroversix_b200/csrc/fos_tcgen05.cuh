// tcgen05 / TMA / mbarrier building blocks shared by the GEMM kernels (sm_100a).
#pragma once

#include <cuda.h>

#include <mutex>
#include <type_traits>

#include "fos_common.cuh"

namespace fos {
namespace {

constexpr unsigned long long WAIT_LIMIT_NS = 2000000000ull;   // waits timed with the global timer give up after 2 s
constexpr long long WAIT_LIMIT_CYCLES = 4000000000ll;         // waits timed in SM cycles: about 2 s at 2 GHz, 4 s at 1 GHz
constexpr int TMEM_COLS = 512;

// Site of the first bounded device-side wait that ever gave up in a kernel of this translation unit on
// this device, 0 if none did (never expected to change). Sticky: nothing resets it, so a launch whose
// caller passed no status word of its own still leaves a trace that fos_wait_failure_site reports.
__device__ int32_t g_wait_failures = 0;
// Bit `site` is set for every wait that was in progress when its CTA gave up (the wait that timed out and
// the waits that then saw the CTA's abort flag): which roles of a kernel were blocked, and where.
__device__ uint32_t g_wait_roles = 0;

// Runs `init` once per device (the first call with that device current), under a lock: for
// cudaFuncSetAttribute and the like, whose results the launch paths cache per device.
struct OncePerDevice {
    std::mutex mu;
    bool done[64] = {};
    template <typename F> cudaError_t run(int dev, F init) {
        if (dev < 0 || dev >= 64) return init();
        std::lock_guard<std::mutex> lock(mu);
        if (done[dev]) return cudaSuccess;
        const cudaError_t e = init();
        if (e == cudaSuccess) done[dev] = true;
        return e;
    }
};

// Device address of this translation unit's g_wait_failures on the current device.
inline cudaError_t wait_failures_ptr(int32_t **out) {
    static std::mutex mu;
    static int32_t *ptrs[64] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    const int slot = (dev >= 0 && dev < 64) ? dev : 0;
    std::lock_guard<std::mutex> lock(mu);
    if (ptrs[slot] == nullptr || dev != slot) {
        void *ptr = nullptr;
        e = cudaGetSymbolAddress(&ptr, g_wait_failures);
        if (e != cudaSuccess) return e;
        if (dev != slot) { *out = static_cast<int32_t *>(ptr); return cudaSuccess; }
        ptrs[slot] = static_cast<int32_t *>(ptr);
    }
    *out = ptrs[slot];
    return cudaSuccess;
}

inline cudaError_t read_wait_failures(int32_t *host_value) {
    return cudaMemcpyFromSymbol(host_value, g_wait_failures, sizeof(int32_t));
}
inline cudaError_t read_wait_roles(uint32_t *host_value) {
    return cudaMemcpyFromSymbol(host_value, g_wait_roles, sizeof(uint32_t));
}

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ unsigned long long global_timer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{ .reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p; }\n"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}

// Bounded wait. Returns false when the CTA is aborting (this wait or another one timed out).
// The limit is counted in SM clock cycles: reading %globaltimer inside the polling loop would add
// its own latency to every hand-over between the roles of a kernel.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag,
                                          int32_t *status, int where) {
#pragma unroll 1
    for (int i = 0; i < 64; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
#pragma unroll 1
    while (true) {
#pragma unroll 1
        for (int i = 0; i < 32; ++i)
            if (mbar_try_wait(bar, parity)) return true;
        if (*abort_flag) {
            atomicOr(&g_wait_roles, 1u << (where & 31));
            return false;
        }
        if (clock64() - t0 > WAIT_LIMIT_CYCLES) {
            *abort_flag = 1;
            if (status) atomicCAS(status, 0, where);
            atomicOr(&g_wait_roles, 1u << (where & 31));
            return false;
        }
    }
}

// Non-suspending probe of a barrier phase.
__device__ __forceinline__ bool mbar_test_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{ .reg .pred p;\n"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p; }\n"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}

// try_wait whose suspension is limited to about `ns` nanoseconds.
__device__ __forceinline__ bool mbar_try_wait_hint(uint32_t bar, uint32_t parity, uint32_t ns) {
    uint32_t ok;
    asm volatile(
        "{ .reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n"
        "selp.u32 %0, 1, 0, p; }\n"
        : "=r"(ok) : "r"(bar), "r"(parity), "r"(ns) : "memory");
    return ok != 0;
}

constexpr uint32_t POLL_SUSPEND_NS = 100;   // longest suspension of one probe in mbar_wait_poll

// mbar_wait for barriers that another CTA of the cluster arrives on. A thread suspended in a plain
// try_wait was not woken promptly by such an arrival (over a microsecond per hand-over), and probing
// with test_wait in a tight loop from a dozen threads takes shared-memory cycles from the copies and
// the MMAs (the CTA-pair GEMM ran a tenth faster without it): each probe here is a try_wait whose
// suspension is limited to POLL_SUSPEND_NS.
__device__ __forceinline__ bool mbar_wait_poll(uint32_t bar, uint32_t parity, volatile int *abort_flag,
                                               int32_t *status, int where) {
    const long long t0 = clock64();
#pragma unroll 1
    while (true) {
#pragma unroll 1
        for (int i = 0; i < 256; ++i)
            if (mbar_try_wait_hint(bar, parity, POLL_SUSPEND_NS)) return true;
        if (*abort_flag) {
            atomicOr(&g_wait_roles, 1u << (where & 31));
            return false;
        }
        if (clock64() - t0 > WAIT_LIMIT_CYCLES) {
            *abort_flag = 1;
            if (status) atomicCAS(status, 0, where);
            atomicOr(&g_wait_roles, 1u << (where & 31));
            return false;
        }
    }
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, int c0, int c1, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(bar) : "memory");
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap *map, int c0, int c1, int c2, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
        ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(bar) : "memory");
}
__device__ __forceinline__ void bulk_load(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}

// True in exactly one lane of a converged warp.
__device__ __forceinline__ bool elect_one() {
    uint32_t is_elected;
    asm volatile("{ .reg .pred p;\n"
                 "elect.sync _|p, 0xffffffff;\n"
                 "selp.u32 %0, 1, 0, p; }" : "=r"(is_elected));
    return is_elected != 0;
}

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// Two 32-column loads and the wait in ONE asm statement, so that no use of the destination
// registers can be scheduled between the loads and the wait.
__device__ __forceinline__ void tc_load_64cols_sync(uint32_t taddr, uint32_t (&a)[32], uint32_t (&b)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%64];\n"
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%32,%33,%34,%35,%36,%37,%38,%39,%40,%41,%42,%43,%44,%45,%46,%47,%48,%49,%50,%51,%52,%53,%54,%55,%56,%57,%58,%59,%60,%61,%62,%63}, [%65];\n"
        "tcgen05.wait::ld.sync.aligned;"
        : "=r"(a[0]), "=r"(a[1]), "=r"(a[2]), "=r"(a[3]), "=r"(a[4]), "=r"(a[5]), "=r"(a[6]), "=r"(a[7]), "=r"(a[8]), "=r"(a[9]), "=r"(a[10]), "=r"(a[11]), "=r"(a[12]), "=r"(a[13]), "=r"(a[14]), "=r"(a[15]), "=r"(a[16]), "=r"(a[17]), "=r"(a[18]), "=r"(a[19]), "=r"(a[20]), "=r"(a[21]), "=r"(a[22]), "=r"(a[23]), "=r"(a[24]), "=r"(a[25]), "=r"(a[26]), "=r"(a[27]), "=r"(a[28]), "=r"(a[29]), "=r"(a[30]), "=r"(a[31]), "=r"(b[0]), "=r"(b[1]), "=r"(b[2]), "=r"(b[3]), "=r"(b[4]), "=r"(b[5]), "=r"(b[6]), "=r"(b[7]), "=r"(b[8]), "=r"(b[9]), "=r"(b[10]), "=r"(b[11]), "=r"(b[12]), "=r"(b[13]), "=r"(b[14]), "=r"(b[15]), "=r"(b[16]), "=r"(b[17]), "=r"(b[18]), "=r"(b[19]), "=r"(b[20]), "=r"(b[21]), "=r"(b[22]), "=r"(b[23]), "=r"(b[24]), "=r"(b[25]), "=r"(b[26]), "=r"(b[27]), "=r"(b[28]), "=r"(b[29]), "=r"(b[30]), "=r"(b[31])
        : "r"(taddr), "r"(taddr + 32) : "memory");
}

// One 32-column load and the wait, again in one asm statement.
__device__ __forceinline__ void tc_load_32cols_sync(uint32_t taddr, uint32_t (&a)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];\n"
        "tcgen05.wait::ld.sync.aligned;"
        : "=r"(a[0]), "=r"(a[1]), "=r"(a[2]), "=r"(a[3]), "=r"(a[4]), "=r"(a[5]), "=r"(a[6]), "=r"(a[7]), "=r"(a[8]), "=r"(a[9]), "=r"(a[10]), "=r"(a[11]), "=r"(a[12]), "=r"(a[13]), "=r"(a[14]), "=r"(a[15]), "=r"(a[16]), "=r"(a[17]), "=r"(a[18]), "=r"(a[19]), "=r"(a[20]), "=r"(a[21]), "=r"(a[22]), "=r"(a[23]), "=r"(a[24]), "=r"(a[25]), "=r"(a[26]), "=r"(a[27]), "=r"(a[28]), "=r"(a[29]), "=r"(a[30]), "=r"(a[31])
        : "r"(taddr) : "memory");
}

// Each lane writes N consecutive 32-bit columns of its own tensor-memory lane.
__device__ __forceinline__ void tc_store_16cols(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]) : "memory");
}
__device__ __forceinline__ void tc_store_8cols(uint32_t taddr, const uint32_t (&r)[8]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]) : "memory");
}
template <int N> __device__ __forceinline__ void tc_store_cols(uint32_t taddr, const uint32_t (&r)[N]) {
    static_assert(N == 8 || N % 16 == 0, "8 columns or a multiple of 16");
    if constexpr (N == 8) {
        tc_store_8cols(taddr, r);
    } else {
#pragma unroll
        for (int c = 0; c < N; c += 16) tc_store_16cols(taddr + c, *reinterpret_cast<const uint32_t (*)[16]>(&r[c]));
    }
}
__device__ __forceinline__ void tc_wait_store() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
// 16-byte read-only load that may stay in L1 (for small data several warps of an SM re-read).
__device__ __forceinline__ uint4 ldg_16_cached(const void *p) {
    uint4 v;
    asm volatile("ld.global.nc.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ void prefetch_l1(const void *p) { asm volatile("prefetch.global.L1 [%0];" ::"l"(p)); }
__device__ __forceinline__ uint4 lds_16(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}

// ---- wrappers used by the CTA-pair (cta_group::2) kernel ----

__device__ __forceinline__ uint32_t cluster_cta_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// Address of `addr` (a shared::cta address of this CTA) in CTA `rank` of the cluster.
__device__ __forceinline__ uint32_t map_to_cta(uint32_t addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_bar) {
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar) : "memory");
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n"
                 "barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Arrive on the barrier at the same shared-memory offset in both CTAs of the pair once all
// tcgen05 operations issued so far by this thread have completed.
__device__ __forceinline__ void tc_commit_pair(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(bar), "h"(static_cast<uint16_t>(3)) : "memory");
}

// Shared-memory matrix descriptor. Bits: [0,14) start address >> 4, [16,30) leading byte
// offset >> 4, [32,46) stride byte offset >> 4, [46,48) version = 1 on sm_100, [61,64)
// swizzle mode (0 none, 2 128-byte).
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes, uint32_t swizzle) {
    return static_cast<uint64_t>((addr & 0x3ffffu) >> 4) | (static_cast<uint64_t>(lbo_bytes >> 4) << 16) |
           (static_cast<uint64_t>(sbo_bytes >> 4) << 32) | (1ull << 46) | (static_cast<uint64_t>(swizzle) << 61);
}


// Tile order: bands of GROUP_M row blocks, column blocks inside a band, so that the CTAs
// running at the same time share a few A and B panels in L2.
constexpr int GROUP_M = 8;
__device__ __forceinline__ void tile_coords(int64_t t, int64_t num_m, int64_t num_n, int64_t &mb, int64_t &nb) {
    const int64_t band = GROUP_M * num_n;
    const int64_t g = t / band, r = t - g * band;
    const int64_t first = g * GROUP_M;
    const int64_t rows = (num_m - first) < GROUP_M ? (num_m - first) : GROUP_M;
    mb = first + r % rows;
    nb = r / rows;
}

// Two floats -> one word of two 16-bit outputs (`lo` in the lower half).
template <typename OUT>
__device__ __forceinline__ uint32_t pack_pair(float lo, float hi) {
    if constexpr (std::is_same<OUT, __half>::value) {
        const __half2 h = __floats2half2_rn(lo, hi);
        return *reinterpret_cast<const uint32_t *>(&h);
    } else {
        const __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
        return *reinterpret_cast<const uint32_t *>(&h);
    }
}

// One accumulator row chunk (32 columns) -> alpha * acc -> OUT, to `dst`; `valid` columns exist.
template <typename OUT>
__device__ __forceinline__ void store_chunk(OUT *dst, const uint32_t (&acc)[32], float alpha, int valid, bool vec_ok) {
    __align__(16) OUT tmp[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) {
        const float v = alpha * __uint_as_float(acc[i]);
        if constexpr (std::is_same<OUT, float>::value) tmp[i] = v;
        else if constexpr (std::is_same<OUT, __half>::value) tmp[i] = __float2half_rn(v);
        else tmp[i] = __float2bfloat16_rn(v);
    }
    if (valid >= 32 && vec_ok) {
        const uint4 *s = reinterpret_cast<const uint4 *>(tmp);
#pragma unroll
        for (int i = 0; i < static_cast<int>(sizeof(OUT)) * 2; ++i) reinterpret_cast<uint4 *>(dst)[i] = s[i];
    } else {
#pragma unroll
        for (int i = 0; i < 32; ++i)
            if (i < valid) dst[i] = tmp[i];
    }
}

// ---------------------------------------------------------------------------- host helpers

using EncodeTiledFn = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                   const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// The driver entry point is looked up through the runtime, so the library has no link-time
// dependency on libcuda and can be loaded (not run) on a machine without a GPU driver.
inline EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = [] {
        void *sym = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            sym = nullptr;
        return reinterpret_cast<EncodeTiledFn>(sym);
    }();
    return fn;
}

// K-major operand [rows, row_bytes] (bytes, row-major); box = `box_bytes` x box_rows with the
// swizzle whose span equals the box width (128 or 64 bytes).
inline int make_operand_map(CUtensorMap *map, const void *base, int64_t rows, int64_t row_bytes, int box_rows,
                            int box_bytes = 128) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return FOS_ERR_CUDA;
    cuuint64_t dims[2] = {static_cast<cuuint64_t>(row_bytes), static_cast<cuuint64_t>(rows)};
    cuuint64_t strides[1] = {static_cast<cuuint64_t>(row_bytes)};
    cuuint32_t box[2] = {static_cast<cuuint32_t>(box_bytes), static_cast<cuuint32_t>(box_rows)};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, box_bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? FOS_OK : FOS_ERR_CUDA;
}

}  // namespace
}  // namespace fos
