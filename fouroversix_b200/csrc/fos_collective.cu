// Second half of the row-parallel exchange. fos_gemm_nvfp4_scatter has written every rank's partial
// product of slab o (the 128-row blocks mb of the output with mb % world == o, in order) into rank o's
// staging buffer, plane by plane, over NVLink while its tiles completed. Here rank o adds the planes of its slab in binary32
// (in rank order, so the sum does not depend on who computes it: only the owner does), rounds once to
// the output type and stores the result into the output buffer of EVERY rank (plain peer stores).
// Between the two kernels, and after this one, the ranks need a barrier in stream order.
#include "fos_common.cuh"

namespace fos {
namespace {

struct ReduceGatherParams {
    const void *staging;     // this rank's staging buffer: [world][slab_rows][ld_staging]
    void *out_peer[8];       // every rank's output buffer [world * slab_rows][ld_out] (peer mappings)
    int world, rank;
    int64_t slab_rows, n, ld_staging, ld_out;
};

template <typename T> __device__ __forceinline__ float2 pair_to_float2(uint32_t w);
template <> __device__ __forceinline__ float2 pair_to_float2<__nv_bfloat16>(uint32_t w) {
    return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u));
}
template <> __device__ __forceinline__ float2 pair_to_float2<__half>(uint32_t w) {
    return __half22float2(*reinterpret_cast<__half2 *>(&w));
}
template <typename T> __device__ __forceinline__ uint32_t float2_to_pair(float lo, float hi);
template <> __device__ __forceinline__ uint32_t float2_to_pair<__nv_bfloat16>(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t *>(&v);
}
template <> __device__ __forceinline__ uint32_t float2_to_pair<__half>(float lo, float hi) {
    const __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t *>(&v);
}

// One thread per 8 output values (16 bytes): world 16-byte loads, one 16-byte store per rank.
template <typename T>
__global__ void __launch_bounds__(256) reduce_gather_kernel(const ReduceGatherParams p) {
    const int64_t chunks_per_row = p.n >> 3, total = p.slab_rows * chunks_per_row;
    const T *staging = static_cast<const T *>(p.staging);
    const int64_t plane = p.slab_rows * p.ld_staging;
    for (int64_t u = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; u < total;
         u += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int64_t i = u / chunks_per_row, j = (u - i * chunks_per_row) * 8;
        float acc[8] = {0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f};
        uint4 w[8];
#pragma unroll
        for (int s = 0; s < 8; ++s)
            if (s < p.world) w[s] = *reinterpret_cast<const uint4 *>(staging + s * plane + i * p.ld_staging + j);
#pragma unroll
        for (int s = 0; s < 8; ++s) {
            if (s >= p.world) break;
            const uint32_t v[4] = {w[s].x, w[s].y, w[s].z, w[s].w};
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const float2 f = pair_to_float2<T>(v[k]);
                acc[2 * k] += f.x;
                acc[2 * k + 1] += f.y;
            }
        }
        const uint4 r = make_uint4(float2_to_pair<T>(acc[0], acc[1]), float2_to_pair<T>(acc[2], acc[3]),
                                   float2_to_pair<T>(acc[4], acc[5]), float2_to_pair<T>(acc[6], acc[7]));
        // slab row i is row i % 128 of the slab's block i / 128, which is row block (i / 128) * world + rank of the output
        const int64_t off = (((i >> 7) * p.world + p.rank) * 128 + (i & 127)) * p.ld_out + j;
#pragma unroll
        for (int t = 0; t < 8; ++t)
            if (t < p.world) *reinterpret_cast<uint4 *>(static_cast<T *>(p.out_peer[t]) + off) = r;
    }
}


// The whole exchange in one kernel, in place, for layers whose GEMM is too short to hide a scatter:
// every rank has stored its full partial product [rows][ld] into its own buffer; rank r LOADS row blocks
// mb % world == r from every rank's buffer (peer loads, 512 contiguous bytes per warp), adds them in
// binary32 in rank order, rounds once and STORES the block back into every rank's buffer. Only rank r
// touches those rows anywhere, so the buffers can be reduced in place; inbound loads and outbound stores
// use the two directions of the links at the same time.
struct PullParams {
    void *buf_peer[8];       // every rank's buffer [rows][ld] (peer mappings; buf_peer[rank] is local)
    int world, rank;
    int64_t rows, n, ld;
};

template <typename T>
__global__ void __launch_bounds__(256) allreduce_pull_kernel(const PullParams p) {
    constexpr int U = 1;                                   // chunks per thread and round (4 measured no faster: the links are the limit)
    const int64_t chunks_per_row = p.n >> 3, slab_rows = p.rows / p.world, total = slab_rows * chunks_per_row;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t u0 = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; u0 < total; u0 += U * stride) {
        int64_t off[U];
        uint4 w[U][8];
#pragma unroll
        for (int q = 0; q < U; ++q) {
            const int64_t u = u0 + q * stride;
            const int64_t i = u / chunks_per_row, j = (u - i * chunks_per_row) * 8;
            off[q] = u < total ? (((i >> 7) * p.world + p.rank) * 128 + (i & 127)) * p.ld + j : -1;
#pragma unroll
            for (int s = 0; s < 8; ++s)
                if (s < p.world && off[q] >= 0)
                    w[q][s] = *reinterpret_cast<const uint4 *>(static_cast<const T *>(p.buf_peer[s]) + off[q]);
        }
#pragma unroll
        for (int q = 0; q < U; ++q) {
            if (off[q] < 0) continue;
            float acc[8] = {0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
            for (int s = 0; s < 8; ++s) {
                if (s >= p.world) break;
                const uint32_t v[4] = {w[q][s].x, w[q][s].y, w[q][s].z, w[q][s].w};
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const float2 f = pair_to_float2<T>(v[k]);
                    acc[2 * k] += f.x;
                    acc[2 * k + 1] += f.y;
                }
            }
            const uint4 r = make_uint4(float2_to_pair<T>(acc[0], acc[1]), float2_to_pair<T>(acc[2], acc[3]),
                                       float2_to_pair<T>(acc[4], acc[5]), float2_to_pair<T>(acc[6], acc[7]));
#pragma unroll
            for (int t = 0; t < 8; ++t)
                if (t < p.world) *reinterpret_cast<uint4 *>(static_cast<T *>(p.buf_peer[t]) + off[q]) = r;
        }
    }
}

// Reduce-scatter over peer memory, for layers that hand row slabs on instead of full activations: every rank has
// stored its partial product into its own buffer; this rank LOADS rows row0 .. row0 + rows of every rank's buffer
// (peer loads, a warp reads 512 contiguous bytes), adds them in binary32 in rank order, rounds once and stores the
// sums into a LOCAL buffer. Nothing is stored to a peer, so per GPU (world - 1) / world of the slab's bytes cross its
// links inbound, once. The caller puts a barrier between the GEMMs and this kernel, and another one before any
// rank overwrites its buffer.
struct ReduceScatterParams {
    const void *buf_peer[8];
    void *out;
    int world;
    int64_t row0, rows, n, ld, ld_out;
};

template <typename T>
__global__ void __launch_bounds__(256) reduce_scatter_peer_kernel(const ReduceScatterParams p) {
    constexpr int U = 2;                                   // chunks of 16 bytes per thread and round, loaded before any is used
    const int64_t chunks_per_row = p.n >> 3, total = p.rows * chunks_per_row;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t u0 = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; u0 < total; u0 += U * stride) {
        int64_t src[U], dst[U];
        uint4 w[U][8];
#pragma unroll
        for (int q = 0; q < U; ++q) {
            const int64_t u = u0 + q * stride;
            const int64_t i = u / chunks_per_row, j = (u - i * chunks_per_row) * 8;
            src[q] = u < total ? (p.row0 + i) * p.ld + j : -1;
            dst[q] = i * p.ld_out + j;
#pragma unroll
            for (int s = 0; s < 8; ++s)
                if (s < p.world && src[q] >= 0)
                    w[q][s] = *reinterpret_cast<const uint4 *>(static_cast<const T *>(p.buf_peer[s]) + src[q]);
        }
#pragma unroll
        for (int q = 0; q < U; ++q) {
            if (src[q] < 0) continue;
            float acc[8] = {0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
            for (int s = 0; s < 8; ++s) {
                if (s >= p.world) break;
                const uint32_t v[4] = {w[q][s].x, w[q][s].y, w[q][s].z, w[q][s].w};
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const float2 f = pair_to_float2<T>(v[k]);
                    acc[2 * k] += f.x;
                    acc[2 * k + 1] += f.y;
                }
            }
            *reinterpret_cast<uint4 *>(static_cast<T *>(p.out) + dst[q]) =
                make_uint4(float2_to_pair<T>(acc[0], acc[1]), float2_to_pair<T>(acc[2], acc[3]),
                           float2_to_pair<T>(acc[4], acc[5]), float2_to_pair<T>(acc[6], acc[7]));
        }
    }
}

// All-gather over peer memory: every rank holds its piece (`bytes` bytes at byte offset src_off of its buffer);
// this rank copies all pieces, in rank order, into a LOCAL buffer: dst[r * bytes ..] = buf_peer[r][src_off ..].
// Plain 16-byte peer loads, four in flight per thread; nothing is stored to a peer.
struct AllGatherParams {
    const void *buf_peer[8];
    void *dst;
    int world;
    int64_t src_off, bytes;
};

__global__ void __launch_bounds__(256) allgather_peer_kernel(const AllGatherParams p) {
    constexpr int U = 4;
    const int64_t per_rank = p.bytes >> 4, total = per_rank * p.world;      // 16-byte chunks
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t u0 = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; u0 < total; u0 += U * stride) {
        uint4 w[U];
#pragma unroll
        for (int q = 0; q < U; ++q) {
            const int64_t u = u0 + q * stride;
            if (u < total) {
                // (total < 2^31 chunks is checked on the host: a 32-bit division)
                const uint32_t r = static_cast<uint32_t>(u) / static_cast<uint32_t>(per_rank);
                const int64_t c = u - static_cast<int64_t>(r) * per_rank;
                w[q] = *reinterpret_cast<const uint4 *>(static_cast<const uint8_t *>(p.buf_peer[r]) + p.src_off + (c << 4));
            }
        }
#pragma unroll
        for (int q = 0; q < U; ++q) {
            const int64_t u = u0 + q * stride;
            if (u < total) *reinterpret_cast<uint4 *>(static_cast<uint8_t *>(p.dst) + (u << 4)) = w[q];
        }
    }
}

}  // namespace
}  // namespace fos

extern "C" int fos_reduce_gather(const void *staging, void *const *out_peers, int world, int rank, int64_t slab_rows,
                                 int64_t n, int64_t ld_staging, int64_t ld_out, int dtype, void *stream_) {
    using namespace fos;
    if (!staging || !out_peers || world < 2 || world > 8 || rank < 0 || rank >= world) return FOS_ERR_INVALID_ARGUMENT;
    if (slab_rows <= 0 || slab_rows % 128 != 0 || n <= 0 || ld_staging < n || ld_out < n) return FOS_ERR_INVALID_ARGUMENT;
    if (dtype != FOS_BF16 && dtype != FOS_FP16) return FOS_ERR_UNSUPPORTED;
    if (n % 8 != 0 || ld_staging % 8 != 0 || ld_out % 8 != 0) return FOS_ERR_UNSUPPORTED;
    if (reinterpret_cast<uintptr_t>(staging) % 16 != 0) return FOS_ERR_MISALIGNED;
    ReduceGatherParams p{};
    p.staging = staging;
    for (int i = 0; i < world; ++i) {
        if (!out_peers[i]) return FOS_ERR_INVALID_ARGUMENT;
        if (reinterpret_cast<uintptr_t>(out_peers[i]) % 16 != 0) return FOS_ERR_MISALIGNED;
        p.out_peer[i] = out_peers[i];
    }
    p.world = world; p.rank = rank;
    p.slab_rows = slab_rows; p.n = n; p.ld_staging = ld_staging; p.ld_out = ld_out;
    const int st = check_device();
    if (st != FOS_OK) return st;
    const int64_t total = slab_rows * (n >> 3);
    int64_t blocks = (total + 255) / 256;
    if (blocks > 148 * 8) blocks = 148 * 8;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (dtype == FOS_BF16) reduce_gather_kernel<__nv_bfloat16><<<static_cast<unsigned>(blocks), 256, 0, stream>>>(p);
    else reduce_gather_kernel<__half><<<static_cast<unsigned>(blocks), 256, 0, stream>>>(p);
    FOS_CUDA_TRY(cudaGetLastError());
    return FOS_OK;
}

extern "C" int fos_allreduce_peer(void *const *buf_peers, int world, int rank, int64_t rows, int64_t n, int64_t ld,
                                  int dtype, void *stream_) {
    using namespace fos;
    if (!buf_peers || world < 2 || world > 8 || rank < 0 || rank >= world) return FOS_ERR_INVALID_ARGUMENT;
    if (rows <= 0 || n <= 0 || ld < n) return FOS_ERR_INVALID_ARGUMENT;
    if (dtype != FOS_BF16 && dtype != FOS_FP16) return FOS_ERR_UNSUPPORTED;
    if (rows % (128 * static_cast<int64_t>(world)) != 0 || n % 8 != 0 || ld % 8 != 0) return FOS_ERR_UNSUPPORTED;
    PullParams p{};
    for (int i = 0; i < world; ++i) {
        if (!buf_peers[i]) return FOS_ERR_INVALID_ARGUMENT;
        if (reinterpret_cast<uintptr_t>(buf_peers[i]) % 16 != 0) return FOS_ERR_MISALIGNED;
        p.buf_peer[i] = buf_peers[i];
    }
    p.world = world; p.rank = rank; p.rows = rows; p.n = n; p.ld = ld;
    const int st = check_device();
    if (st != FOS_OK) return st;
    const int64_t total = (rows / world) * (n >> 3);
    int64_t blocks = (total + 255) / 256;
    if (blocks > 148 * 8) blocks = 148 * 8;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (dtype == FOS_BF16) allreduce_pull_kernel<__nv_bfloat16><<<static_cast<unsigned>(blocks), 256, 0, stream>>>(p);
    else allreduce_pull_kernel<__half><<<static_cast<unsigned>(blocks), 256, 0, stream>>>(p);
    FOS_CUDA_TRY(cudaGetLastError());
    return FOS_OK;
}

extern "C" int fos_reduce_scatter_peer(void *const *buf_peers, int world, int64_t row0, int64_t rows, int64_t n, int64_t ld,
                                       void *out, int64_t ld_out, int dtype, int max_ctas, void *stream_) {
    using namespace fos;
    if (!buf_peers || !out || world < 2 || world > 8) return FOS_ERR_INVALID_ARGUMENT;
    if (row0 < 0 || rows <= 0 || n <= 0 || ld < n || ld_out < n || max_ctas < 0) return FOS_ERR_INVALID_ARGUMENT;
    if (dtype != FOS_BF16 && dtype != FOS_FP16) return FOS_ERR_UNSUPPORTED;
    if (n % 8 != 0 || ld % 8 != 0 || ld_out % 8 != 0) return FOS_ERR_UNSUPPORTED;
    if (reinterpret_cast<uintptr_t>(out) % 16 != 0) return FOS_ERR_MISALIGNED;
    ReduceScatterParams p{};
    for (int i = 0; i < world; ++i) {
        if (!buf_peers[i]) return FOS_ERR_INVALID_ARGUMENT;
        if (reinterpret_cast<uintptr_t>(buf_peers[i]) % 16 != 0) return FOS_ERR_MISALIGNED;
        p.buf_peer[i] = buf_peers[i];
    }
    p.out = out;
    p.world = world;
    p.row0 = row0; p.rows = rows; p.n = n; p.ld = ld; p.ld_out = ld_out;
    const int st = check_device();
    if (st != FOS_OK) return st;
    const int64_t total = rows * (n >> 3);
    int64_t blocks = (total + 511) / 512;
    const int64_t cap = max_ctas > 0 ? max_ctas : 148 * 8;
    if (blocks > cap) blocks = cap;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (dtype == FOS_BF16) reduce_scatter_peer_kernel<__nv_bfloat16><<<static_cast<unsigned>(blocks), 256, 0, stream>>>(p);
    else reduce_scatter_peer_kernel<__half><<<static_cast<unsigned>(blocks), 256, 0, stream>>>(p);
    FOS_CUDA_TRY(cudaGetLastError());
    return FOS_OK;
}

extern "C" int fos_allgather_peer(void *const *buf_peers, int world, int64_t src_off, int64_t bytes, void *dst,
                                  int max_ctas, void *stream_) {
    using namespace fos;
    if (!buf_peers || !dst || world < 2 || world > 8 || src_off < 0 || bytes <= 0 || max_ctas < 0) return FOS_ERR_INVALID_ARGUMENT;
    if (bytes % 16 != 0 || src_off % 16 != 0) return FOS_ERR_UNSUPPORTED;
    if (reinterpret_cast<uintptr_t>(dst) % 16 != 0) return FOS_ERR_MISALIGNED;
    if ((bytes >> 4) * world >= (int64_t(1) << 31)) return FOS_ERR_TOO_LARGE;
    AllGatherParams p{};
    for (int i = 0; i < world; ++i) {
        if (!buf_peers[i]) return FOS_ERR_INVALID_ARGUMENT;
        if (reinterpret_cast<uintptr_t>(buf_peers[i]) % 16 != 0) return FOS_ERR_MISALIGNED;
        p.buf_peer[i] = buf_peers[i];
    }
    p.dst = dst;
    p.world = world;
    p.src_off = src_off;
    p.bytes = bytes;
    const int st = check_device();
    if (st != FOS_OK) return st;
    const int64_t total = (bytes >> 4) * world;
    int64_t blocks = (total + 1023) / 1024;
    const int64_t cap = max_ctas > 0 ? max_ctas : 148 * 8;
    if (blocks > cap) blocks = cap;
    allgather_peer_kernel<<<static_cast<unsigned>(blocks), 256, 0, static_cast<cudaStream_t>(stream_)>>>(p);
    FOS_CUDA_TRY(cudaGetLastError());
    return FOS_OK;
}
