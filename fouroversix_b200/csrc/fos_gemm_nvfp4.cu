// Block-scaled NVFP4 GEMM for sm_100a: D[m, n] = alpha * sum_k A[m, k] * B[n, k].
//
// Both operands are K-major packed E2M1 with one UE4M3 scale per 16 values, stored as
// fos_quantize writes them (scales in 128-row x 4-block tiles of 512 bytes). The kernel
// is persistent (one CTA per SM, static tile schedule) and warp specialised. Every role that
// issues TMA or tcgen05 instructions runs as a WHOLE warp with one elected lane issuing: with
// every value of its loop the same in all lanes the compiler keeps addresses and descriptors in
// uniform registers, which those instructions take directly; a lone thread's values live in
// ordinary registers and each instruction pays for moving its operands over (the single change
// from "one thread" to "one warp, one elected lane" took 8192^3 from 256 to 235 us, and the MMA
// rate of the CTA-pair kernel from 182 to 152 us).
//
//   warp 0      TMA loads: per stage the A / B tiles (128-byte swizzle, no multicast) into a ring of
//               shared-memory stages guarded by full / empty mbarriers, and - one stage AHEAD of
//               them, because their way into the MMA is longer - the two tensor copies of the
//               scale tiles into a ring of their own that is one slot longer
//   warp 1      allocates tensor memory; issues tcgen05.mma kind::mxf4nvf4.block_scale
//               (K = 64 per instruction) with the fp32 accumulator in tensor memory;
//               tcgen05.commit releases the stage
//   warps 2..9  epilogue: tcgen05.ld the accumulator (each warp owns the 32 lanes of its
//               quadrant and half of the tile's columns), multiply by alpha, convert, store
//               rows < m and columns < n. 16-bit outputs are packed while they are read, so the
//               warp's whole row segment sits in registers and the accumulator is handed back
//               to the MMA warp before the first store; stores are 32 bytes per lane.
//               (FUSED_A: the same warps first build the A tiles and their scales, see below.)
//   warps 10-11 copy each stage's scale tiles shared -> tensor memory with tcgen05.cp
//               32x128b.warpx4 (a 512-byte tile is 32 rows of 16 bytes, which every 32-lane
//               quadrant of tensor memory needs: the copy broadcasts it) into a ring of scale
//               columns, one slot per scale stage, taking stages in turn, and tcgen05.commit
//               the slot's `ready` barrier. Issued from the MMA warp the copies queue up in
//               line with the MMAs (372 us at 8192^3); from warps of their own they overlap
//               them, and two warps issue them faster than one (235 -> 219 us).
//
// What bounds the kernel now (8192^3, parts switched off in a -DFOS_GEMM_DEBUG build): MMAs alone
// 150 us, loads alone 148, loads + MMAs 176, everything 219. The scale copies are the largest
// single cost: twelve per stage, each about 30 ns of the copying warp and about 14 cycles of the
// tensor pipe that no MMA gets. Loads and MMAs together lose 26 us to the round trip of a stage
// (four 48 KB stages cannot cover it) and to the shared-memory port both use.
//
// Every mbarrier wait is bounded (in SM cycles). A wait that gives up records where
// in *status, raises a CTA-wide abort flag, and all roles fall through to the common exit,
// which lets in-flight copies land, releases tensor memory and returns.
#include "fos_tcgen05.cuh"

namespace fos {
namespace {

constexpr int BLOCK_M = 128;
constexpr int BLOCK_K_BYTES = 128;                 // 256 E2M1 values: one 128-byte swizzle row
constexpr int KB_PER_STAGE = 4;                    // MMA K-blocks (64 values, 32 bytes) per stage
constexpr int SF_TILE_BYTES = 512;                 // scales of 128 rows x 64 values
constexpr int A_BYTES = BLOCK_M * BLOCK_K_BYTES;   // 16 KiB
constexpr int SFA_BYTES = KB_PER_STAGE * SF_TILE_BYTES;
#ifndef FOS_GEMM_SF_LEAD
#define FOS_GEMM_SF_LEAD 1
#endif
constexpr int SF_LEAD = FOS_GEMM_SF_LEAD;   // 0 or 1: how many stages the scales are requested ahead of the operands
#ifndef FOS_GEMM_ST256
#define FOS_GEMM_ST256 1
#endif

constexpr int SF_CP_WARPS = 2;                     // warps 10 and 11 issue the scale copies, taking stages in turn
constexpr int NUM_THREADS = 384;                   // warps: 0 TMA, 1 MMA, 2-9 epilogue (FUSED_A: also the A operand), 10-11 scale copies
constexpr int MAX_GROUPS = 256;                    // of a grouped launch (their row ranges are kept in shared memory)
constexpr int SF_COL0 = 256;                       // tensor-memory columns: accumulators first, then per
                                                   // stage 16 columns of A scales and N/8 of B scales

template <int BLOCK_N> struct Cfg {
    static constexpr int B_BYTES = BLOCK_N * BLOCK_K_BYTES;
    static constexpr int N_GROUPS = BLOCK_N / 128;                 // 128-row scale groups of B
    static constexpr int SFB_BYTES = N_GROUPS * KB_PER_STAGE * SF_TILE_BYTES;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;          // operand tiles of one stage
    static constexpr int SF_SLOT_BYTES = SFA_BYTES + SFB_BYTES;    // scale tiles of one stage
    static constexpr int STAGES = BLOCK_N == 256 ? 4 : 6;
    // The scales of a stage are requested one stage earlier than its operands and have a ring of
    // their own (shared memory and tensor memory) with one slot more than there are stages.
    static constexpr int SF_SLOTS = STAGES + SF_LEAD;
    static constexpr int ACC_STAGES = BLOCK_N == 256 ? 1 : 2;
    static constexpr int BARRIER_BYTES = 512;
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + SF_SLOTS * SF_SLOT_BYTES + 1024 /*alignment slack*/ + BARRIER_BYTES;
    static constexpr int SFB_COLS = KB_PER_STAGE * (BLOCK_N / 32);  // per stage
    static constexpr int SF_STAGE_COLS = 16 + SFB_COLS;
    static_assert(STAGE_BYTES % 1024 == 0, "stages must keep the 1024-byte swizzle alignment");
    static_assert(ACC_STAGES * BLOCK_N <= SF_COL0, "accumulators overlap the scale columns");
    static_assert(SF_COL0 + SF_SLOTS * SF_STAGE_COLS <= TMEM_COLS, "scale ring does not fit tensor memory");
    static_assert(SMEM_BYTES <= 232448, "more shared memory than a CTA can have");
    static_assert((2 * STAGES + (SF_CP_WARPS + 1) * SF_SLOTS + 2 * ACC_STAGES + 1) * 8 + 8 <= BARRIER_BYTES, "barrier area too small");
};

struct GemmParams {
    const uint8_t *a_sf;
    const uint8_t *b_sf;
    const float *alpha;
    void *d;
    int32_t *status;         // where a bounded wait that gives up records its site: the caller's word, or the sticky one
    int64_t m_p, n_p, k_p;   // padded problem (k_p in values)
    int64_t m, n, ldd;       // region of D that is written
    int out_dtype;
    int debug;               // timing-experiment bits; only read in builds with -DFOS_GEMM_DEBUG (results are wrong with any set)
    int mx;                  // operands are MXFP4: E8M0 scales per 32 values, a 512-byte scale tile spans 128 values of K
    // Row-parallel layers: this rank's partial product is not stored to d but scattered, tile by tile as
    // the tiles complete, into the staging buffers of the ranks that will reduce them. Row block mb (128
    // rows) belongs to rank mb % scatter_world and is block mb / scatter_world of that rank's slab of
    // `slab_rows` rows; its staging buffer d_peer[o] (a peer mapping unless o is this rank) is
    // [world][slab_rows][ldd], and this rank writes plane scatter_rank.
    // Fused activation quantization (gemm_nvfp4_kernel<.., FUSED_A>): A is not read packed but made in the
    // kernel from x[m, k] (bf16 / fp16, row stride x_ld elements) with NVFP4 static_6 / static_4 and the
    // per-tensor amax at x_amax; a_sf is unused.
    const void *x;
    int64_t x_ld;
    const float *x_amax;
    int x_rule;
    int x_is_fp16;
    int scatter_world;       // 0: plain store to d
    int scatter_rank;
    int64_t slab_rows;
    void *d_peer[8];
    // Grouped problems (gemm_nvfp4_kernel<.., GROUPED>): A, its scales and D are the groups' rows one after
    // the other, group g at rows group_start[g] .. group_start[g + 1] (multiples of 128, read on the device: the
    // host need not know them) of which the first group_rows[g] are written to D; B and its scales are
    // num_groups matrices of n_p rows each, one after the other; alpha has one entry per group.
    const int32_t *group_start;
    const int32_t *group_rows;
    int num_groups;
};

// ---------------------------------------------------------------------------- MMA wrappers

// MXFP4: two E8M0 scales per row and K-block (scale_vec::2X); which two of the four bytes of a
// scale column an instruction uses is part of its descriptor.
__device__ __forceinline__ void tc_mma_mxf4(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                            uint32_t sfa_tmem, uint32_t sfb_tmem, uint32_t accumulate) {
    asm volatile(
        "{ .reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::mxf4.block_scale.scale_vec::2X [%0], %1, %2, %3, [%5], [%6], p; }\n"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem)
        : "memory");
}

// Descriptors in two halves. The upper word of a shared-memory matrix descriptor is the same for every
// tile of a kind (stride byte offset, version, swizzle) and the lower word is the start address >> 4
// (shared-memory addresses stay below 2^18, so adding a byte offset >> 4 never carries out of the field):
// the issuing threads keep one lower word per stage and add constants, instead of rebuilding 64-bit
// descriptors for every instruction - a single thread issues every copy and every MMA of an SM, and
// what it executes between two of them is what bounds its rate.
constexpr uint32_t DESC_HI_OPERAND = (1024u >> 4) | (1u << 14) | (2u << 29);   // SBO 1024, version 1, 128-byte swizzle
constexpr uint32_t DESC_HI_SCALES = (128u >> 4) | (1u << 14);                   // SBO 128, version 1, no swizzle
__device__ __forceinline__ uint32_t desc_lo(uint32_t addr, uint32_t lbo_bytes = 0) {
    return ((addr & 0x3ffffu) >> 4) | ((lbo_bytes >> 4) << 16);
}
__device__ __forceinline__ void tc_copy_sf_lo(uint32_t taddr, uint32_t lo) {
    asm volatile("{ .reg .b64 d;\n"
                 "mov.b64 d, {%1, %2};\n"
                 "tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], d; }" ::"r"(taddr), "r"(lo), "r"(DESC_HI_SCALES) : "memory");
}
__device__ __forceinline__ void tc_copy_sf_pair_lo(uint32_t taddr, uint32_t lo) {
    asm volatile("{ .reg .b64 d;\n"
                 "mov.b64 d, {%1, %2};\n"
                 "tcgen05.cp.cta_group::2.32x128b.warpx4 [%0], d; }" ::"r"(taddr), "r"(lo), "r"(DESC_HI_SCALES) : "memory");
}
__device__ __forceinline__ void tc_mma_nvf4_lo(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t idesc,
                                               uint32_t sfa_tmem, uint32_t sfb_tmem, uint32_t accumulate) {
    asm volatile(
        "{ .reg .pred p;\n"
        ".reg .b64 da, db;\n"
        "mov.b64 da, {%1, %7};\n"
        "mov.b64 db, {%2, %7};\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], da, db, %3, [%5], [%6], p; }\n"
        ::"r"(d_tmem), "r"(a_lo), "r"(b_lo), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem), "r"(DESC_HI_OPERAND)
        : "memory");
}
__device__ __forceinline__ void tc_mma_nvf4_pair_lo(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t idesc,
                                                    uint32_t sfa_tmem, uint32_t sfb_tmem, uint32_t accumulate) {
    asm volatile(
        "{ .reg .pred p;\n"
        ".reg .b64 da, db;\n"
        "mov.b64 da, {%1, %7};\n"
        "mov.b64 db, {%2, %7};\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::2.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], da, db, %3, [%5], [%6], p; }\n"
        ::"r"(d_tmem), "r"(a_lo), "r"(b_lo), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem), "r"(DESC_HI_OPERAND)
        : "memory");
}

// Instruction descriptor of kind::mxf4nvf4 block-scaled MMA: A and B E2M1 (code 1 in bits
// [7,10) and [10,13)), both K-major, N >> 3 in [17,23), UE4M3 scales (bit 23 = 0), M >> 4 in
// [24,29), scale-factor byte ids 0, dense K = 64. MXFP4: E8M0 scales (bit 23 = 1) and the byte
// offset (0 or 2) of the instruction's two scales inside the 32-bit scale column in [4,6) for B
// and [29,31) for A.
__device__ __forceinline__ uint32_t mma_idesc(int n, int m = BLOCK_M) {
    return (1u << 7) | (1u << 10) | (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(m >> 4) << 24);
}
__device__ __forceinline__ uint32_t mma_idesc_mx(uint32_t idesc, uint32_t sf_byte) {
    return idesc | (1u << 23) | (sf_byte << 4) | (sf_byte << 29);
}

// ---------------------------------------------------------------------------- kernel

template <int BLOCK_N, typename OUT, bool FUSED_A = false, bool GROUPED = false>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_nvfp4_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                  const __grid_constant__ CUtensorMap map_sfa, const __grid_constant__ CUtensorMap map_sfb,
                  const GemmParams p) {
    using C = Cfg<BLOCK_N>;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));

    // shared memory: operand stages, scale slots, barriers
    const uint32_t sf_base = smem_base + C::STAGES * C::STAGE_BYTES;
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem_gen + C::STAGES * C::STAGE_BYTES + C::SF_SLOTS * C::SF_SLOT_BYTES);
    const uint32_t full_bar = smem_u32(bars);                       // [STAGES] operand tiles landed
    const uint32_t empty_bar = full_bar + 8 * C::STAGES;            // [STAGES] the stage's MMAs are done
    const uint32_t sf_full_bar = empty_bar + 8 * C::STAGES;         // [SF_CP_WARPS][SF_SLOTS] scale tiles landed
    const uint32_t sf_ready_bar = sf_full_bar + 8 * SF_CP_WARPS * C::SF_SLOTS;   // [SF_SLOTS] scales are in tensor memory
    const uint32_t acc_full_bar = sf_ready_bar + 8 * C::SF_SLOTS;   // [ACC_STAGES]
    const uint32_t acc_empty_bar = acc_full_bar + 8 * C::ACC_STAGES;
    const uint32_t drain_bar = acc_empty_bar + 8 * C::ACC_STAGES;   // only used when the CTA gives up
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 2 * C::STAGES + (SF_CP_WARPS + 1) * C::SF_SLOTS + 2 * C::ACC_STAGES + 1);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    // GROUPED: first row of every group (and one past the last group), and one past each group's last valid row
    __shared__ int32_t grp_start[GROUPED ? MAX_GROUPS + 1 : 1], grp_end[GROUPED ? MAX_GROUPS : 1];
    if constexpr (GROUPED) {
        const int32_t cap = static_cast<int32_t>(p.m_p);
        // (the same number of rounds in every thread, and the warps converged again before the warp-wide
        // instructions below - tcgen05.alloc, elect.sync: a loop that only some lanes of a warp enter leaves
        // the warp split, and those instructions are undefined for a split warp)
        for (int g0 = 0; g0 <= p.num_groups; g0 += NUM_THREADS) {
            const int g = g0 + static_cast<int>(threadIdx.x);
            if (g <= p.num_groups) {
                int32_t s0 = __ldg(p.group_start + g);
                s0 = (s0 < 0 ? 0 : (s0 > cap ? cap : s0)) & ~127;             // never beyond the buffers
                grp_start[g] = s0;
                if (g < p.num_groups) {
                    // valid rows end inside the group's own range, whatever group_rows claims
                    int32_t s1 = __ldg(p.group_start + g + 1);
                    s1 = (s1 < s0 ? s0 : (s1 > cap ? cap : s1)) & ~127;
                    const int32_t r = __ldg(p.group_rows + g), e = s0 + (r < 0 ? 0 : r);
                    grp_end[g] = e > s1 ? s1 : e;
                }
            }
        }
        __syncwarp();
    }

    if (threadIdx.x == 0) {
        // FUSED_A: besides the copy engine (B, B's scales), the eight warps that make A and its scales arrive
        for (int s = 0; s < C::STAGES; ++s) {
            mbar_init(full_bar + 8 * s, FUSED_A ? 9 : 1);
            mbar_init(empty_bar + 8 * s, 1);
        }
        for (int j = 0; j < C::SF_SLOTS; ++j) {
            for (int w = 0; w < SF_CP_WARPS; ++w) mbar_init(sf_full_bar + 8 * (w * C::SF_SLOTS + j), FUSED_A ? 9 : 1);
            mbar_init(sf_ready_bar + 8 * j, 1);                   // one commit by the warp that copied the slot
        }
        for (int a = 0; a < C::ACC_STAGES; ++a) {
            mbar_init(acc_full_bar + 8 * a, 1);
            mbar_init(acc_empty_bar + 8 * a, 8);   // one arrival per epilogue warp
        }
        mbar_init(drain_bar, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        __syncwarp();
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    const int64_t num_m = GROUPED ? grp_start[p.num_groups] / BLOCK_M : p.m_p / BLOCK_M;
    const int64_t num_n = (p.n_p + BLOCK_N - 1) / BLOCK_N;
    // GROUPED: the group that row block mb lies in (the last g with grp_start[g] <= row; empty groups are skipped)
    auto group_of = [&](int64_t mb) -> int {
        if constexpr (!GROUPED) return 0;
        const int32_t row = static_cast<int32_t>(mb * BLOCK_M);
        int lo = 0, hi = p.num_groups - 1;
        while (lo < hi) {
            const int mid = (lo + hi + 1) >> 1;
            if (grp_start[mid] <= row) lo = mid; else hi = mid - 1;
        }
        return lo;
    };
    const int64_t num_tiles = num_m * num_n;
    const int64_t k_blocks = p.k_p / 64;                       // MMA K-blocks in the problem
    const int64_t k_tiles = (k_blocks + KB_PER_STAGE - 1) / KB_PER_STAGE;

#ifdef FOS_GEMM_DEBUG
    const bool dbg_no_sf = p.debug & 1, dbg_no_load = p.debug & 2, dbg_no_store = p.debug & 4;
    const bool dbg_no_mma = p.debug & 16;
#else
    constexpr bool dbg_no_sf = false, dbg_no_load = false, dbg_no_store = false, dbg_no_mma = false;
#endif
    if (warp == 0 && !dbg_no_load) {
        // ------------------------------------------------------------------ TMA producer: operands and scales
        // One warp, one elected lane: per stage the two operand tiles and, SF_LEAD stages ahead of them (their
        // way into the MMA is longer: shared memory -> tcgen05.cp -> tensor memory), the two scale copies into
        // a ring of their own that is one slot longer.
        const bool issue = elect_one();
        int64_t f_t = blockIdx.x, f_kt = 0;          // the stage whose scales are requested next
        uint32_t slot = 0, f_w = 0;                  // its ring slot, and which copying warp will take it
        int a_group = 0, b_group = 0;
        auto enter_tile = [&]() {
            if (f_t >= num_tiles) return;
            int64_t mb, nb;
            tile_coords(f_t, num_m, num_n, mb, nb);
            a_group = static_cast<int>(mb);
            b_group = static_cast<int>(nb * C::N_GROUPS) + group_of(mb) * static_cast<int>(p.n_p / 128);
        };
        auto issue_next_scales = [&]() {
            if (f_t >= num_tiles || dbg_no_sf) return;
            // two tensor copies per stage: [K-blocks kb0 .. kb0+3] x [one / N_GROUPS row groups] of 512-byte tiles;
            // what lies beyond K or N is zero-filled and still counted (MXFP4: a tile spans two K-blocks, so the
            // box of its maps is two tiles per group)
            const int kb0 = static_cast<int>(f_kt * (p.mx ? KB_PER_STAGE / 2 : KB_PER_STAGE));
            const uint32_t dst = sf_base + slot * C::SF_SLOT_BYTES, bar = sf_full_bar + 8 * (f_w * C::SF_SLOTS + slot);
            if (issue) {
                if (FUSED_A) {
                    mbar_expect_tx(bar, C::SFB_BYTES);
                } else {
                    mbar_expect_tx(bar, p.mx ? C::SF_SLOT_BYTES / 2 : C::SF_SLOT_BYTES);
                    tma_load_3d(dst, &map_sfa, 0, kb0, a_group, bar);
                }
                tma_load_3d(dst + SFA_BYTES, &map_sfb, 0, kb0, b_group, bar);
            }
            if (++slot == C::SF_SLOTS) slot = 0;
            if (++f_w == SF_CP_WARPS) f_w = 0;
            if (++f_kt == k_tiles) {
                f_kt = 0;
                f_t += gridDim.x;
                enter_tile();
            }
        };
        enter_tile();
        for (int i = 0; i < SF_LEAD; ++i) issue_next_scales();
        uint32_t s = 0, ph = 0;
        bool ok = true;
        for (int64_t t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
            int64_t mb, nb;
            tile_coords(t, num_m, num_n, mb, nb);
            const int m0 = static_cast<int>(mb * BLOCK_M);
            const int n0 = static_cast<int>(nb * BLOCK_N) + group_of(mb) * static_cast<int>(p.n_p);   // row of B
            for (int64_t kt = 0; kt < k_tiles; ++kt) {
                // the stage is free; so is the scale slot of the iteration SF_LEAD ahead (SF_SLOTS = STAGES +
                // SF_LEAD back from it: its MMAs were done before this stage's)
                ok = __all_sync(0xffffffffu, mbar_wait(empty_bar + 8 * s, ph ^ 1u, abort_flag, p.status, 1));
                if (!ok) break;
                const uint32_t stage = smem_base + s * C::STAGE_BYTES, bar = full_bar + 8 * s;
                // rows beyond N and bytes beyond K are zero-filled by the TMA unit and still counted
                if (issue) {
                    mbar_expect_tx(bar, FUSED_A ? C::B_BYTES : C::STAGE_BYTES);
                    if (!FUSED_A) tma_load_2d(stage, &map_a, static_cast<int>(kt * BLOCK_K_BYTES), m0, bar);
                    tma_load_2d(stage + A_BYTES, &map_b, static_cast<int>(kt * BLOCK_K_BYTES), n0, bar);
                }
                issue_next_scales();
                __syncwarp();
                if (++s == C::STAGES) { s = 0; ph ^= 1u; }
            }
        }
        if (!ok) {
            // give copies that are still in flight time to land before the CTA exits
            const unsigned long long t0 = global_timer_ns();
            while (global_timer_ns() - t0 < 200000ull) __nanosleep(1000);
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        // (The whole warp runs this loop and one elected lane issues. With every value of the loop the same in
        // all lanes the compiler keeps descriptors and addresses in uniform registers, which the tcgen05
        // instructions take directly; a lone thread's values live in ordinary registers and every instruction
        // pays for moving its operands over: 256 -> 235 us at 8192^3, the CTA-pair kernel 343 -> 249 us.)
        const bool issue = elect_one();
        uint32_t s = 0, ph = 0, j = 0, jph = 0, tile_i = 0;      // operand stage / scale slot and their phases
        bool ok = true;
        for (int64_t t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++tile_i) {
            int64_t mb, nb;
            tile_coords(t, num_m, num_n, mb, nb);
            const int64_t n0 = nb * BLOCK_N;
            const int n_valid = static_cast<int>((p.n_p - n0) < BLOCK_N ? (p.n_p - n0) : BLOCK_N);
            const uint32_t idesc = mma_idesc(n_valid);
            const uint32_t acc = tile_i % C::ACC_STAGES, acc_ph = (tile_i / C::ACC_STAGES) & 1u;
            ok = mbar_wait(acc_empty_bar + 8 * acc, acc_ph ^ 1u, abort_flag, p.status, 3);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
            const uint32_t d_tmem = tmem_base + acc * BLOCK_N;
            for (int64_t kt = 0; kt < k_tiles; ++kt) {
                if (!dbg_no_load) {
                    ok = mbar_wait(full_bar + 8 * s, ph, abort_flag, p.status, 2);
                    if (ok && !dbg_no_sf) ok = mbar_wait(sf_ready_bar + 8 * j, jph, abort_flag, p.status, 5);
                }
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                tc_fence_after();
                const int64_t kb0 = kt * KB_PER_STAGE;
                const int nkb = static_cast<int>((k_blocks - kb0) < KB_PER_STAGE ? (k_blocks - kb0) : KB_PER_STAGE);
                const uint32_t stage = smem_base + s * C::STAGE_BYTES;
                // operands: 128-byte swizzled rows, 8-row groups 1024 bytes apart; each K-block
                // of 64 values is 32 bytes further along the row. Scales: this iteration's ring slot.
                const uint64_t a_desc = smem_desc(stage, 16, 1024, 2);
                const uint64_t b_desc = smem_desc(stage + A_BYTES, 16, 1024, 2);
                const uint32_t sfa_tmem = tmem_base + SF_COL0 + j * C::SF_STAGE_COLS, sfb_tmem = sfa_tmem + 16;
                if (p.mx) {
                    for (int kb = 0; kb < nkb && !dbg_no_mma && issue; ++kb)
                        tc_mma_mxf4(d_tmem, a_desc + 2 * kb, b_desc + 2 * kb, mma_idesc_mx(idesc, (kb & 1) * 2),
                                    sfa_tmem + 4 * (kb >> 1), sfb_tmem + (BLOCK_N / 32) * (kb >> 1),
                                    (kt > 0 || kb > 0) ? 1u : 0u);
                } else {
                    const uint32_t a_lo = desc_lo(stage, 16), b_lo = desc_lo(stage + A_BYTES, 16);
#pragma unroll
                    for (int kb = 0; kb < KB_PER_STAGE; ++kb) {
                        if (kb < nkb && !dbg_no_mma && issue)
                            tc_mma_nvf4_lo(d_tmem, a_lo + 2 * kb, b_lo + 2 * kb, idesc, sfa_tmem + 4 * kb,
                                           sfb_tmem + (BLOCK_N / 32) * kb, (kt > 0 || kb > 0) ? 1u : 0u);
                    }
                }
                if (issue) tc_commit(empty_bar + 8 * s);          // stage (and scale slot) reusable once these MMAs are done
                __syncwarp();
                if (++s == C::STAGES) { s = 0; ph ^= 1u; }
                if (++j == C::SF_SLOTS) { j = 0; jph ^= 1u; }
            }
            if (ok && issue) tc_commit(acc_full_bar + 8 * acc);  // accumulator complete
        }
        if (!ok) {
            // giving up: the MMAs already issued must have finished before tensor memory is released
            if (issue) tc_commit(drain_bar);
            __syncwarp();
            const long long t0 = clock64();
            while (!mbar_try_wait(drain_bar, 0) && clock64() - t0 < 20000000ll) {}   // about 10 ms
        }
    } else if (warp >= 2 && warp < 10) {
        // ------------------------------------------------------------------ epilogue
        const int quad = warp & 3;                       // tensor-memory lanes 32*quad .. +31
        constexpr int COLS = BLOCK_N / 2;                // columns per warp: left or right half
        const int half = (warp - 2) >> 2;
        float alpha = GROUPED ? 0.0f : __ldg(p.alpha);
        int64_t row_end = p.m;
        OUT *out = static_cast<OUT *>(p.d);
        const bool vec_ok = (reinterpret_cast<uintptr_t>(out) % 16 == 0) && ((p.ldd * sizeof(OUT)) % 16 == 0);
        const bool vec32_ok = FOS_GEMM_ST256 && (reinterpret_cast<uintptr_t>(out) % 32 == 0) && ((p.ldd * sizeof(OUT)) % 32 == 0);
        uint32_t tile_i = 0;
        bool ok = true;
        // FUSED_A: these eight warps are idle while a tile's MMAs run (one accumulator: the epilogue and the
        // next main loop do not overlap anyway), so they make the A operand: thread e owns row e / 2 of the
        // stage and 8 of its 16 blocks (128 values, 256 contiguous bytes of x).
        __shared__ float2 a_lut[FUSED_A ? 128 : 1];
        StaticQuantConsts qc{};
        uint32_t a_s = 0, a_ph = 0, a_j = 0, a_w = 0;
        const int e_tid = static_cast<int>(threadIdx.x) - 64, a_row = e_tid >> 1, a_half = e_tid & 1;
        if constexpr (FUSED_A) {
            qc = static_quant_consts(__ldg(p.x_amax), p.x_rule);
            if (e_tid < 128) a_lut[e_tid] = static_scale_entry(e_tid, qc.decode);
            asm volatile("bar.sync 1, 256;" ::: "memory");
        }
        for (int64_t t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++tile_i) {
            int64_t mb, nb;
            tile_coords(t, num_m, num_n, mb, nb);
            if constexpr (FUSED_A) {
                const int64_t x_row = mb * BLOCK_M + a_row;
                for (int64_t kt = 0; kt < k_tiles && ok; ++kt) {
                    // the values first (the loads do not depend on the stage), then the stage
                    uint32_t w[8][8];
                    const int64_t col0 = kt * 256 + a_half * 128;
#pragma unroll
                    for (int b = 0; b < 8; ++b) {
                        const int64_t col = col0 + 16 * b;
                        if (x_row < p.m && col < p.k_p) {
                            ldg_nc_32(static_cast<const uint16_t *>(p.x) + x_row * p.x_ld + col, w[b]);
                        } else {
#pragma unroll
                            for (int i = 0; i < 8; ++i) w[b][i] = 0u;
                        }
                    }
                    ok = mbar_wait(empty_bar + 8 * a_s, a_ph ^ 1u, abort_flag, p.status, 8);
                    ok = __all_sync(0xffffffffu, ok);
                    if (!ok) break;
                    const uint32_t a_stage = smem_base + a_s * C::STAGE_BYTES + a_row * 128;
                    const uint32_t sfa_slot = sf_base + a_j * C::SF_SLOT_BYTES + (a_row & 31) * 16 + (a_row >> 5) * 4;
                    uint32_t sf_word = 0u, codes[4] = {0u, 0u, 0u, 0u};
#pragma unroll
                    for (int b = 0; b < 8; ++b) {
                        float v[16];
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            const float2 f = p.x_is_fp16 ? unpack2<__half>(w[b][i]) : unpack2<__nv_bfloat16>(w[b][i]);
                            v[2 * i] = f.x;
                            v[2 * i + 1] = f.y;
                        }
                        uint32_t lo, hi, sfb;
                        quantize_block_static(v, qc, a_lut, lo, hi, sfb);
                        codes[2 * (b & 1)] = lo;
                        codes[2 * (b & 1) + 1] = hi;
                        sf_word |= sfb << (8 * (b & 3));
                        if (b & 1) {
                            // blocks 2c, 2c + 1 of the row are its 16-byte chunk c, stored where the 128-byte swizzle puts it
                            const int chunk = a_half * 4 + (b >> 1);
                            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};"
                                         ::"r"(a_stage + ((chunk ^ (a_row & 7)) << 4)), "r"(codes[0]), "r"(codes[1]), "r"(codes[2]), "r"(codes[3]) : "memory");
                        }
                        if ((b & 3) == 3) {
                            // the four scales of one K-block (64 values): one word of that K-block's 512-byte tile
                            asm volatile("st.shared.b32 [%0], %1;" ::"r"(sfa_slot + (a_half * 2 + (b >> 2)) * SF_TILE_BYTES), "r"(sf_word) : "memory");
                            sf_word = 0u;
                        }
                    }
                    // what these threads wrote is read by the tensor core and by tcgen05.cp: make it visible to that proxy
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    __syncwarp();
                    if (lane == 0) {
                        mbar_arrive(full_bar + 8 * a_s);
                        mbar_arrive(sf_full_bar + 8 * (a_w * C::SF_SLOTS + a_j));
                    }
                    if (++a_s == C::STAGES) { a_s = 0; a_ph ^= 1u; }
                    if (++a_j == C::SF_SLOTS) a_j = 0;
                    if (++a_w == SF_CP_WARPS) a_w = 0;
                }
                if (!ok) break;
            }
            const int64_t row = mb * BLOCK_M + quad * 32 + lane, n0 = nb * BLOCK_N + half * COLS;
            if constexpr (GROUPED) {
                const int grp = group_of(mb);
                alpha = __ldg(p.alpha + grp);
                row_end = grp_end[grp];
            }
            if (p.scatter_world > 1) {
                // row block mb belongs to rank mb % world (interleaved, so that the peer traffic is spread
                // over the whole run instead of coming in one burst per slab) and is block mb / world of
                // that rank's slab; plane `scatter_rank` of its buffer, addressed here by the global row
                const int o = static_cast<int>(mb % p.scatter_world);
                const int64_t first = static_cast<int64_t>(p.scatter_rank) * p.slab_rows + (mb / p.scatter_world) * BLOCK_M - mb * BLOCK_M;
                out = static_cast<OUT *>(p.d_peer[o]) + first * p.ldd;
            }
            const uint32_t acc = tile_i % C::ACC_STAGES, acc_ph = (tile_i / C::ACC_STAGES) & 1u;
            ok = mbar_wait(acc_full_bar + 8 * acc, acc_ph, abort_flag, p.status, 4);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
            const uint32_t t_acc = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + acc * BLOCK_N + half * COLS;
            const bool row_ok = row < row_end && !dbg_no_store;
            if constexpr (sizeof(OUT) == 2) {
                // 16-bit outputs: scale, convert and pack while reading, so that the warp's whole
                // row segment fits in registers and the accumulator goes back to the MMA warp
                // before the first store is issued
                uint32_t pk[COLS / 2];
#pragma unroll
                for (int c = 0; c < COLS / 32; ++c) {
                    uint32_t v[32];
                    tc_load_32cols_sync(t_acc + 32 * c, v);
                    if (c + 1 == COLS / 32) {
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(acc_empty_bar + 8 * acc);
                    }
#pragma unroll
                    for (int i = 0; i < 16; ++i)
                        pk[16 * c + i] = pack_pair<OUT>(alpha * __uint_as_float(v[2 * i]), alpha * __uint_as_float(v[2 * i + 1]));
                }
                const int64_t left = p.n - n0;
                if (row_ok && left > 0) {
                    OUT *dst = out + row * p.ldd + n0;
                    if (left >= COLS && vec32_ok) {
#ifdef FOS_GEMM_DEBUG
                        if (p.debug & 8) {
                            // timing experiment (values land in the wrong places): the same bytes stored so that
                            // every instruction of the warp fills four whole 256-byte row segments
                            uint8_t *wbase = reinterpret_cast<uint8_t *>(out + (row - lane) * p.ldd + n0);
#pragma unroll
                            for (int i = 0; i < COLS / 16; ++i)
                                if (row - lane + 4 * i + (lane >> 3) < row_end)
                                    stg_32_stream(wbase + (4 * i + (lane >> 3)) * p.ldd * sizeof(OUT) + (lane & 7) * 32, &pk[8 * i]);
                        } else
#endif
                        // 32 bytes per store: every instruction of the warp fills whole 32-byte sectors
#pragma unroll
                        for (int i = 0; i < COLS / 16; ++i) stg_32_stream(reinterpret_cast<uint8_t *>(dst) + 32 * i, &pk[8 * i]);
                    } else if (left >= COLS && vec_ok) {
#pragma unroll
                        for (int i = 0; i < COLS / 8; ++i)
                            reinterpret_cast<uint4 *>(dst)[i] = make_uint4(pk[4 * i], pk[4 * i + 1], pk[4 * i + 2], pk[4 * i + 3]);
                    } else {
                        uint16_t *d16 = reinterpret_cast<uint16_t *>(dst);
#pragma unroll
                        for (int i = 0; i < COLS; ++i)
                            if (i < left) d16[i] = static_cast<uint16_t>(pk[i >> 1] >> ((i & 1) * 16));
                    }
                }
            } else {
#pragma unroll 1
                for (int c = 0; c < COLS / 32; c += 2) {
                    uint32_t v0[32], v1[32];
                    tc_load_64cols_sync(t_acc + 32 * c, v0, v1);
                    if (c + 2 >= COLS / 32) {                // everything is in registers: release the accumulator
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(acc_empty_bar + 8 * acc);
                    }
                    const int64_t col = n0 + 32 * c;
                    const int64_t left0 = p.n - col, left1 = left0 - 32;
                    if (row_ok && left0 > 0)
                        store_chunk<OUT>(out + row * p.ldd + col, v0, alpha, left0 < 32 ? static_cast<int>(left0) : 32, vec_ok);
                    if (row_ok && left1 > 0)
                        store_chunk<OUT>(out + row * p.ldd + col + 32, v1, alpha, left1 < 32 ? static_cast<int>(left1) : 32, vec_ok);
                }
            }
        }
    } else if (warp >= 10 && warp < 10 + SF_CP_WARPS && !dbg_no_load && !dbg_no_sf) {
        // ------------------------------------------------------------------ scale copies by tcgen05.cp
        const bool issue = elect_one();
        // The warps take the stages in turn, and every (warp, slot) pair has a landing barrier of its own, which
        // the producer arms for the warp whose turn the stage will be: each barrier has one waiter, which sees
        // every one of its phases in order. (With ONE barrier per slot and an odd number of slots, a slot
        // alternated between the warps: a warp whose own stages had landed could reach its next use of a slot
        // before the other warp's stage in that slot had landed, take the barrier's not-yet-completed phase for
        // the one after it - a parity wait cannot tell them apart - and copy stale scales. Loads land out of
        // order when the kernel is bound by HBM: skinny problems computed with wrong scales and then hung.)
        const uint32_t me = static_cast<uint32_t>(warp - 10);
        uint32_t j = 0, turn = 0, seen = 0;          // bit j of `seen`: parity of this warp's next phase of slot j
        bool ok = true;
        for (int64_t t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
            for (int64_t kt = 0; kt < k_tiles; ++kt) {
                const bool mine = turn == me;
                if (++turn == SF_CP_WARPS) turn = 0;
                if (!mine) {
                    if (++j == C::SF_SLOTS) j = 0;
                    continue;
                }
                const uint32_t jph = (seen >> j) & 1u;
                seen ^= 1u << j;
                ok = mbar_wait(sf_full_bar + 8 * (me * C::SF_SLOTS + j), jph, abort_flag, p.status, 6);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                tc_fence_after();
                const uint32_t src = sf_base + j * C::SF_SLOT_BYTES, dst = tmem_base + SF_COL0 + j * C::SF_STAGE_COLS;
                // tiles: 32 rows of 16 bytes, 8-row groups 128 bytes apart, no swizzle
                // (MXFP4: a tile spans two K-blocks, so a stage has two tiles per group)
                const int ntile = p.mx ? KB_PER_STAGE / 2 : KB_PER_STAGE;
                const uint32_t src_lo = desc_lo(src);
#pragma unroll
                for (int kb = 0; kb < KB_PER_STAGE; ++kb) {
                    if (kb >= ntile || !issue) break;
                    tc_copy_sf_lo(dst + 4 * kb, src_lo + ((kb * SF_TILE_BYTES) >> 4));
#pragma unroll
                    for (int g = 0; g < C::N_GROUPS; ++g)
                        tc_copy_sf_lo(dst + 16 + (BLOCK_N / 32) * kb + 4 * g,
                                      src_lo + ((SFA_BYTES + (g * ntile + kb) * SF_TILE_BYTES) >> 4));
                }
                if (issue) tc_commit(sf_ready_bar + 8 * j);     // arrives when the copies above are done
                __syncwarp();
                if (++j == C::SF_SLOTS) j = 0;
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

// ---------------------------------------------------------------------------- CTA-pair kernel
//
// Two CTAs of a cluster (two SMs) compute one 256 x 256 tile with cta_group::2 MMAs: CTA r of
// the pair holds rows m0 + 128 r .. of A and rows n0 + 128 r .. of B in its shared memory,
// and the tensor cores of both SMs read both halves of B. Per MMA an SM moves a third less
// through shared memory than the single-CTA kernel, whose limit that is. Only the even CTA (the
// leader) issues MMAs; both CTAs run the two TMA producers, scale movers and an epilogue for their
// own 128 rows of the tile, with the same roles per warp as the single-CTA kernel.
//
//   full[s]      leader's barrier: one arrive.expect_tx by the leader's producer for the bytes of
//                BOTH CTAs; the peer's TMA loads complete on it too (cta_group::2 form of the copy)
//   empty[s]     one per CTA, released in both CTAs by the leader's multicast tcgen05.commit
//   sf_full[w][j] leader's barriers, one per (copying warp, slot) as in the single-CTA kernel: the scale
//                tiles of both CTAs have landed (each in its own CTA's shared memory), announced and
//                completed like full[s]
//   sf_ready[j]  leader's barrier: one of the leader's two copying warps has moved the slot's scales into
//                the tensor memory of both CTAs (tcgen05.cp with cta_group::2, one commit)
//   acc_full     one per CTA, multicast commit
//   acc_empty    leader's barrier, 16 arrivals: 8 epilogue warps of each CTA
//
// Barriers that the other SM arrives on are polled (test_wait) by their single waiting thread: a
// thread suspended in try_wait did not see such arrivals promptly. Remote arrives use the
// default (CTA-scope release) form: the cluster-scope release form cost about a microsecond each.
namespace pair {

constexpr int TILE_N = 256;
constexpr int B_HALF_BYTES = 128 * BLOCK_K_BYTES;                         // this CTA's 128 rows of B
constexpr int STAGE_BYTES = A_BYTES + B_HALF_BYTES;                       // 32 KiB
constexpr int SFB_BYTES = 2 * KB_PER_STAGE * SF_TILE_BYTES;               // scales of all 256 B rows
constexpr int SF_SLOT_BYTES = SFA_BYTES + SFB_BYTES;                      // 6 KiB
constexpr int STAGES = 6;
constexpr int SF_SLOTS = 5;                                               // what tensor memory has room for
constexpr int BARRIER_BYTES = 512;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + SF_SLOTS * SF_SLOT_BYTES + 1024 + BARRIER_BYTES;
constexpr int THREADS = 384;                                              // warps: 0 TMA (operands and scales), 1 MMA, 2-9 epilogue, 10-11 scale copies
constexpr int CP_WARPS = 2;                                               // they take the stages in turn (leader only)
constexpr int SF_STAGE_COLS = 16 + 32;                                    // A scales, B scales
static_assert(STAGE_BYTES % 1024 == 0, "stages must keep the 1024-byte swizzle alignment");
static_assert(SF_COL0 + SF_SLOTS * SF_STAGE_COLS <= TMEM_COLS, "scale ring does not fit tensor memory");
static_assert(SMEM_BYTES <= 232448, "more shared memory than a CTA can have");
static_assert((2 * STAGES + (CP_WARPS + 1) * SF_SLOTS + 2) * 8 + 8 <= BARRIER_BYTES, "barrier area too small");
static_assert(SF_SLOTS < STAGES, "the producer requests a stage's scales one iteration after its operands");

// 3-D form of the same (scale tiles).
__device__ __forceinline__ void tma_load_3d_pair(uint32_t dst, const CUtensorMap *map, int c0, int c1, int c2, uint32_t cluster_bar) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes.cta_group::2 [%0], [%1, {%2, %3, %4}], [%5];"
        ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(cluster_bar) : "memory");
}

// Arrive (once, on a barrier of this CTA) when the tcgen05 operations this thread issued for the pair are done.
__device__ __forceinline__ void tc_commit_pair_local(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// TMA tile load whose completion is signalled on a barrier of either CTA of the pair.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap *map, int c0, int c1, uint32_t cluster_bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes.cta_group::2 [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(cluster_bar) : "memory");
}

template <typename OUT>
__global__ void __launch_bounds__(THREADS, 1)
gemm_nvfp4_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                       const __grid_constant__ CUtensorMap map_sfa, const __grid_constant__ CUtensorMap map_sfb,
                       const GemmParams p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
    const uint32_t sf_base = smem_base + STAGES * STAGE_BYTES;
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem_gen + STAGES * STAGE_BYTES + SF_SLOTS * SF_SLOT_BYTES);
    const uint32_t full_bar = smem_u32(bars);                 // [STAGES], used in the leader only
    const uint32_t empty_bar = full_bar + 8 * STAGES;         // [STAGES]
    const uint32_t sf_full_bar = empty_bar + 8 * STAGES;      // [CP_WARPS][SF_SLOTS], used in the leader only
    const uint32_t sf_ready_bar = sf_full_bar + 8 * CP_WARPS * SF_SLOTS; // [SF_SLOTS], used in the leader only
    const uint32_t acc_full_bar = sf_ready_bar + 8 * SF_SLOTS;
    const uint32_t acc_empty_bar = acc_full_bar + 8;          // used in the leader only
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 2 * STAGES + (CP_WARPS + 1) * SF_SLOTS + 2);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_cta_rank();                 // 0 = leader
    const bool leader = rank == 0;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(full_bar + 8 * s, 1);
            mbar_init(empty_bar + 8 * s, 1);
        }
        for (int j = 0; j < SF_SLOTS; ++j) {
            for (int w = 0; w < CP_WARPS; ++w)
                mbar_init(sf_full_bar + 8 * (w * SF_SLOTS + j), 1);   // the scale tiles of BOTH CTAs have landed
            mbar_init(sf_ready_bar + 8 * j, 1);    // one commit after the copies into tensor memory
        }
        mbar_init(acc_full_bar, 1);
        mbar_init(acc_empty_bar, 16);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();            // both CTAs have initialised their barriers and tensor memory
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    const int64_t num_m = p.m_p / 256, num_n = p.n_p / TILE_N;
    const int64_t num_tiles = num_m * num_n;
    const int64_t k_blocks = p.k_p / 64;
    const int64_t k_tiles = (k_blocks + KB_PER_STAGE - 1) / KB_PER_STAGE;
    const int64_t pair_id = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
#ifdef FOS_GEMM_DEBUG
    const bool dbg_no_sf = p.debug & 1, dbg_no_load = p.debug & 2, dbg_no_store = p.debug & 4;
    const bool dbg_no_mma = p.debug & 16;
#else
    constexpr bool dbg_no_sf = false, dbg_no_load = false, dbg_no_store = false, dbg_no_mma = false;
#endif

    if (warp == 0 && lane == 0 && !dbg_no_load) {
        // ------------------------------------------------------------------ TMA producer: operands and scales (both CTAs)
        // Each CTA fetches its 128 rows of A and of B, and the scales of its own rows of A and of all 256 rows of B,
        // into its own shared memory; everything completes on the LEADER's barriers. The scale ring has one slot
        // less than the operand ring (tensor memory has room for five), so a stage's scales are requested one
        // iteration AFTER its operands: the wait that frees operand stage i (the MMAs of iteration i - STAGES are
        // done) also frees the scale slot of iteration i - 1. The first SF_SLOTS requests need no wait.
        const uint32_t leader_full = map_to_cta(full_bar, 0), leader_sf_full = map_to_cta(sf_full_bar, 0);
        int64_t f_t = pair_id, f_kt = 0;             // the stage whose scales are requested next
        uint32_t slot = 0, f_w = 0;                  // its ring slot, and which copying warp will take it
        int a_group = 0, b_group = 0;
        int64_t requested = 0, i = 0;                // scale requests and operand stages issued so far
        auto enter_tile = [&]() {
            if (f_t >= num_tiles) return;
            int64_t mb, nb;
            tile_coords(f_t, num_m, num_n, mb, nb);
            a_group = static_cast<int>(mb * 2 + rank);
            b_group = static_cast<int>(nb * 2);
        };
        auto issue_next_scales = [&]() {
            ++requested;
            if (f_t >= num_tiles || dbg_no_sf) return;
            const int kb0 = static_cast<int>(f_kt * KB_PER_STAGE);
            const uint32_t idx = 8 * (f_w * SF_SLOTS + slot);
            const uint32_t dst = sf_base + slot * SF_SLOT_BYTES, bar = leader_sf_full + idx;
            if (leader) mbar_expect_tx(sf_full_bar + idx, 2 * SF_SLOT_BYTES);
            tma_load_3d_pair(dst, &map_sfa, 0, kb0, a_group, bar);
            tma_load_3d_pair(dst + SFA_BYTES, &map_sfb, 0, kb0, b_group, bar);
            if (++slot == SF_SLOTS) slot = 0;
            if (++f_w == CP_WARPS) f_w = 0;
            if (++f_kt == k_tiles) {
                f_kt = 0;
                f_t += num_pairs;
                enter_tile();
            }
        };
        enter_tile();
        uint32_t s = 0, ph = 0;
        bool ok = true;
        for (int64_t t = pair_id; t < num_tiles && ok; t += num_pairs) {
            int64_t mb, nb;
            tile_coords(t, num_m, num_n, mb, nb);
            const int m0 = static_cast<int>(mb * 256 + rank * 128), n0 = static_cast<int>(nb * TILE_N + rank * 128);
            for (int64_t kt = 0; kt < k_tiles; ++kt, ++i) {
                if (i < SF_SLOTS) issue_next_scales();
                ok = mbar_wait_poll(empty_bar + 8 * s, ph ^ 1u, abort_flag, p.status, 1);
                if (!ok) break;
                if (i >= STAGES) issue_next_scales();
                const uint32_t stage = smem_base + s * STAGE_BYTES, bar = leader_full + 8 * s;
                // out-of-range parts of a box are zero-filled and still counted: fixed byte counts.
                // The leader announces the bytes of both CTAs; its barrier may see the peer's bytes
                // first, which only makes the pending count negative for a moment.
                if (leader) mbar_expect_tx(full_bar + 8 * s, 2 * STAGE_BYTES);
                tma_load_2d_pair(stage, &map_a, static_cast<int>(kt * BLOCK_K_BYTES), m0, bar);
                tma_load_2d_pair(stage + A_BYTES, &map_b, static_cast<int>(kt * BLOCK_K_BYTES), n0, bar);
                if (++s == STAGES) { s = 0; ph ^= 1u; }
            }
        }
        // the scales of the last iteration (when there were more than SF_SLOTS): their slot is free once the
        // operand stage that would come next is
        while (ok && requested < i) {
            ok = mbar_wait_poll(empty_bar + 8 * s, ph ^ 1u, abort_flag, p.status, 7);
            if (!ok) break;
            issue_next_scales();
            if (++s == STAGES) { s = 0; ph ^= 1u; }
        }
        if (!ok) {
            const unsigned long long t0 = global_timer_ns();
            while (global_timer_ns() - t0 < 200000ull) __nanosleep(1000);
        }
    } else if (warp == 1 && leader) {
        // ------------------------------------------------------------------ MMA issuer (leader only)
        const bool issue = elect_one();
        const uint32_t idesc = mma_idesc(TILE_N, 256);
        uint32_t s = 0, ph = 0, j = 0, jph = 0, tile_i = 0;
        bool ok = true;
        for (int64_t t = pair_id; t < num_tiles && ok; t += num_pairs, ++tile_i) {
            ok = mbar_wait_poll(acc_empty_bar, (tile_i & 1u) ^ 1u, abort_flag, p.status, 3);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
            for (int64_t kt = 0; kt < k_tiles; ++kt) {
                if (!dbg_no_load) {
                    ok = mbar_wait_poll(full_bar + 8 * s, ph, abort_flag, p.status, 2);
                    if (ok && !dbg_no_sf) ok = mbar_wait_poll(sf_ready_bar + 8 * j, jph, abort_flag, p.status, 5);
                }
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                tc_fence_after();
                const int64_t kb0 = kt * KB_PER_STAGE;
                const int nkb = static_cast<int>((k_blocks - kb0) < KB_PER_STAGE ? (k_blocks - kb0) : KB_PER_STAGE);
                const uint32_t stage = smem_base + s * STAGE_BYTES;
                const uint32_t sfa_tmem = tmem_base + SF_COL0 + j * SF_STAGE_COLS, sfb_tmem = sfa_tmem + 16;
                const uint32_t a_lo = desc_lo(stage, 16), b_lo = desc_lo(stage + A_BYTES, 16);
#pragma unroll
                for (int kb = 0; kb < KB_PER_STAGE; ++kb) {
                    if (kb < nkb && !dbg_no_mma && issue)
                        tc_mma_nvf4_pair_lo(tmem_base, a_lo + 2 * kb, b_lo + 2 * kb, idesc, sfa_tmem + 4 * kb,
                                            sfb_tmem + 8 * kb, (kt > 0 || kb > 0) ? 1u : 0u);
                }
                if (issue) tc_commit_pair(empty_bar + 8 * s);
                __syncwarp();
                if (++s == STAGES) { s = 0; ph ^= 1u; }
                if (++j == SF_SLOTS) { j = 0; jph ^= 1u; }
            }
            if (ok && issue) tc_commit_pair(acc_full_bar);
        }
    } else if (warp >= 2 && warp < 10) {
        // ------------------------------------------------------------------ epilogue (both CTAs)
        const int quad = warp & 3;                       // tensor-memory lanes 32*quad .. +31
        const int half = (warp - 2) >> 2;                // which 128 of the 256 columns
        constexpr int COLS = 128;
        const float alpha = __ldg(p.alpha);
        OUT *out = static_cast<OUT *>(p.d);
        const bool vec_ok = (reinterpret_cast<uintptr_t>(out) % 16 == 0) && ((p.ldd * sizeof(OUT)) % 16 == 0);
        const bool vec32_ok = FOS_GEMM_ST256 && (reinterpret_cast<uintptr_t>(out) % 32 == 0) && ((p.ldd * sizeof(OUT)) % 32 == 0);
        const uint32_t leader_acc_empty = map_to_cta(acc_empty_bar, 0);
        uint32_t tile_i = 0;
        bool ok = true;
        for (int64_t t = pair_id; t < num_tiles && ok; t += num_pairs, ++tile_i) {
            int64_t mb, nb;
            tile_coords(t, num_m, num_n, mb, nb);
            const int64_t row = mb * 256 + rank * 128 + quad * 32 + lane, n0 = nb * TILE_N + half * COLS;
            // in the peer this barrier is arrived on from the leader's SM: one lane polls for the warp
            if (lane == 0) ok = mbar_wait_poll(acc_full_bar, tile_i & 1u, abort_flag, p.status, 4);
            ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
            if (!ok) break;
            tc_fence_after();
            const uint32_t t_acc = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + half * COLS;
            const bool row_ok = row < p.m && !dbg_no_store;
            if constexpr (sizeof(OUT) == 2) {
                uint32_t pk[COLS / 2];
#pragma unroll
                for (int c = 0; c < COLS / 32; ++c) {
                    uint32_t v[32];
                    tc_load_32cols_sync(t_acc + 32 * c, v);
                    if (c + 1 == COLS / 32) {            // everything is in registers: release the accumulator
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive_cluster(leader_acc_empty);
                    }
#pragma unroll
                    for (int i = 0; i < 16; ++i)
                        pk[16 * c + i] = pack_pair<OUT>(alpha * __uint_as_float(v[2 * i]), alpha * __uint_as_float(v[2 * i + 1]));
                }
                const int64_t left = p.n - n0;
                if (row_ok && left > 0) {
                    OUT *dst = out + row * p.ldd + n0;
                    if (left >= COLS && vec32_ok) {
#pragma unroll
                        for (int i = 0; i < COLS / 16; ++i) stg_32_stream(reinterpret_cast<uint8_t *>(dst) + 32 * i, &pk[8 * i]);
                    } else if (left >= COLS && vec_ok) {
#pragma unroll
                        for (int i = 0; i < COLS / 8; ++i)
                            reinterpret_cast<uint4 *>(dst)[i] = make_uint4(pk[4 * i], pk[4 * i + 1], pk[4 * i + 2], pk[4 * i + 3]);
                    } else {
                        uint16_t *d16 = reinterpret_cast<uint16_t *>(dst);
#pragma unroll
                        for (int i = 0; i < COLS; ++i)
                            if (i < left) d16[i] = static_cast<uint16_t>(pk[i >> 1] >> ((i & 1) * 16));
                    }
                }
            } else {
#pragma unroll 1
                for (int c = 0; c < 4; c += 2) {
                    uint32_t v0[32], v1[32];
                    tc_load_64cols_sync(t_acc + 32 * c, v0, v1);
                    if (c + 2 >= 4) {
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive_cluster(leader_acc_empty);
                    }
                    const int64_t col = n0 + 32 * c;
                    const int64_t left0 = p.n - col, left1 = left0 - 32;
                    if (row_ok && left0 > 0)
                        store_chunk<OUT>(out + row * p.ldd + col, v0, alpha, left0 < 32 ? static_cast<int>(left0) : 32, vec_ok);
                    if (row_ok && left1 > 0)
                        store_chunk<OUT>(out + row * p.ldd + col + 32, v1, alpha, left1 < 32 ? static_cast<int>(left1) : 32, vec_ok);
                }
            }
        }
    } else if (warp >= 10 && warp < 10 + CP_WARPS && leader && !dbg_no_load && !dbg_no_sf) {
        // ------------------------------------------------------------------ scale copies (leader, for both CTAs)
        // tcgen05.cp with cta_group::2 copies, in each CTA, from that CTA's shared memory into its
        // tensor memory: one thread of the pair moves the scales of both, and no warp of the peer
        // has to report back. Two warps take the stages in turn (one alone cannot issue twelve copies
        // per stage as fast as the MMAs consume them), each with a landing barrier of its own per slot.
        const bool issue = elect_one();
        const uint32_t me = static_cast<uint32_t>(warp - 10);
        uint32_t j = 0, turn = 0, seen = 0;          // bit j of `seen`: parity of this warp's next phase of slot j
        bool ok = true;
        for (int64_t t = pair_id; t < num_tiles && ok; t += num_pairs) {
            for (int64_t kt = 0; kt < k_tiles; ++kt) {
                const bool mine = turn == me;
                if (++turn == CP_WARPS) turn = 0;
                if (!mine) {
                    if (++j == SF_SLOTS) j = 0;
                    continue;
                }
                const uint32_t jph = (seen >> j) & 1u;
                seen ^= 1u << j;
                ok = mbar_wait_poll(sf_full_bar + 8 * (me * SF_SLOTS + j), jph, abort_flag, p.status, 6);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                tc_fence_after();
                const uint32_t src = sf_base + j * SF_SLOT_BYTES, dst = tmem_base + SF_COL0 + j * SF_STAGE_COLS;
                const uint32_t src_lo = desc_lo(src);
#pragma unroll
                for (int kb = 0; kb < KB_PER_STAGE; ++kb) {
                    if (!issue) break;
                    tc_copy_sf_pair_lo(dst + 4 * kb, src_lo + ((kb * SF_TILE_BYTES) >> 4));
#pragma unroll
                    for (int g = 0; g < 2; ++g)
                        tc_copy_sf_pair_lo(dst + 16 + 8 * kb + 4 * g,
                                           src_lo + ((SFA_BYTES + (g * KB_PER_STAGE + kb) * SF_TILE_BYTES) >> 4));
                }
                if (issue) tc_commit_pair_local(sf_ready_bar + 8 * j);
                __syncwarp();
                if (++j == SF_SLOTS) j = 0;
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    cluster_sync_all();            // nobody leaves while the peer may still touch this CTA's memory
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

}  // namespace pair

// ---------------------------------------------------------------------------- host side

// Scale tiles as a 3-D tensor [row groups][tiles along K][512 bytes]; box = `groups` x the tiles of one stage
// (four; two for MXFP4, whose tiles span two K-blocks).
int make_scale_map(CUtensorMap *map, const uint8_t *sf, int64_t row_groups, int64_t k_blocks, int groups,
                   int tiles_per_stage = KB_PER_STAGE) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return FOS_ERR_CUDA;
    cuuint64_t dims[3] = {128, static_cast<cuuint64_t>(k_blocks), static_cast<cuuint64_t>(row_groups)};
    cuuint64_t strides[2] = {512, static_cast<cuuint64_t>(k_blocks) * 512};
    cuuint32_t box[3] = {128, static_cast<cuuint32_t>(tiles_per_stage), static_cast<cuuint32_t>(groups)};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT32, 3, const_cast<uint8_t *>(sf), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? FOS_OK : FOS_ERR_CUDA;
}

template <typename OUT>
int launch_pair(const CUtensorMap &ma, const CUtensorMap &mb, const CUtensorMap &msa, const CUtensorMap &msb,
                const GemmParams &p, cudaStream_t stream) {
    auto kernel = pair::gemm_nvfp4_pair_kernel<OUT>;
    static int max_clusters[64] = {};   // per device: how many CTA pairs can be resident at once
    static std::mutex mu;
    int dev = 0;
    FOS_CUDA_TRY(cudaGetDevice(&dev));
    const int slot = (dev >= 0 && dev < 64) ? dev : 0;
    std::lock_guard<std::mutex> lock(mu);
    cudaLaunchConfig_t cfg = {};
    cfg.blockDim = dim3(pair::THREADS);
    cfg.dynamicSmemBytes = pair::SMEM_BYTES;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (max_clusters[slot] == 0) {
        FOS_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, pair::SMEM_BYTES));
        int sms = 0, n = 0;
        FOS_CUDA_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
        cfg.gridDim = dim3(static_cast<unsigned>(sms & ~1));
        FOS_CUDA_TRY(cudaOccupancyMaxActiveClusters(&n, kernel, &cfg));
        max_clusters[slot] = n > 0 ? n : 1;
    }
    const int64_t tiles = (p.m_p / 256) * (p.n_p / 256);
    const int64_t pairs = tiles < max_clusters[slot] ? tiles : max_clusters[slot];
    cfg.gridDim = dim3(static_cast<unsigned>(2 * pairs));
    FOS_CUDA_TRY(cudaLaunchKernelEx(&cfg, kernel, ma, mb, msa, msb, p));
    return FOS_OK;
}

template <int BLOCK_N, typename OUT, bool FUSED_A = false, bool GROUPED = false>
int launch(const CUtensorMap &ma, const CUtensorMap &mb, const CUtensorMap &msa, const CUtensorMap &msb,
           const GemmParams &p, int sms, cudaStream_t stream) {
    using C = Cfg<BLOCK_N>;
    auto kernel = gemm_nvfp4_kernel<BLOCK_N, OUT, FUSED_A, GROUPED>;
    static OncePerDevice configured;   // per instantiation
    int dev = 0;
    FOS_CUDA_TRY(cudaGetDevice(&dev));
    FOS_CUDA_TRY(configured.run(dev, [&] {
        return cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES);
    }));
    const int64_t tiles = (p.m_p / BLOCK_M) * ((p.n_p + BLOCK_N - 1) / BLOCK_N);
    const unsigned grid = static_cast<unsigned>(tiles < sms ? tiles : sms);
    kernel<<<grid, NUM_THREADS, C::SMEM_BYTES, stream>>>(ma, mb, msa, msb, p);
    FOS_CUDA_TRY(cudaGetLastError());
    return FOS_OK;
}

template <int BLOCK_N, bool FUSED_A = false, bool GROUPED = false>
int launch_out(const CUtensorMap &ma, const CUtensorMap &mb, const CUtensorMap &msa, const CUtensorMap &msb,
               const GemmParams &p, int sms, cudaStream_t stream) {
    if (p.out_dtype == FOS_BF16) return launch<BLOCK_N, __nv_bfloat16, FUSED_A, GROUPED>(ma, mb, msa, msb, p, sms, stream);
    if (p.out_dtype == FOS_FP16) return launch<BLOCK_N, __half, FUSED_A, GROUPED>(ma, mb, msa, msb, p, sms, stream);
    return launch<BLOCK_N, float, FUSED_A, GROUPED>(ma, mb, msa, msb, p, sms, stream);
}

#ifdef FOS_GEMM_DEBUG
int g_gemm_debug = 0;     // timing experiments of a debug build (fos_gemm_debug_set)
#endif

}  // namespace
}  // namespace fos

#ifdef FOS_GEMM_DEBUG
// Debug builds only (not declared in the public header): bit 0 skips the scale copies, bit 1 the operand
// loads, bit 2 the output stores, bit 4 the MMAs. The GEMM's result is wrong with any of them set.
extern "C" int fos_gemm_debug_set(int bits) {
    fos::g_gemm_debug = bits;
    return FOS_OK;
}
#endif

static int gemm_fp4_entry(const uint8_t *a_codes, const uint8_t *a_sf, const uint8_t *b_codes,
                          const uint8_t *b_sf, const float *alpha, void *d, int out_dtype, int64_t m_p,
                          int64_t n_p, int64_t k_p, int64_t m, int64_t n, int64_t ldd, const fos_gemm_opts *opts,
                          int32_t *status, void *stream_, int mx, void *const *d_peers = nullptr, int world = 0,
                          int rank = 0) {
    using namespace fos;
    const int variant = opts ? opts->variant : 0, max_ctas = opts ? opts->max_ctas : 0;
    if ((variant != 0 && variant != 128 && variant != 256 && variant != 2) || max_ctas < 0) return FOS_ERR_INVALID_ARGUMENT;
    if (d_peers) {
        if (world < 2 || world > 8 || rank < 0 || rank >= world) return FOS_ERR_INVALID_ARGUMENT;
        if (m_p % (128 * static_cast<int64_t>(world)) != 0) return FOS_ERR_UNSUPPORTED;   // slabs of whole row blocks
        for (int i = 0; i < world; ++i) {
            if (!d_peers[i]) return FOS_ERR_INVALID_ARGUMENT;
            if (reinterpret_cast<uintptr_t>(d_peers[i]) % 32 != 0) return FOS_ERR_MISALIGNED;
        }
        d = d_peers[rank];
    }
    if (!a_codes || !a_sf || !b_codes || !b_sf || !alpha || !d) return FOS_ERR_INVALID_ARGUMENT;
    if (m_p <= 0 || n_p <= 0 || k_p < 64 || m_p % 128 || n_p % 128 || k_p % (mx ? 128 : 64)) return FOS_ERR_INVALID_ARGUMENT;
    if (m <= 0 || n <= 0 || m > m_p || n > n_p || ldd < n) return FOS_ERR_INVALID_ARGUMENT;
    if (out_dtype != FOS_BF16 && out_dtype != FOS_FP16 && out_dtype != FOS_FP32) return FOS_ERR_INVALID_ARGUMENT;
    if (reinterpret_cast<uintptr_t>(a_codes) % 16 || reinterpret_cast<uintptr_t>(b_codes) % 16 ||
        reinterpret_cast<uintptr_t>(a_sf) % 16 || reinterpret_cast<uintptr_t>(b_sf) % 16)
        return FOS_ERR_MISALIGNED;
    if (m_p > INT32_MAX || n_p > INT32_MAX || k_p / 2 > INT32_MAX) return FOS_ERR_TOO_LARGE;
    int st = check_device();
    if (st != FOS_OK) return st;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);

    int dev = 0, sms = 0;
    FOS_CUDA_TRY(cudaGetDevice(&dev));
    FOS_CUDA_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    if (max_ctas > 0 && max_ctas < sms) sms = max_ctas;   // leave SMs to concurrent kernels

#ifdef FOS_GEMM_DEBUG
    const int debug_bits = g_gemm_debug;
#else
    const int debug_bits = 0;
#endif
    GemmParams p{a_sf, b_sf, alpha, d, status, m_p, n_p, k_p, m, n, ldd, out_dtype, debug_bits, mx, nullptr, 0, nullptr, 0, 0,
                 0, 0, 0, {}};
    if (d_peers) {
        p.scatter_world = world;
        p.scatter_rank = rank;
        p.slab_rows = m_p / world;
        for (int i = 0; i < world; ++i) p.d_peer[i] = d_peers[i];
    }
    const int64_t sf_k_tiles = mx ? k_p / 128 : k_p / 64;     // 512-byte scale tiles along K
    if (status) {
        FOS_CUDA_TRY(cudaMemsetAsync(status, 0, sizeof(int32_t), stream));
    } else {
        // no word of the caller's: a wait that gives up leaves its site in the library's sticky word
        FOS_CUDA_TRY(wait_failures_ptr(&p.status));
    }
    CUtensorMap map_a, map_b;

    // The CTA-pair kernel is correct but still measures slower than the single-CTA kernel on B200
    // (its hand-overs between the two SMs lengthen the load round trip), so it only runs when
    // asked for.
    const bool pair_fits = m_p % 256 == 0 && n_p % 256 == 0;
    const bool use_pair = pair_fits && variant == 2 && !mx && !d_peers;
    if (use_pair) {
        CUtensorMap map_sfa, map_sfb;
        if ((st = make_operand_map(&map_a, a_codes, m_p, k_p / 2, 128)) != FOS_OK) return st;
        if ((st = make_operand_map(&map_b, b_codes, n_p, k_p / 2, 128)) != FOS_OK) return st;
        if ((st = make_scale_map(&map_sfa, a_sf, m_p / 128, k_p / 64, 1)) != FOS_OK) return st;
        if ((st = make_scale_map(&map_sfb, b_sf, n_p / 128, k_p / 64, 2)) != FOS_OK) return st;
        if (out_dtype == FOS_BF16) return launch_pair<__nv_bfloat16>(map_a, map_b, map_sfa, map_sfb, p, stream);
        if (out_dtype == FOS_FP16) return launch_pair<__half>(map_a, map_b, map_sfa, map_sfb, p, stream);
        return launch_pair<float>(map_a, map_b, map_sfa, map_sfb, p, stream);
    }

    // single-CTA kernel: 128 x 256 tiles unless they would fill less than half of the SMs (a 128 x 128
    // tile takes nine tenths of the time of a 128 x 256 one, so the narrow kernel only pays when it
    // doubles the number of busy SMs)
    const int64_t tiles_256 = (m_p / BLOCK_M) * ((n_p + 255) / 256);
    bool wide = n_p >= 256 && tiles_256 * 2 > sms;
    if (variant == 128) wide = false;
    if (variant == 256) wide = true;
    if ((st = make_operand_map(&map_a, a_codes, m_p, k_p / 2, BLOCK_M)) != FOS_OK) return st;
    if ((st = make_operand_map(&map_b, b_codes, n_p, k_p / 2, wide ? 256 : 128)) != FOS_OK) return st;
    CUtensorMap map_sfa, map_sfb;
    const int sf_box_k = mx ? KB_PER_STAGE / 2 : KB_PER_STAGE;
    if ((st = make_scale_map(&map_sfa, a_sf, m_p / 128, sf_k_tiles, 1, sf_box_k)) != FOS_OK) return st;
    if ((st = make_scale_map(&map_sfb, b_sf, n_p / 128, sf_k_tiles, wide ? 2 : 1, sf_box_k)) != FOS_OK) return st;
    return wide ? launch_out<256>(map_a, map_b, map_sfa, map_sfb, p, sms, stream)
                : launch_out<128>(map_a, map_b, map_sfa, map_sfb, p, sms, stream);
}

cudaError_t fos::gemm_wait_failures(int32_t *host_value) { return fos::read_wait_failures(host_value); }
cudaError_t fos::gemm_wait_roles(uint32_t *host_value) { return fos::read_wait_roles(host_value); }

extern "C" int fos_gemm_nvfp4(const uint8_t *a_codes, const uint8_t *a_sf, const uint8_t *b_codes,
                              const uint8_t *b_sf, const float *alpha, void *d, int out_dtype, int64_t m_p,
                              int64_t n_p, int64_t k_p, int64_t m, int64_t n, int64_t ldd, int32_t *status,
                              void *stream) {
    return gemm_fp4_entry(a_codes, a_sf, b_codes, b_sf, alpha, d, out_dtype, m_p, n_p, k_p, m, n, ldd, nullptr, status, stream, 0);
}

extern "C" int fos_gemm_nvfp4_ex(const uint8_t *a_codes, const uint8_t *a_sf, const uint8_t *b_codes,
                                 const uint8_t *b_sf, const float *alpha, void *d, int out_dtype, int64_t m_p,
                                 int64_t n_p, int64_t k_p, int64_t m, int64_t n, int64_t ldd, const fos_gemm_opts *opts,
                                 int32_t *status, void *stream) {
    return gemm_fp4_entry(a_codes, a_sf, b_codes, b_sf, alpha, d, out_dtype, m_p, n_p, k_p, m, n, ldd, opts, status, stream, 0);
}

extern "C" int fos_gemm_nvfp4_fused_a(const void *x, int x_dtype, int64_t x_ld, const float *x_amax, int x_rule,
                                      const uint8_t *b_codes, const uint8_t *b_sf, const float *alpha, void *d,
                                      int out_dtype, int64_t m, int64_t n_p, int64_t k, int64_t n, int64_t ldd,
                                      int32_t *status, void *stream_) {
    using namespace fos;
    if (!x || !x_amax || !b_codes || !b_sf || !alpha || !d) return FOS_ERR_INVALID_ARGUMENT;
    if (x_dtype != FOS_BF16 && x_dtype != FOS_FP16) return FOS_ERR_INVALID_ARGUMENT;
    if (x_rule != FOS_RULE_STATIC_6 && x_rule != FOS_RULE_STATIC_4) return FOS_ERR_UNSUPPORTED;   // 4/6 stays un-fused
    if (m <= 0 || n_p <= 0 || k < 64 || n_p % 128 || n <= 0 || n > n_p || ldd < n || x_ld < k) return FOS_ERR_INVALID_ARGUMENT;
    if (k % 64) return FOS_ERR_UNSUPPORTED;          // whole scale tiles only: pad K, or quantize first
    if (out_dtype != FOS_BF16 && out_dtype != FOS_FP16 && out_dtype != FOS_FP32) return FOS_ERR_INVALID_ARGUMENT;
    if (reinterpret_cast<uintptr_t>(x) % 32 || (x_ld * 2) % 32) return FOS_ERR_MISALIGNED;   // 32-byte loads of x
    if (reinterpret_cast<uintptr_t>(b_codes) % 16 || reinterpret_cast<uintptr_t>(b_sf) % 16) return FOS_ERR_MISALIGNED;
    const int64_t m_p = round_up64(m, 128);
    if (m_p > INT32_MAX || n_p > INT32_MAX || k / 2 > INT32_MAX) return FOS_ERR_TOO_LARGE;
    int st = check_device();
    if (st != FOS_OK) return st;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    int dev = 0, sms = 0;
    FOS_CUDA_TRY(cudaGetDevice(&dev));
    FOS_CUDA_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    GemmParams p{nullptr, b_sf, alpha, d, status, m_p, n_p, k, m, n, ldd, out_dtype, 0, 0, x, x_ld, x_amax, x_rule,
                 x_dtype == FOS_FP16 ? 1 : 0, 0, 0, 0, {}};
    if (status) {
        FOS_CUDA_TRY(cudaMemsetAsync(status, 0, sizeof(int32_t), stream));
    } else {
        FOS_CUDA_TRY(wait_failures_ptr(&p.status));
    }
    const int64_t tiles_256 = (m_p / BLOCK_M) * ((n_p + 255) / 256);
    const bool wide = n_p >= 256 && tiles_256 * 2 > sms;
    CUtensorMap map_b, map_sfb;
    if ((st = make_operand_map(&map_b, b_codes, n_p, k / 2, wide ? 256 : 128)) != FOS_OK) return st;
    if ((st = make_scale_map(&map_sfb, b_sf, n_p / 128, k / 64, wide ? 2 : 1, KB_PER_STAGE)) != FOS_OK) return st;
    // (the kernel never touches the A maps in this mode; B's stand in for them)
    return wide ? launch_out<256, true>(map_b, map_b, map_sfb, map_sfb, p, sms, stream)
                : launch_out<128, true>(map_b, map_b, map_sfb, map_sfb, p, sms, stream);
}

extern "C" int fos_gemm_nvfp4_grouped(const uint8_t *a_codes, const uint8_t *a_sf, const uint8_t *b_codes,
                                      const uint8_t *b_sf, const float *alpha, void *d, int out_dtype,
                                      const int32_t *group_start, const int32_t *group_rows, int num_groups,
                                      int64_t rows_capacity, int64_t n_p, int64_t k_p, int64_t n, int64_t ldd,
                                      const fos_gemm_opts *opts, int32_t *status, void *stream_) {
    using namespace fos;
    const int variant = opts ? opts->variant : 0, max_ctas = opts ? opts->max_ctas : 0;
    if ((variant != 0 && variant != 128 && variant != 256) || max_ctas < 0) return FOS_ERR_INVALID_ARGUMENT;
    if (!a_codes || !a_sf || !b_codes || !b_sf || !alpha || !d || !group_start || !group_rows) return FOS_ERR_INVALID_ARGUMENT;
    if (num_groups <= 0 || num_groups > MAX_GROUPS) return FOS_ERR_INVALID_ARGUMENT;
    if (rows_capacity <= 0 || rows_capacity % 128 || n_p <= 0 || n_p % 128 || k_p < 64 || k_p % 64) return FOS_ERR_INVALID_ARGUMENT;
    if (n <= 0 || n > n_p || ldd < n) return FOS_ERR_INVALID_ARGUMENT;
    if (out_dtype != FOS_BF16 && out_dtype != FOS_FP16 && out_dtype != FOS_FP32) return FOS_ERR_INVALID_ARGUMENT;
    if (reinterpret_cast<uintptr_t>(a_codes) % 16 || reinterpret_cast<uintptr_t>(b_codes) % 16 ||
        reinterpret_cast<uintptr_t>(a_sf) % 16 || reinterpret_cast<uintptr_t>(b_sf) % 16)
        return FOS_ERR_MISALIGNED;
    const int64_t b_rows = n_p * num_groups;
    if (rows_capacity > INT32_MAX || b_rows > INT32_MAX || k_p / 2 > INT32_MAX) return FOS_ERR_TOO_LARGE;
    int st = check_device();
    if (st != FOS_OK) return st;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    int dev = 0, sms = 0;
    FOS_CUDA_TRY(cudaGetDevice(&dev));
    FOS_CUDA_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    if (max_ctas > 0 && max_ctas < sms) sms = max_ctas;
    GemmParams p{a_sf, b_sf, alpha, d, status, rows_capacity, n_p, k_p, rows_capacity, n, ldd, out_dtype, 0, 0, nullptr, 0,
                 nullptr, 0, 0, 0, 0, 0, {}};
    p.group_start = group_start;
    p.group_rows = group_rows;
    p.num_groups = num_groups;
    if (status) {
        FOS_CUDA_TRY(cudaMemsetAsync(status, 0, sizeof(int32_t), stream));
    } else {
        FOS_CUDA_TRY(wait_failures_ptr(&p.status));
    }
    // how many row blocks are in use is known on the device only: the grid is sized for the buffers, and
    // CTAs that find no tile leave at once
    const int64_t tiles_256 = (rows_capacity / BLOCK_M) * ((n_p + 255) / 256);
    bool wide = n_p >= 256 && tiles_256 * 2 > sms;
    if (variant == 128) wide = false;
    if (variant == 256 && n_p >= 256) wide = true;
    CUtensorMap map_a, map_b, map_sfa, map_sfb;
    if ((st = make_operand_map(&map_a, a_codes, rows_capacity, k_p / 2, BLOCK_M)) != FOS_OK) return st;
    if ((st = make_operand_map(&map_b, b_codes, b_rows, k_p / 2, wide ? 256 : 128)) != FOS_OK) return st;
    if ((st = make_scale_map(&map_sfa, a_sf, rows_capacity / 128, k_p / 64, 1, KB_PER_STAGE)) != FOS_OK) return st;
    if ((st = make_scale_map(&map_sfb, b_sf, b_rows / 128, k_p / 64, wide ? 2 : 1, KB_PER_STAGE)) != FOS_OK) return st;
    return wide ? launch_out<256, false, true>(map_a, map_b, map_sfa, map_sfb, p, sms, stream)
                : launch_out<128, false, true>(map_a, map_b, map_sfa, map_sfb, p, sms, stream);
}

extern "C" int fos_gemm_mxfp4(const uint8_t *a_codes, const uint8_t *a_sf, const uint8_t *b_codes,
                              const uint8_t *b_sf, const float *alpha, void *d, int out_dtype, int64_t m_p,
                              int64_t n_p, int64_t k_p, int64_t m, int64_t n, int64_t ldd, int32_t *status,
                              void *stream) {
    return gemm_fp4_entry(a_codes, a_sf, b_codes, b_sf, alpha, d, out_dtype, m_p, n_p, k_p, m, n, ldd, nullptr, status, stream, 1);
}

extern "C" int fos_gemm_mxfp4_ex(const uint8_t *a_codes, const uint8_t *a_sf, const uint8_t *b_codes,
                                 const uint8_t *b_sf, const float *alpha, void *d, int out_dtype, int64_t m_p,
                                 int64_t n_p, int64_t k_p, int64_t m, int64_t n, int64_t ldd, const fos_gemm_opts *opts,
                                 int32_t *status, void *stream) {
    return gemm_fp4_entry(a_codes, a_sf, b_codes, b_sf, alpha, d, out_dtype, m_p, n_p, k_p, m, n, ldd, opts, status, stream, 1);
}

extern "C" int fos_gemm_nvfp4_scatter(const uint8_t *a_codes, const uint8_t *a_sf, const uint8_t *b_codes,
                                      const uint8_t *b_sf, const float *alpha, void *const *d_peers, int world, int rank,
                                      int out_dtype, int64_t m_p, int64_t n_p, int64_t k_p, int64_t m, int64_t n,
                                      int64_t ldd, int32_t *status, void *stream) {
    if (!d_peers) return FOS_ERR_INVALID_ARGUMENT;
    if (out_dtype != FOS_BF16 && out_dtype != FOS_FP16) return FOS_ERR_UNSUPPORTED;
    return gemm_fp4_entry(a_codes, a_sf, b_codes, b_sf, alpha, nullptr, out_dtype, m_p, n_p, k_p, m, n, ldd, nullptr, status, stream, 0,
                          d_peers, world, rank);
}
