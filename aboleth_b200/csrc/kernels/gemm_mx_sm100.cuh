// Block-scaled e4m3 GEMM main loop: tcgen05.mma.kind::mxf8f6f4.block_scale with ue8m0 scale
// factors in tensor memory.
//
//   C[M, N] = sum over K blocks of 128:  (A_blk * sa[m, blk]) * (B_blk * sb[n, blk])^T
//
// A and B are e4m3, K-major.  The tensor core multiplies every 32-element K segment of a row by a
// power-of-two scale (ue8m0: the exponent byte of an fp32) before it accumulates, so operands
// that carry one scale per 1 x 128 (activations) or 128 x 128 (weights) block are multiplied at
// the fp8 rate with no expansion pass: the one scale of a 128-K block is given to its four
// 32-K segments.
//
// Scale factors reach the tensor core through tensor memory.  The host-side packer
// (pack_scales kernels in gemm_kernels.cu) lays them out in 512-byte atoms, one per (128 rows,
// 128 K): byte (r % 32) * 16 + (r / 32) * 4 + s holds the scale of row r and K segment s.  That
// is the order `tcgen05.cp.32x128b.warpx4` wants: it copies 32 rows x 16 bytes from shared memory
// into 32 lanes x 4 columns of tensor memory and repeats them over the four lane quarters; the
// MMA then picks byte s of a column through the scale-factor id in its instruction descriptor.
// Per K block the producer brings in the A tile and the B tile by TMA (16 + 32 KiB, or 32 + 24 KiB
// for the wider tile) and one A atom per 128-row block plus two B atoms (512 bytes each) by untiled
// bulk copies on the same mbarrier; nothing is multicast.  B's atoms are stored per 64-column
// granule (atom g = columns [64 g, 64 g + 128)), so a tile that starts at any multiple of 64
// columns finds its two atoms at g and g + 2.
//
// Two tile shapes.  128 x 256: one accumulator of 256 columns plus 12 columns of scale factors.
// 256 x 192: two 128-row accumulators of 192 columns that share each B tile (a fifth fewer
// shared-memory bytes per FLOP, which is what bounds this loop) plus 16 columns of scale factors.
// Either way tensor memory has no room for a second accumulator buffer, so the epilogue of a tile
// is not overlapped with the next tile's main loop.
//
// Same roles, same bounded waits and the same policy interface as gemm_sm100.cuh.
#pragma once

#include "gemm_sm100.cuh"

namespace ab::gemm::mx {

constexpr int kBlockK = 128;                    // e4m3 elements (= bytes) of K per stage
constexpr int kStagesMx = 3;
constexpr unsigned kAtomBytes = 512;            // scale factors of 128 rows x 128 K

// HALVES row blocks of 128 rows per tile; the tile is 256 columns wide with one, 192 with two.
template <int HALVES>
struct MxGeometry {
    static constexpr int kRows = BM * HALVES;
    static constexpr int kCols = HALVES == 1 ? 256 : 192;
    static constexpr unsigned kBytesA = kRows * kBlockK;
    static constexpr unsigned kBytesB = kCols * kBlockK;
    static constexpr unsigned kOffSfa = kBytesA + kBytesB;          // HALVES atoms
    static constexpr unsigned kOffSfb = kOffSfa + HALVES * kAtomBytes;  // two atoms (256 columns' worth)
    static constexpr unsigned kStageTx = kBytesA + kBytesB + (HALVES + 2) * kAtomBytes;
    static constexpr unsigned kStageStride = (kStageTx + 1023) / 1024 * 1024;  // keeps tiles swizzle-aligned
    static constexpr unsigned kSmemBytes = kStagesMx * kStageStride + kEpilogueStageBytes + 1024;
    // tensor-memory columns: accumulators first, then A's scale factors (4 per row block), then B's (8)
    static constexpr unsigned kSfaCol = HALVES * kCols, kSfbCol = kSfaCol + 4 * HALVES;
};

// Instruction descriptor of kind::mxf8f6f4.block_scale: e4m3 A and B (format 0), K-major, ue8m0
// scales, N >> 3 at bit 17, M >> 4 at bit 24; `sf` (0..3) selects the byte of the scale columns
// that belongs to this MMA's 32-element K segment, for A (bits 29-30) and for B (bits 4-5).
__host__ __device__ constexpr std::uint32_t idesc_mx(int m, int n, unsigned sf) {
    return (sf << 4) | (static_cast<std::uint32_t>(n >> 3) << 17) | (1u << 23) |
           (static_cast<std::uint32_t>(m >> 4) << 24) | (sf << 29);
}

// Shared-memory descriptor of one scale-factor atom: no swizzle, 8-row x 16-byte core matrices
// 128 bytes apart (the atom is 32 contiguous rows of 16 bytes).
__device__ __forceinline__ std::uint64_t sf_desc(std::uint32_t smem_addr) {
    return static_cast<std::uint64_t>((smem_addr & 0x3ffffu) >> 4) |
           (static_cast<std::uint64_t>(128 >> 4) << 32) | (1ull << 46);
}

__device__ __forceinline__ void sf_copy(std::uint32_t tmem_addr, std::uint64_t desc) {
    asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(tmem_addr), "l"(desc) : "memory");
}

__device__ __forceinline__ void umma_mx(std::uint32_t d_tmem, std::uint64_t a_desc, std::uint64_t b_desc,
                                        std::uint32_t idesc, std::uint32_t sfa_tmem, std::uint32_t sfb_tmem,
                                        std::uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem)
        : "memory");
}

// Where the packed scale factors of a problem live.  A: atoms [row block][K block], one row block
// more than the rows need.  B: atoms [K block][granule]; atom g covers columns
// [64 g, 64 g + 128), so a tile that starts at any multiple of 64 columns reads atoms g and g + 2.
struct ScaleFactors {
    const std::uint8_t *a;
    const std::uint8_t *b;
    int k_blocks;     // K / 128
    int b_blocks;     // granules per K block
    const std::uint8_t *a_alt = nullptr;  // atoms of the second A operand (tiles with a_sel = 1)
};

// Row blocks of A's atoms and 64-column granules of B's.  One row block more than the rows need: a
// 256-row tile may start on the last 128-row block (grouped problems) and still reads two atoms.
__host__ __device__ inline long long mx_row_blocks(int m) { return static_cast<long long>((m + 127) / 128) + 1; }
inline int mx_granules(int n) { return (n + 63) / 64 + 3; }

template <int HALVES, typename Policy>
__device__ __forceinline__ void gemm_mx_mainloop(Policy &policy, const CUtensorMap *map_a,
                                                 const CUtensorMap *map_b, const ScaleFactors sf,
                                                 unsigned long long *status,
                                                 const CUtensorMap *map_a_alt = nullptr) {
    using G = MxGeometry<HALVES>;
    constexpr unsigned kBytesA = G::kBytesA, kOffSfa = G::kOffSfa, kOffSfb = G::kOffSfb;
    constexpr unsigned kStageStride = G::kStageStride, kStageTx = G::kStageTx;
    constexpr unsigned kSfaCol = G::kSfaCol, kSfbCol = G::kSfbCol;
    extern __shared__ std::uint8_t smem_raw[];
    __shared__ SharedState st;
    std::uint8_t *tiles = reinterpret_cast<std::uint8_t *>(
        (reinterpret_cast<std::uintptr_t>(smem_raw) + 1023) & ~static_cast<std::uintptr_t>(1023));
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStagesMx; ++s) {
            mbar_init(&st.full[s], 1);
            mbar_init(&st.empty[s], 1);
        }
        mbar_init(&st.tmem_full[0], 1);
        mbar_init(&st.tmem_empty[0], kEpilogueWarps);
        st.abort = 0;
        mbar_fence_init();
        prefetch_tensormap(map_a);
        prefetch_tensormap(map_b);
        if (map_a_alt != nullptr)
            prefetch_tensormap(map_a_alt);
    }
    if (warp == 1)
        tmem_alloc(&st.tmem_base, kTmemCols);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const std::uint32_t tmem_base = st.tmem_base;

    if (warp == 0) {
        // ---------------- producer: TMA tiles and scale-factor atoms ----------------
        if (lane == 0) {
            int stage = 0;
            unsigned phase = 0;
            Tile t;
            for (int it = 0; !st.abort && policy.next(it, t); ++it) {
                if (!policy.ready(t)) {
                    st.abort = 1;
                    set_status(status, aboleth::Status::Timeout, 0x3000 + t.tag);
                    break;
                }
                const bool alt = t.a_sel != 0 && map_a_alt != nullptr;
                const CUtensorMap *tile_map_a = alt ? map_a_alt : map_a;
                const std::uint8_t *sfa = (alt ? sf.a_alt : sf.a) +
                                          static_cast<std::size_t>(t.a_row / BM) * sf.k_blocks * kAtomBytes;
                const std::uint8_t *sfb = sf.b + static_cast<std::size_t>(t.b_row / 64) * kAtomBytes;
                for (int kb = 0; kb < t.k_blocks; ++kb) {
                    if (!mbar_wait(&st.empty[stage], phase ^ 1) || st.abort) {
                        st.abort = 1;
                        set_status(status, aboleth::Status::Timeout, 0x3100 + stage);
                        break;
                    }
                    std::uint8_t *sa = tiles + stage * kStageStride;
                    mbar_expect_tx(&st.full[stage], kStageTx);
                    tma_load_2d(sa, tile_map_a, kb * kBlockK, t.a_row, &st.full[stage]);
                    tma_load_2d(sa + kBytesA, map_b, kb * kBlockK, t.b_row, &st.full[stage]);
#pragma unroll
                    for (int h = 0; h < HALVES; ++h)  // row block h of the tile: its atoms are k_blocks apart
                        bulk_load(sa + kOffSfa + h * kAtomBytes,
                                  sfa + (static_cast<std::size_t>(h) * sf.k_blocks + kb) * kAtomBytes, kAtomBytes,
                                  &st.full[stage]);
#pragma unroll
                    for (int half = 0; half < 2; ++half)  // columns [0, 128) and [128, 256) of the tile
                        bulk_load(sa + kOffSfb + half * kAtomBytes,
                                  sfb + (static_cast<std::size_t>(kb) * sf.b_blocks + 2 * half) * kAtomBytes,
                                  kAtomBytes, &st.full[stage]);
                    if (++stage == kStagesMx) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            int stage = 0;
            unsigned phase = 0;
            Tile t;
            for (int it = 0; !st.abort && policy.next(it, t); ++it) {
                // The accumulator must have been drained by the epilogue of the tile before.
                if (!mbar_wait(&st.tmem_empty[0], (it & 1) ^ 1)) {
                    st.abort = 1;
                    set_status(status, aboleth::Status::Timeout, 0x3200);
                    break;
                }
                tc_fence_after();
                for (int kb = 0; kb < t.k_blocks && !st.abort; ++kb) {
                    if (!mbar_wait(&st.full[stage], phase)) {
                        st.abort = 1;
                        set_status(status, aboleth::Status::Timeout, 0x3300 + stage);
                        break;
                    }
                    tc_fence_after();
                    const std::uint32_t sa = smem_u32(tiles + stage * kStageStride);
                    // This K block's scale factors: shared memory -> tensor memory.  Copies and MMAs
                    // issued by one thread run in order, so the MMAs below read these scales and the
                    // copies of the next block wait for them.
#pragma unroll
                    for (int h = 0; h < HALVES; ++h)
                        sf_copy(tmem_base + kSfaCol + 4 * h, sf_desc(sa + kOffSfa + h * kAtomBytes));
                    sf_copy(tmem_base + kSfbCol, sf_desc(sa + kOffSfb));
                    sf_copy(tmem_base + kSfbCol + 4, sf_desc(sa + kOffSfb + kAtomBytes));
                    const std::uint64_t db = smem_desc_sw128(sa + kBytesA);
#pragma unroll
                    for (int h = 0; h < HALVES; ++h) {
                        const std::uint64_t da = smem_desc_sw128(sa + h * (BM * kBlockK));
#pragma unroll
                        for (unsigned k = 0; k < 4; ++k) {
                            // 32 e4m3 = 32 bytes further along K inside the swizzle atom.
                            umma_mx(tmem_base + h * G::kCols, da + (k * 32 >> 4), db + (k * 32 >> 4),
                                    idesc_mx(BM, G::kCols, k), tmem_base + kSfaCol + 4 * h, tmem_base + kSfbCol,
                                    (kb | static_cast<int>(k)) != 0);
                        }
                    }
                    umma_commit(&st.empty[stage]);  // stage reusable once MMAs and copies have read it
                    if (++stage == kStagesMx) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
                umma_commit(&st.tmem_full[0]);  // accumulator complete
            }
        }
    } else {
        // ---------------- epilogue (warps 2..5) ----------------
        const int quarter = warp & 3;  // TMEM lanes 32*quarter .. +31
        const int epi_thread = (warp - 2) * 32 + lane;
        uint4 *epi_stage = reinterpret_cast<uint4 *>(tiles + kStagesMx * kStageStride +
                                                     (warp - 2) * kEpilogueWarpStageBytes);
        auto epilogue_aborted = [&]() -> bool {
            if (epi_thread == 0)
                st.epi_abort = st.abort;
            asm volatile("bar.sync 1, 128;" ::: "memory");
            const int sample = st.epi_abort;
            asm volatile("bar.sync 1, 128;" ::: "memory");
            return sample != 0;
        };
        Tile t;
        bool aborted = false;
        for (int it = 0; policy.next(it, t); ++it) {
            if ((aborted = epilogue_aborted()))
                break;
            if constexpr (Policy::kBackground) {
                // While the accumulator is not ready the four warps run the policy's background
                // items (communication); one thread polls and a named barrier shares the decision.
                for (;;) {
                    if (epi_thread == 0)
                        st.epi_ready = mbar_try_wait(&st.tmem_full[0], it & 1) ? 1 : 0;
                    asm volatile("bar.sync 1, 128;" ::: "memory");
                    const int ready_now = st.epi_ready;
                    asm volatile("bar.sync 1, 128;" ::: "memory");
                    if (ready_now || !policy.background(epi_thread, kEpilogueWarps * 32))
                        break;
                }
            }
            if (!mbar_wait(&st.tmem_full[0], it & 1)) {
                st.abort = 1;
                set_status(status, aboleth::Status::Timeout, 0x3400);
            } else {
                tc_fence_after();
#pragma unroll
                for (int h = 0; h < HALVES; ++h) {
                    const std::uint32_t taddr = tmem_base + (static_cast<std::uint32_t>(quarter * 32) << 16) +
                                                h * G::kCols;
                    drain_rows32(policy, t, taddr, h * BM + quarter * 32, epi_stage, lane);
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0)
                    mbar_arrive(&st.tmem_empty[0]);
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if constexpr (Policy::kDrainedHook) {  // the accumulator is released: this overlaps the next main loop
                policy.drained(t, epi_thread, kEpilogueWarps * 32);
                asm volatile("bar.sync 1, 128;" ::: "memory");
            }
            if (warp == 2 && lane == 0)
                policy.tile_done(t);
        }
        if constexpr (Policy::kBackground) {
            while (!aborted && !(aborted = epilogue_aborted()) &&
                   policy.background(epi_thread, kEpilogueWarps * 32)) {
            }
        }
        if (!aborted && !epilogue_aborted())
            policy.finish(epi_thread, kEpilogueWarps * 32, status);
    }

    // ---------------- teardown ----------------
    __syncwarp();
    if (st.abort) {
        // Let copies that are still in flight land before the CTA's shared memory is handed on.
        const std::uint64_t t0 = aboleth::detail::globaltimer_ns();
        while (aboleth::detail::globaltimer_ns() - t0 < 2000000ull)
            __nanosleep(1000);
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (warp == 1)
        tmem_dealloc(tmem_base, kTmemCols);
}

}  // namespace ab::gemm::mx
