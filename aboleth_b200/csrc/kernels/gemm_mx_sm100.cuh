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
// Per K block the producer brings in the A tile (16 KiB), the B tile (32 KiB) by TMA and the A
// atom (512 B) and two B atoms (1 KiB) by untiled bulk copies on the same mbarrier; nothing is
// multicast.
//
// One 128 x 256 accumulator (256 columns) plus 12 columns of scale factors: the second
// accumulator buffer of the bf16 loop does not fit beside them, so the epilogue of a tile is not
// overlapped with the next tile's main loop here.
//
// Same roles, same bounded waits and the same policy interface as gemm_sm100.cuh.
#pragma once

#include "gemm_sm100.cuh"

namespace ab::gemm::mx {

constexpr int kBlockK = 128;                    // e4m3 elements (= bytes) of K per stage
constexpr int kStagesMx = 3;
constexpr unsigned kBytesA = BM * kBlockK;      // 16 KiB
constexpr unsigned kBytesB = BN * kBlockK;      // 32 KiB
constexpr unsigned kAtomBytes = 512;            // scale factors of 128 rows x 128 K
constexpr unsigned kOffSfa = kBytesA + kBytesB;
constexpr unsigned kOffSfb = kOffSfa + kAtomBytes;
constexpr unsigned kStageStride = 50 * 1024;    // tiles + 3 atoms, rounded up to the swizzle alignment
constexpr unsigned kStageTx = kBytesA + kBytesB + 3 * kAtomBytes;
constexpr unsigned kSmemBytes = kStagesMx * kStageStride + kEpilogueStageBytes + 1024;
constexpr unsigned kSfaCol = 256, kSfbCol = 260;  // tensor-memory columns behind the accumulator

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

// Where the packed scale factors of a problem live.  A: atoms [row block][K block]; B: atoms
// [K block][column block], column block fastest and padded to an even count so that the two atoms
// of a 256-column tile are adjacent.
struct ScaleFactors {
    const std::uint8_t *a;
    const std::uint8_t *b;
    int k_blocks;     // K / 128
    int b_blocks;     // padded column blocks per K block
};

template <typename Policy>
__device__ __forceinline__ void gemm_mx_mainloop(Policy &policy, const CUtensorMap *map_a,
                                                 const CUtensorMap *map_b, const ScaleFactors sf,
                                                 unsigned long long *status) {
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
                const std::uint8_t *sfa = sf.a + static_cast<std::size_t>(t.a_row / BM) * sf.k_blocks * kAtomBytes;
                const std::uint8_t *sfb = sf.b + static_cast<std::size_t>(t.b_row / 128) * kAtomBytes;
                for (int kb = 0; kb < t.k_blocks; ++kb) {
                    if (!mbar_wait(&st.empty[stage], phase ^ 1) || st.abort) {
                        st.abort = 1;
                        set_status(status, aboleth::Status::Timeout, 0x3100 + stage);
                        break;
                    }
                    std::uint8_t *sa = tiles + stage * kStageStride;
                    mbar_expect_tx(&st.full[stage], kStageTx);
                    tma_load_2d(sa, map_a, kb * kBlockK, t.a_row, &st.full[stage]);
                    tma_load_2d(sa + kBytesA, map_b, kb * kBlockK, t.b_row, &st.full[stage]);
                    bulk_load(sa + kOffSfa, sfa + static_cast<std::size_t>(kb) * kAtomBytes, kAtomBytes,
                              &st.full[stage]);
                    bulk_load(sa + kOffSfb, sfb + static_cast<std::size_t>(kb) * sf.b_blocks * kAtomBytes,
                              2 * kAtomBytes, &st.full[stage]);
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
                    sf_copy(tmem_base + kSfaCol, sf_desc(sa + kOffSfa));
                    sf_copy(tmem_base + kSfbCol, sf_desc(sa + kOffSfb));
                    sf_copy(tmem_base + kSfbCol + 4, sf_desc(sa + kOffSfb + kAtomBytes));
                    const std::uint64_t da = smem_desc_sw128(sa);
                    const std::uint64_t db = smem_desc_sw128(sa + kBytesA);
#pragma unroll
                    for (unsigned k = 0; k < 4; ++k) {
                        // 32 e4m3 = 32 bytes further along K inside the swizzle atom.
                        umma_mx(tmem_base, da + (k * 32 >> 4), db + (k * 32 >> 4), idesc_mx(BM, BN, k),
                                tmem_base + kSfaCol, tmem_base + kSfbCol, (kb | static_cast<int>(k)) != 0);
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
            if (!mbar_wait(&st.tmem_full[0], it & 1)) {
                st.abort = 1;
                set_status(status, aboleth::Status::Timeout, 0x3400);
            } else {
                tc_fence_after();
                const std::uint32_t taddr = tmem_base + (static_cast<std::uint32_t>(quarter * 32) << 16);
                drain_rows32(policy, t, taddr, quarter * 32, epi_stage, lane);
                tc_fence_before();
                __syncwarp();
                if (lane == 0)
                    mbar_arrive(&st.tmem_empty[0]);
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if (warp == 2 && lane == 0)
                policy.tile_done(t);
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
