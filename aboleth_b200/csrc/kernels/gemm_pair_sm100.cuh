// The CTA-pair form of the tcgen05 GEMM main loop (tcgen05 `cta_group::2`).
//
// Two CTAs of one cluster (the two SMs of a TPC) compute one 256 x 256 tile together:
//
//   * CTA r of the pair loads rows [r*128, r*128+128) of the A tile and rows
//     [r*128, r*128+128) of the B tile (half of N) into ITS OWN shared memory - 32 KiB per
//     K step of 64 instead of 64 KiB, so the same 192 KiB of shared memory holds a
//     6-deep ring (about 3.3 us of tensor work in flight at full rate) instead of 3.
//   * Only the pair's leader (cluster rank 0) issues tcgen05.mma.cta_group::2 with
//     M = 256, N = 256: the instruction reads A and B from both CTAs' shared memory and
//     accumulates rows r*128.. of the tile in CTA r's tensor memory, 256 fp32 columns.
//   * Each CTA therefore needs 256 of its 512 TMEM columns per tile: the accumulator is
//     double buffered, and the epilogue of tile i overlaps the main loop of tile i+1.
//
// Barriers.  `full[s]` lives in the leader: both CTAs' TMA loads complete their bytes on
// it (the peer's loads name the leader's barrier through its shared::cluster address); the
// leader's producer makes the one arrival and announces the bytes of both.  `empty[s]`, `tmem_full[b]` exist in both CTAs and are
// signalled by one tcgen05.commit that is multicast to the pair.  `tmem_empty[b]` lives in
// the leader and counts the epilogue warps of both CTAs.  No TMA load is multicast.
//
// Every wait is bounded as in the single-CTA loop; the two CTAs meet at a cluster barrier
// before the tensor memory is freed, so neither leaves while its peer can still touch it.
#pragma once

#include "gemm_sm100.cuh"

namespace ab::gemm::pair {

// MH = 128-row blocks of A per CTA.
//   MH = 1: tile 256 x 256, 32 KiB per CTA and K step, 6 stages, accumulator double buffered.
//   MH = 2: tile 512 x 256: each CTA holds 256 rows of A and its half of B (48 KiB per K step,
//           4 stages); two pair-MMAs per K step share the B tile, which cuts the bytes fetched
//           from L2 per FLOP by a third - the plain 256 x 256 tiling runs at the L2 read
//           bandwidth (about 12 TB/s measured), not at the tensor rate.  Each TMEM half holds
//           one accumulator; the epilogue drains half 0 first.
template <int MH>
struct PairGeometry {
    static constexpr int kRowsPerCta = MH * BM;
    static constexpr int kTileRows = 2 * kRowsPerCta;
    static constexpr int kStages = MH == 1 ? 6 : 4;
    static constexpr unsigned kBytesA = kRowsPerCta * BK * 2;    // per CTA and stage
    static constexpr unsigned kBytesB = (BN / 2) * BK * 2;
    static constexpr unsigned kStageBytes = kBytesA + kBytesB;
    static constexpr unsigned kSmemBytes = kStages * kStageBytes + kEpilogueStageBytes + 1024;
};
constexpr int kPairMaxStages = 6;

struct PairState {
    std::uint64_t full[kPairMaxStages];    // used in the leader only
    std::uint64_t empty[kPairMaxStages];
    std::uint64_t tmem_full[2];
    std::uint64_t tmem_empty[2];        // used in the leader only
    std::uint32_t tmem_base;
    volatile int abort;
    volatile int epi_ready;
    volatile int epi_abort;  // epilogue warps: shared sample of `abort`
};

// Raise `abort` in this CTA and in its pair CTA: either of them giving up must end both, because
// each one's barriers are completed by the other.
__device__ __forceinline__ void raise_abort(PairState &st, unsigned rank);

__device__ __forceinline__ unsigned cluster_rank() {
    unsigned r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}

// shared::cluster address of `local` (a shared::cta address of this CTA) in CTA `rank`.
__device__ __forceinline__ std::uint32_t map_to_cta(std::uint32_t local, unsigned rank) {
    std::uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local), "r"(rank));
    return remote;
}

__device__ __forceinline__ void raise_abort(PairState &st, unsigned rank) {
    st.abort = 1;
    const std::uint32_t remote = map_to_cta(smem_u32(const_cast<int *>(&st.abort)), rank ^ 1u);
    asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(remote), "r"(1) : "memory");
}

__device__ __forceinline__ void cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

__device__ __forceinline__ void pair_tmem_alloc(std::uint32_t *holder, unsigned cols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(holder)),
                 "r"(cols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void pair_tmem_dealloc(std::uint32_t base, unsigned cols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(base), "r"(cols)
                 : "memory");
}

template <typename Op>
__device__ __forceinline__ void pair_umma(std::uint32_t d_tmem, std::uint64_t a_desc, std::uint64_t b_desc,
                                          std::uint32_t idesc, std::uint32_t accumulate) {
    if constexpr (Op::kBK == 64) {
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "setp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
            ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
            : "memory");
    } else {
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "setp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
            ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
            : "memory");
    }
}

// One arrival on the barrier at this shared-memory offset in BOTH CTAs of the pair once
// every tcgen05 operation issued so far by this thread is done.
__device__ __forceinline__ void pair_umma_commit(std::uint64_t *bar) {
    const std::uint16_t mask = 3;
    asm volatile(
        "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::
            "r"(smem_u32(bar)),
        "h"(mask)
        : "memory");
}

// Tiled load into this CTA's shared memory whose bytes complete on a barrier that may
// belong to the peer CTA (shared::cluster address).  Not multicast.
__device__ __forceinline__ void pair_tma_load_2d(void *smem_dst, const CUtensorMap *map, int x, int y,
                                                 std::uint32_t bar_cluster_addr) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes "
        "[%0], [%1, {%3, %4}], [%2];" ::"r"(smem_u32(smem_dst)),
        "l"(map), "r"(bar_cluster_addr), "r"(x), "r"(y)
        : "memory");
}

__device__ __forceinline__ void remote_arrive(std::uint32_t bar_cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar_cluster_addr)
                 : "memory");
}

__device__ __forceinline__ void remote_arrive_expect_tx(std::uint32_t bar_cluster_addr, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.release.cluster.shared::cluster.b64 _, [%0], %1;" ::"r"(
                     bar_cluster_addr),
                 "r"(bytes)
                 : "memory");
}

// A wait that also acquires, at cluster scope, what the peer CTA released.  Used once per tile
// (the accumulator hand-back); the per-K-step waits use the CTA-scope form.
__device__ __forceinline__ bool pair_try_wait(std::uint64_t *bar, unsigned parity) {
    unsigned ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}

__device__ __forceinline__ bool pair_wait(std::uint64_t *bar, unsigned parity) {
    for (int i = 0; i < 4096; ++i)
        if (pair_try_wait(bar, parity))
            return true;
    const std::uint64_t start = aboleth::detail::globaltimer_ns();
    while (!pair_try_wait(bar, parity)) {
        if (aboleth::detail::globaltimer_ns() - start > 4000000000ull)
            return false;
    }
    return true;
}

// Policy concept: the one of gemm_mainloop, with tiles of PairGeometry<MH>::kTileRows rows.
// `policy.next` must hand the SAME tile to both CTAs of a pair (index tiles by blockIdx.x / 2
// out of gridDim.x / 2).  Rows passed to `store16` are rows of the tile.  map_a boxes are
// (MH * 128) rows x 128 bytes, map_b boxes 128 rows x 128 bytes; `Op` selects bf16 or e4m3 operands.
template <int MH, typename Op, typename Policy>
__device__ __forceinline__ void gemm_mainloop_pair(Policy &policy, const CUtensorMap *map_a,
                                                   const CUtensorMap *map_b, unsigned long long *status,
                                                   const CUtensorMap *map_a_alt = nullptr) {
    using G = PairGeometry<MH>;
    constexpr int kStagesG = G::kStages;
    if (map_a_alt == nullptr)
        map_a_alt = map_a;
    extern __shared__ std::uint8_t smem_raw[];
    __shared__ PairState st;
    std::uint8_t *tiles = reinterpret_cast<std::uint8_t *>(
        (reinterpret_cast<std::uintptr_t>(smem_raw) + 1023) & ~static_cast<std::uintptr_t>(1023));
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const unsigned rank = cluster_rank();  // 0: leader
    const bool leader = rank == 0;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStagesG; ++s) {
            mbar_init(&st.full[s], 1);   // the leader's arrival carries the byte count of BOTH CTAs' loads
            mbar_init(&st.empty[s], 1);  // one multicast commit
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&st.tmem_full[b], 1);
            mbar_init(&st.tmem_empty[b], 2 * kEpilogueWarps);
        }
        st.abort = 0;
        mbar_fence_init();
        prefetch_tensormap(map_a);
        prefetch_tensormap(map_b);
    }
    if (warp == 1)
        pair_tmem_alloc(&st.tmem_base, kTmemCols);
    tc_fence_before();
    __syncthreads();
    cluster_sync();  // both CTAs' barriers exist before anything is signalled across
    tc_fence_after();
    const std::uint32_t tmem_base = st.tmem_base;

    // Accumulator slot (TMEM half) and barrier parity of block `h` of tile `it`.
    auto slot_of = [](int it, int h) { return MH == 1 ? (it & 1) : h; };
    auto use_of = [](int it) -> unsigned { return MH == 1 ? ((it >> 1) & 1) : (it & 1); };

    if (warp == 0) {
        // ---------------- TMA producer (both CTAs) ----------------
        if (lane == 0) {
            int stage = 0;
            unsigned phase = 0;
            Tile t;
#ifdef AB_GEMM_TRACE
            long long t_wait = 0, t_begin = clock64();
#endif
            for (int it = 0; !st.abort && policy.next(it, t); ++it) {
                if (!policy.ready(t)) {
                    raise_abort(st, rank);
                    set_status(status, aboleth::Status::Timeout, 0x3000 + t.tag);
                    break;
                }
                for (int kb = 0; kb < t.k_blocks; ++kb) {
#ifdef AB_GEMM_TRACE
                    const long long w0 = clock64();
#endif
                    const bool got = mbar_wait(&st.empty[stage], phase ^ 1);
#ifdef AB_GEMM_TRACE
                    t_wait += clock64() - w0;
#endif
                    if (!got || st.abort) {
                        raise_abort(st, rank);
                        set_status(status, aboleth::Status::Timeout, 0x3100 + stage);
                        break;
                    }
                    std::uint8_t *sa = tiles + stage * G::kStageBytes;
                    const std::uint32_t full_in_leader = map_to_cta(smem_u32(&st.full[stage]), 0);
                    // The peer does not arrive: its loads only complete bytes on the leader's barrier.
                    // (A cluster-scope release arrive per K step cost ~1400 cycles and starved the pipe.)
                    if (leader)
                        mbar_expect_tx(&st.full[stage], 2 * G::kStageBytes);
                    pair_tma_load_2d(sa, t.a_sel ? map_a_alt : map_a, kb * Op::kBK,
                                     t.a_row + static_cast<int>(rank) * G::kRowsPerCta, full_in_leader);
                    pair_tma_load_2d(sa + G::kBytesA, map_b, kb * Op::kBK, t.b_row + static_cast<int>(rank) * (BN / 2),
                                     full_in_leader);
                    if (++stage == kStagesG) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
            }
#ifdef AB_GEMM_TRACE
            if (blockIdx.x < 2 && status != nullptr) {
                status[2 + 2 * blockIdx.x] = t_wait;                 // producer: cycles waiting for a free stage
                status[3 + 2 * blockIdx.x] = clock64() - t_begin;    // producer: cycles in its loop
            }
#endif
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer (leader only) ----------------
        if (lane == 0 && leader) {
            constexpr std::uint32_t idesc = Op::idesc(2 * BM, BN);
            int stage = 0;
            unsigned phase = 0;
            Tile t;
#ifdef AB_GEMM_TRACE
            long long t_full = 0, t_acc = 0, t_begin = clock64();
#endif
            for (int it = 0; !st.abort && policy.next(it, t); ++it) {
                const unsigned use = use_of(it);
                for (int kb = 0; kb < t.k_blocks && !st.abort; ++kb) {
#ifdef AB_GEMM_TRACE
                    const long long f0 = clock64();
#endif
                    const bool filled = mbar_wait(&st.full[stage], phase);
#ifdef AB_GEMM_TRACE
                    t_full += clock64() - f0;
#endif
                    if (!filled) {
                        raise_abort(st, rank);
                        set_status(status, aboleth::Status::Timeout, 0x3300 + stage);
                        break;
                    }
                    tc_fence_after();
                    const std::uint32_t sa = smem_u32(tiles + stage * G::kStageBytes);
                    const std::uint64_t db = smem_desc_sw128(sa + G::kBytesA);
#pragma unroll
                    for (int h = 0; h < MH; ++h) {
                        const int slot = slot_of(it, h);
                        if (kb == 0) {
                            // Both CTAs' epilogues must have drained this accumulator.
#ifdef AB_GEMM_TRACE
                            const long long a0 = clock64();
#endif
                            const bool free_acc = pair_wait(&st.tmem_empty[slot], use ^ 1);
#ifdef AB_GEMM_TRACE
                            t_acc += clock64() - a0;
#endif
                            if (!free_acc) {
                                raise_abort(st, rank);
                                set_status(status, aboleth::Status::Timeout, 0x3200 + slot);
                                break;
                            }
                            tc_fence_after();
                        }
                        const std::uint32_t d = tmem_base + slot * BN;
                        const std::uint64_t da = smem_desc_sw128(sa + h * (BM * BK * 2));
#pragma unroll
                        for (int k = 0; k < 4; ++k)  // four MMAs per stage, 32 bytes of K each
                            pair_umma<Op>(d, da + 2 * k, db + 2 * k, idesc, (kb | k) != 0);
                    }
                    pair_umma_commit(&st.empty[stage]);  // frees the stage in both CTAs
                    if (++stage == kStagesG) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
#pragma unroll
                for (int h = 0; h < MH; ++h)
                    pair_umma_commit(&st.tmem_full[slot_of(it, h)]);  // accumulators complete, both CTAs
            }
#ifdef AB_GEMM_TRACE
            if (blockIdx.x == 0 && status != nullptr) {
                status[6] = t_full;                  // MMA issuer: cycles waiting for operands
                status[7] = t_acc;                   // MMA issuer: cycles waiting for a free accumulator
                status[8] = clock64() - t_begin;     // MMA issuer: cycles in its loop
            }
#endif
        }
    } else {
        // ---------------- epilogue (warps 2..5, both CTAs) ----------------
        const int quarter = warp & 3;
        const int epi_thread = (warp - 2) * 32 + lane;
        constexpr int kEpiThreads = kEpilogueWarps * 32;
        uint4 *epi_stage = reinterpret_cast<uint4 *>(tiles + kStagesG * G::kStageBytes +
                                                     (warp - 2) * kEpilogueWarpStageBytes);
        // `abort` is raised asynchronously by the producer or the MMA lane.  The four epilogue warps
        // meet at named barrier 1, so they must all take the same way out: one thread samples the
        // flag and the sample is what all 128 threads branch on.
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
            const unsigned use = use_of(it);
#pragma unroll
            for (int h = 0; h < MH; ++h) {
                const int slot = slot_of(it, h);
                if constexpr (Policy::kBackground) {
                    for (;;) {
                        if (epi_thread == 0)
                            st.epi_ready = mbar_try_wait(&st.tmem_full[slot], use) ? 1 : 0;
                        asm volatile("bar.sync 1, 128;" ::: "memory");
                        const int ready_now = st.epi_ready;
                        asm volatile("bar.sync 1, 128;" ::: "memory");
                        if (ready_now || !policy.background(epi_thread, kEpiThreads))
                            break;
                    }
                }
                if (!mbar_wait(&st.tmem_full[slot], use)) {
                    raise_abort(st, rank);
                    set_status(status, aboleth::Status::Timeout, 0x3400 + slot);
                    break;
                }
                tc_fence_after();
                const std::uint32_t taddr = tmem_base + (static_cast<std::uint32_t>(quarter * 32) << 16) +
                                            slot * BN;
                drain_rows32(policy, t, taddr, static_cast<int>(rank) * G::kRowsPerCta + h * BM + quarter * 32,
                             epi_stage, lane);
                tc_fence_before();
                __syncwarp();
                if (lane == 0)
                    remote_arrive(map_to_cta(smem_u32(&st.tmem_empty[slot]), 0));
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if constexpr (Policy::kDrainedHook) {
                policy.drained(t, epi_thread, kEpiThreads);
                asm volatile("bar.sync 1, 128;" ::: "memory");
            }
            if (warp == 2 && lane == 0)
                policy.tile_done(t);
        }
        if constexpr (Policy::kBackground) {
            while (!aborted && !(aborted = epilogue_aborted()) &&
                   policy.background(epi_thread, kEpiThreads)) {
            }
        }
        if (!aborted && !epilogue_aborted())
            policy.finish(epi_thread, kEpiThreads, status);
    }

    // ---------------- teardown ----------------
    __syncwarp();
    if (st.abort) {
        const std::uint64_t t0 = aboleth::detail::globaltimer_ns();
        while (aboleth::detail::globaltimer_ns() - t0 < 2000000ull)
            __nanosleep(1000);
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync();  // the peer no longer reads this CTA's shared memory or signals its barriers
    tc_fence_after();
    if (warp == 1)
        pair_tmem_dealloc(tmem_base, kTmemCols);
}

}  // namespace ab::gemm::pair
