// tcgen05 / TMEM / TMA building blocks and the persistent warp-specialised GEMM
// main loop shared by the plain, grouped, all-gather->GEMM and
// GEMM->reduce-scatter kernels.
//
//   C[M, N] (+)= A[M, K] * B[N, K]^T      A, B bf16 K-major, fp32 accumulate in TMEM
//
// CTA = 192 threads: warp 0 issues TMA loads (one lane), warp 1 allocates TMEM
// and issues tcgen05.mma (one lane), warps 2..5 are the epilogue (each owns the
// 32 TMEM lanes its warp id selects).  One CTA per SM, persistent over tiles of
// 128 x 256; the accumulator is double buffered in TMEM (2 x 256 columns) so
// the epilogue of tile i overlaps the main loop of tile i+1.  Operands travel
// global -> shared by TMA (cp.async.bulk.tensor, 128-byte swizzle, never
// multicast) through a 4-stage ring of 48 KiB stages.
//
// Every wait is bounded.  A role that gives up sets the CTA's abort flag; all
// roles then leave their loops, the CTA lets copies in flight land, frees its
// TMEM and returns with Status::Timeout recorded.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>

#include "common.cuh"

namespace ab::gemm {

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int BK = 64;   // 64 bf16 = 128 bytes = one swizzle atom row
constexpr int UMMA_K = 16;
constexpr int kStages = 4;  // upper bound over configurations (barrier array size)
constexpr int kThreads = 192;
constexpr int kEpilogueWarps = 4;
constexpr unsigned kTmemCols = 512;
// Per epilogue warp: 32 rows x 128 bf16 columns, through which an accumulator is transposed so
// that the stores to C are row-contiguous (two 256-byte row pieces per warp instruction).
constexpr unsigned kEpilogueWarpStageBytes = 32 * 128 * 2;
constexpr unsigned kEpilogueStageBytes = kEpilogueWarps * kEpilogueWarpStageBytes;

struct SharedState {
    std::uint64_t full[kStages];
    std::uint64_t empty[kStages];
    std::uint64_t tmem_full[2];
    std::uint64_t tmem_empty[2];
    std::uint32_t tmem_base;
    volatile int abort;
    volatile int epi_ready;  // epilogue warps: shared outcome of one accumulator poll
    volatile int epi_abort;  // epilogue warps: shared sample of `abort`
};

// ---- tcgen05 wrappers --------------------------------------------------------------

__device__ __forceinline__ void tmem_alloc(std::uint32_t *holder, unsigned cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(holder)),
                 "r"(cols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_dealloc(std::uint32_t base, unsigned cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(base), "r"(cols)
                 : "memory");
}

__device__ __forceinline__ void tc_fence_before() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}

__device__ __forceinline__ void tc_fence_after() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// D[tmem] (+)= A[smem desc] * B[smem desc]; accumulate selects += over =.
__device__ __forceinline__ void umma_bf16(std::uint32_t d_tmem, std::uint64_t a_desc,
                                          std::uint64_t b_desc, std::uint32_t idesc,
                                          std::uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// mbarrier arrives once every tcgen05 operation issued so far by this thread is done.
__device__ __forceinline__ void umma_commit(std::uint64_t *bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                     smem_u32(bar))
                 : "memory");
}

// 32 lanes x 32 consecutive fp32 columns: thread i of the warp gets row i.
__device__ __forceinline__ void tmem_ld32(std::uint32_t addr, float *v) {
    std::uint32_t r[32];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
        "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
          "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
          "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]),
          "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]),
          "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(addr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 32; ++i)
        v[i] = __uint_as_float(r[i]);
}

// Instruction descriptor, kind::f16: fp32 accumulate, bf16 A and B, both K-major.
__host__ __device__ constexpr std::uint32_t idesc_bf16(int m, int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<std::uint32_t>(n >> 3) << 17) |
           (static_cast<std::uint32_t>(m >> 4) << 24);
}

// Shared-memory matrix descriptor: K-major tile of 128-byte rows, 128-byte
// swizzle, 8-row groups 1024 bytes apart; the tile base is 1024-byte aligned.
__device__ __forceinline__ std::uint64_t smem_desc_sw128(std::uint32_t smem_addr) {
    return static_cast<std::uint64_t>((smem_addr & 0x3ffffu) >> 4) | (1ull << 16) |
           (static_cast<std::uint64_t>(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}

// Instruction descriptor, kind::f8f6f4 with e4m3 A and B (format code 0), fp32 accumulate, K-major.
__host__ __device__ constexpr std::uint32_t idesc_e4m3(int m, int n) {
    return (1u << 4) | (static_cast<std::uint32_t>(n >> 3) << 17) | (static_cast<std::uint32_t>(m >> 4) << 24);
}

// Operand kinds of the main loops.  Both fill a 128-byte swizzle row per K step (64 bf16 or
// 128 e4m3) and advance the shared-memory descriptors by 32 bytes per MMA, so the loops differ
// only in the K extent of a step, the instruction kind and its descriptor.
struct OpBf16 {
    static constexpr int kBK = 64;  // elements of K per stage
    static constexpr const char *kName = "bf16";
    __host__ __device__ static constexpr std::uint32_t idesc(int m, int n) { return idesc_bf16(m, n); }
};
struct OpE4m3 {
    static constexpr int kBK = 128;
    static constexpr const char *kName = "e4m3";
    __host__ __device__ static constexpr std::uint32_t idesc(int m, int n) { return idesc_e4m3(m, n); }
};

// ---- TMA (tiled, no multicast) --------------------------------------------------------

__device__ __forceinline__ void tma_load_2d(void *smem_dst, const CUtensorMap *map, int x, int y,
                                            std::uint64_t *bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes "
        "[%0], [%1, {%3, %4}], [%2];" ::"r"(smem_u32(smem_dst)),
        "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y)
        : "memory");
}

__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap *map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}

// ---- epilogue: one 128-row accumulator block, one warp's 32 rows ----------------------------
//
// TMEM -> registers (32 lanes x 32 columns at a time) -> bf16 -> this warp's staging in shared
// memory (row r at r*256 bytes, its sixteen 16-byte units XOR-swizzled with r & 15, which keeps
// both directions free of bank conflicts) -> `policy.store16`, 16 lanes per row.
__device__ __forceinline__ uint4 pack8_bf16(const float *v) {
    __nv_bfloat162 p0 = __floats2bfloat162_rn(v[0], v[1]);
    __nv_bfloat162 p1 = __floats2bfloat162_rn(v[2], v[3]);
    __nv_bfloat162 p2 = __floats2bfloat162_rn(v[4], v[5]);
    __nv_bfloat162 p3 = __floats2bfloat162_rn(v[6], v[7]);
    uint4 o;
    o.x = *reinterpret_cast<std::uint32_t *>(&p0);
    o.y = *reinterpret_cast<std::uint32_t *>(&p1);
    o.z = *reinterpret_cast<std::uint32_t *>(&p2);
    o.w = *reinterpret_cast<std::uint32_t *>(&p3);
    return o;
}

template <typename Policy, typename TileT>
__device__ __forceinline__ void drain_rows32(Policy &policy, const TileT &t, std::uint32_t taddr,
                                             int row_base, uint4 *stage, int lane) {
#pragma unroll 1
    for (int g = 0; g < BN / 128; ++g) {
        if (g * 128 >= t.cols_valid)
            break;
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
            float v[32];
            tmem_ld32(taddr + g * 128 + c * 32, v);
            if constexpr (Policy::kScaled) {
                const float alpha = policy.alpha;
#pragma unroll
                for (int i = 0; i < 32; ++i)
                    v[i] *= alpha;
            }
#pragma unroll
            for (int q = 0; q < 4; ++q)
                stage[lane * 16 + ((c * 4 + q) ^ (lane & 15))] = pack8_bf16(v + q * 8);
        }
        __syncwarp();
#pragma unroll 4
        for (int j = 0; j < 16; ++j) {
            const int idx = j * 32 + lane;
            const int r = idx >> 4, unit = idx & 15;
            const uint4 value = stage[r * 16 + (unit ^ (r & 15))];
            const int row = row_base + r, col = g * 128 + unit * 8;
            if (row < t.rows_valid && col < t.cols_valid)
                policy.store16(t, row, col, value);
        }
        __syncwarp();
    }
}

// ---- tile description handed out by a policy -------------------------------------------

struct Tile {
    int a_row;       // first row of the A tile in the A tensor map
    int b_row;       // first row of the B tile in the B tensor map
    int k_blocks;    // K / BK
    int c_row;       // first output row
    int c_col;       // first output column
    int rows_valid;  // output rows of this tile that exist (<= 128 * HALVES)
    int cols_valid;  // output columns that exist (<= BN)
    int tag;         // policy-defined (expert, source rank, ...)
    int a_sel;       // 0: first A tensor map, 1: the alternate one
};

// Policy concept:
//   __device__ bool next(int iteration, Tile &t)          - tile `iteration` of this CTA, false when done
//   __device__ bool ready(const Tile &t)                  - producer-side gate before loading A (bounded)
//   __device__ void store16(const Tile &t, int row, int col, const uint4 &v)
//                                                         - eight bf16 of tile row `row` at tile columns
//                                                           col..col+7 (col a multiple of 8); only called
//                                                           for rows and columns that exist; consecutive
//                                                           lanes get consecutive 16-byte pieces of a row
//   __device__ void tile_done(const Tile &t)              - called by ONE epilogue thread after the
//                                                           whole tile was stored (CTA-wide ordered)
//   __device__ void finish(int thread, int nthreads, status) - epilogue warps, after the last tile
//   static constexpr bool kScaled      - if true: the accumulator is multiplied by `float alpha` (a policy
//                                        member) before it is rounded to bf16
//   static constexpr bool kBackground  - if true: bool background(int thread, int nthreads) is called by
//                                        all 128 epilogue threads together while they would otherwise
//                                        wait for an accumulator, and after the last tile until it
//                                        returns false (no item left); it may use `bar.sync 1, 128`
//   static constexpr bool kDrainedHook - if true: void drained(const Tile &, int thread, int nthreads) is
//                                        called by all 128 epilogue threads after a tile was stored and
//                                        its accumulator released, before tile_done
// `map_a_alt` is the tensor map used by tiles with a_sel == 1 (pass map_a when unused).
// Geometry of one configuration.  HALVES = 1: 128 x 256 tiles, the two 256-column
// halves of TMEM double-buffer the accumulator (epilogue of tile i overlaps the main
// loop of tile i+1), 4 stages of 48 KiB.  HALVES = 2: 256 x 256 tiles - two 128-row
// MMAs per K step share one B tile, which cuts shared-memory fill traffic per FLOP by
// a third - each TMEM half holds one 128-row accumulator, the epilogue drains half 0
// first so the next tile's first MMAs can start while half 1 drains; 3 stages of 64 KiB.
template <int HALVES>
struct Geometry {
    static constexpr int kRows = BM * HALVES;
    static constexpr int kStages = HALVES == 1 ? 4 : 3;
    static constexpr unsigned kBytesA = kRows * BK * 2;
    static constexpr unsigned kBytesB = BN * BK * 2;
    static constexpr unsigned kStageBytes = kBytesA + kBytesB;
    static constexpr unsigned kSmemBytes = kStages * kStageBytes + kEpilogueStageBytes + 1024;
};

template <int HALVES, typename Policy>
__device__ __forceinline__ void gemm_mainloop(Policy &policy, const CUtensorMap *map_a,
                                              const CUtensorMap *map_b,
                                              unsigned long long *status,
                                              const CUtensorMap *map_a_alt = nullptr) {
    using G = Geometry<HALVES>;
    constexpr int kStagesG = G::kStages;
    if (map_a_alt == nullptr)
        map_a_alt = map_a;
    extern __shared__ std::uint8_t smem_raw[];
    __shared__ SharedState st;
    std::uint8_t *tiles = reinterpret_cast<std::uint8_t *>(
        (reinterpret_cast<std::uintptr_t>(smem_raw) + 1023) & ~static_cast<std::uintptr_t>(1023));
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStagesG; ++s) {
            mbar_init(&st.full[s], 1);
            mbar_init(&st.empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&st.tmem_full[b], 1);
            mbar_init(&st.tmem_empty[b], kEpilogueWarps);
        }
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

    // Accumulator slot (TMEM half) and barrier parity of half `h` of tile `it`.
    auto slot_of = [](int it, int h) { return HALVES == 1 ? (it & 1) : h; };
    auto use_of = [](int it) -> unsigned { return HALVES == 1 ? ((it >> 1) & 1) : (it & 1); };

    if (warp == 0) {
        // ---------------- TMA producer ----------------
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
                for (int kb = 0; kb < t.k_blocks; ++kb) {
                    if (!mbar_wait(&st.empty[stage], phase ^ 1) || st.abort) {
                        st.abort = 1;
                        set_status(status, aboleth::Status::Timeout, 0x3100 + stage);
                        break;
                    }
                    std::uint8_t *sa = tiles + stage * G::kStageBytes;
                    mbar_expect_tx(&st.full[stage], G::kStageBytes);
                    tma_load_2d(sa, t.a_sel ? map_a_alt : map_a, kb * BK, t.a_row, &st.full[stage]);
                    tma_load_2d(sa + G::kBytesA, map_b, kb * BK, t.b_row, &st.full[stage]);
                    if (++stage == kStagesG) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            constexpr std::uint32_t idesc = idesc_bf16(BM, BN);
            int stage = 0;
            unsigned phase = 0;
            Tile t;
            for (int it = 0; !st.abort && policy.next(it, t); ++it) {
                const unsigned use = use_of(it);
                for (int kb = 0; kb < t.k_blocks && !st.abort; ++kb) {
                    if (!mbar_wait(&st.full[stage], phase)) {
                        st.abort = 1;
                        set_status(status, aboleth::Status::Timeout, 0x3300 + stage);
                        break;
                    }
                    tc_fence_after();
                    const std::uint32_t sa = smem_u32(tiles + stage * G::kStageBytes);
                    const std::uint64_t db = smem_desc_sw128(sa + G::kBytesA);
#pragma unroll
                    for (int h = 0; h < HALVES; ++h) {
                        const int slot = slot_of(it, h);
                        if (kb == 0) {
                            // The accumulator must have been drained by the epilogue.
                            if (!mbar_wait(&st.tmem_empty[slot], use ^ 1)) {
                                st.abort = 1;
                                set_status(status, aboleth::Status::Timeout, 0x3200 + slot);
                                break;
                            }
                            tc_fence_after();
                        }
                        const std::uint32_t d = tmem_base + slot * BN;
                        const std::uint64_t da = smem_desc_sw128(sa + h * (BM * BK * 2));
#pragma unroll
                        for (int k = 0; k < BK / UMMA_K; ++k) {
                            // 16 bf16 = 32 bytes further along K inside the swizzle atom.
                            umma_bf16(d, da + (k * UMMA_K * 2 >> 4), db + (k * UMMA_K * 2 >> 4), idesc,
                                      (kb | k) != 0);
                        }
                    }
                    umma_commit(&st.empty[stage]);  // stage reusable once these MMAs read it
                    if (++stage == kStagesG) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
#pragma unroll
                for (int h = 0; h < HALVES; ++h)
                    umma_commit(&st.tmem_full[slot_of(it, h)]);  // accumulators complete
            }
        }
    } else {
        // ---------------- epilogue (warps 2..5) ----------------
        const int quarter = warp & 3;  // TMEM lanes 32*quarter .. +31
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
            for (int h = 0; h < HALVES; ++h) {
                const int slot = slot_of(it, h);
                if constexpr (Policy::kBackground) {
                    // While the accumulator is not ready the four warps run the policy's
                    // background items (communication).  One thread polls; the decision is
                    // shared through a named barrier because an item contains barriers.
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
                    st.abort = 1;
                    set_status(status, aboleth::Status::Timeout, 0x3400 + slot);
                    break;
                }
                tc_fence_after();
                const std::uint32_t taddr = tmem_base + (static_cast<std::uint32_t>(quarter * 32) << 16) +
                                            slot * BN;
                drain_rows32(policy, t, taddr, h * BM + quarter * 32, epi_stage, lane);
                tc_fence_before();
                __syncwarp();
                if (lane == 0)
                    mbar_arrive(&st.tmem_empty[slot]);
            }
            // Tile-complete hooks: they need all four epilogue warps' stores.  The accumulator
            // is already released, so whatever `drained` does overlaps the next main loop.
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
        // Let TMA copies that are still in flight land before the CTA's shared
        // memory is handed to another CTA.
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

// ---- host: tensor maps ---------------------------------------------------------------------

using EncodeTiledFn = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *,
                                   const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                                   const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_tiled() {
    static EncodeTiledFn fn = nullptr;
    if (fn == nullptr) {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess)
            return nullptr;
        fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    return fn;
}

// bf16 [rows, cols] row-major with `ld` elements between rows; box = box_rows x 64 columns.
inline bool make_map_bf16(CUtensorMap *map, const void *base, std::uint64_t rows, std::uint64_t cols,
                          std::uint64_t ld, unsigned box_rows) {
    EncodeTiledFn fn = encode_tiled();
    if (fn == nullptr)
        return false;
    const cuuint64_t dims[2] = {cols, rows};
    const cuuint64_t strides[1] = {ld * 2};
    const cuuint32_t box[2] = {static_cast<cuuint32_t>(BK), box_rows};
    const cuuint32_t elem[2] = {1, 1};
    const CUresult rc = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void *>(base), dims,
                           strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                           CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (rc != CUDA_SUCCESS)
        fprintf(stderr, "aboleth_b200: cuTensorMapEncodeTiled failed with CUresult %d\n", static_cast<int>(rc));
    return rc == CUDA_SUCCESS;
}

// e4m3 [rows, cols] row-major with `ld` bytes between rows; box = box_rows x 128 columns.
inline bool make_map_e4m3(CUtensorMap *map, const void *base, std::uint64_t rows, std::uint64_t cols,
                          std::uint64_t ld, unsigned box_rows) {
    EncodeTiledFn fn = encode_tiled();
    if (fn == nullptr)
        return false;
    const cuuint64_t dims[2] = {cols, rows};
    const cuuint64_t strides[1] = {ld};
    const cuuint32_t box[2] = {128u, box_rows};
    const cuuint32_t elem[2] = {1, 1};
    const CUresult rc = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(base), dims, strides, box,
                           elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                           CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (rc != CUDA_SUCCESS)
        fprintf(stderr, "aboleth_b200: cuTensorMapEncodeTiled failed with CUresult %d\n", static_cast<int>(rc));
    return rc == CUDA_SUCCESS;
}

// Convert 32 fp32 to bf16 and store 64 contiguous bytes (row-major C).
__device__ __forceinline__ void store_row32_bf16(__nv_bfloat16 *dst, const float (&v)[32],
                                                 int cols_left) {
    if (cols_left >= 32 && (reinterpret_cast<std::uintptr_t>(dst) & 15) == 0) {
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            uint4 o;
            __nv_bfloat162 p0 = __floats2bfloat162_rn(v[q * 8 + 0], v[q * 8 + 1]);
            __nv_bfloat162 p1 = __floats2bfloat162_rn(v[q * 8 + 2], v[q * 8 + 3]);
            __nv_bfloat162 p2 = __floats2bfloat162_rn(v[q * 8 + 4], v[q * 8 + 5]);
            __nv_bfloat162 p3 = __floats2bfloat162_rn(v[q * 8 + 6], v[q * 8 + 7]);
            o.x = *reinterpret_cast<std::uint32_t *>(&p0);
            o.y = *reinterpret_cast<std::uint32_t *>(&p1);
            o.z = *reinterpret_cast<std::uint32_t *>(&p2);
            o.w = *reinterpret_cast<std::uint32_t *>(&p3);
            *reinterpret_cast<uint4 *>(dst + q * 8) = o;
        }
    } else {
#pragma unroll
        for (int i = 0; i < 32; ++i)
            if (i < cols_left)
                dst[i] = __float2bfloat16_rn(v[i]);
    }
}

}  // namespace ab::gemm
