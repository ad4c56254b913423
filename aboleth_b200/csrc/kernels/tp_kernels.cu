// Tensor-parallel GEMMs fused with their collective, one launch each.
//
// ALL-GATHER -> GEMM   C[world*Ml, Nl] = gather_ranks(A_local[Ml, K]) * B_local[Nl, K]^T
//   The four epilogue warps of every CTA store the CTA's share of this rank's A shard
//   into every peer's gathered-A staging over NVLink, in 64 KiB items, whenever they
//   would otherwise wait for an accumulator - so the push runs under the tensor-core
//   main loop of the rank's own rows.  The item that completes a 256-row chunk for a
//   peer publishes it with one release flag.  The TMA producer of a tile whose rows came from rank s waits
//   (bounded) on the chunk's flag and then loads the tile from LOCAL staging -
//   a remote tile crosses NVLink once and TMA never touches peer memory.  Tiles of the
//   rank's own rows read A_local through a second tensor map and start at once; remote
//   sources follow in arrival order.  When the staging buffers of all ranks are bound to one
//   NVLink multicast object the push uses `multimem.st` instead: one store per 16 bytes
//   is replicated by NVSwitch into every rank's staging, so the shard leaves the GPU once
//   instead of world - 1 times (the flags stay one release store per receiver).
//
// GEMM -> REDUCE-SCATTER   out[Ml, N] = sum_ranks(A_local[world*Ml, Kl] * B_local[N, Kl]^T)[own rows]
//   The epilogue converts each fp32 accumulator tile from TMEM to bf16 into a per-CTA
//   staging tile in local memory (L2-resident) and releases the accumulator; while the
//   next tile's main loop runs, the same four warps copy the staged tile into the OWNER
//   rank's partial buffer with row-contiguous 512-byte peer stores and publish it with
//   one release flag.  (Storing straight from the TMEM registers - 16 bytes per lane,
//   every lane another row - reached a quarter of the link rate and stalled the
//   accumulator.)  Every rank computes tile j of all owners before tile j + 1 of any, so
//   an owner's tile is complete on all ranks early; whenever the epilogue warps would wait
//   for an accumulator they reduce the next owned tile whose partials have all arrived
//   (fp32 sum), and after the last GEMM tile they finish the rest with bounded waits.
//
// No reference kernel exists for these; the baseline is NCCL all-gather /
// reduce-scatter around a library GEMM.
#include <algorithm>
#include <cstdlib>

#include "gemm_mx_sm100.cuh"

namespace {

using namespace ab::gemm;
using aboleth::Status;

constexpr int kHalves = 2;          // 256-row tiles
constexpr int kRows = BM * kHalves;  // rows per chunk / tile
constexpr unsigned kSmem = Geometry<kHalves>::kSmemBytes;

// Position `pos` inside one rank's block of chunks x tiles_n tiles -> (chunk, tile column): all
// chunks of `group_n` tile columns before the next group, column fastest, so the B panels of a group
// (group_n * 256 * K * 2 bytes, about 48 MiB) stay in L2 while the A rows stream past them.
__device__ __forceinline__ void raster(int pos, int chunks, int tiles_n, int group_n, int &chunk, int &tn) {
    const int per_group = group_n * chunks;
    const int group = pos / per_group;
    const int width = min(group_n, tiles_n - group * group_n);
    const int in_group = pos - group * per_group;
    chunk = in_group / width;
    tn = group * group_n + (in_group - chunk * width);
}

constexpr int kPhaseProduce = 1;  // AG: push shard.  RS: GEMM + partial stores.
constexpr int kPhaseConsume = 2;  // AG: GEMM.        RS: reduction of owned tiles.

// ---- all-gather -> GEMM -----------------------------------------------------------------

// COLS: tile width; ESIZE: bytes per A element (2 = bf16; 1 = e4m3 with scale-factor atoms that
// travel with the rows); KBLK: K elements per main-loop stage.
template <int COLS, int ESIZE, int KBLK>
struct AgGemmPolicyT {
    static constexpr bool kBackground = true, kDrainedHook = false, kScaled = false;
    __nv_bfloat16 *c;
    const std::uint64_t *flags;       // local: [world * chunks] epochs
    unsigned long long *status;
    std::uint64_t epoch;
    int rank, world, m_local, n, k, ldc, phases;
    int tiles_n, chunks;              // chunks = m_local / 256 (row blocks per rank)
    int group_n;                      // tile columns per raster group
    // push of this rank's shard (background work of the epilogue warps)
    const std::uint8_t *a_local;          // [m_local, k] bf16
    const std::uint64_t *peer_staging;    // [world] address of each peer's gathered-A buffer
    const std::uint64_t *peer_flags;      // [world] address of each peer's flag array
    unsigned *arrivals;                   // local scratch [world * chunks], zero between calls
    int parts;                            // items that share one (peer, chunk)
    int pushed;                           // items this CTA has pushed so far (same in every thread)
    // e4m3 only: this rank's packed scale factors ([m_local / 128][K / 128] atoms) and where the
    // gathered atoms start inside a staging buffer (behind the gathered rows).
    const std::uint8_t *sfa_local = nullptr;
    std::size_t staging_sfa_offset = 0;
    // Multicast address of the staging buffers (0 = none): one multimem store per 16 bytes reaches every
    // peer's staging through NVSwitch, so the shard leaves this GPU once instead of world - 1 times.
    std::uint64_t mc_staging = 0;

    __device__ __forceinline__ bool next(int it, Tile &t) const {
        if (!(phases & kPhaseConsume))
            return false;
        const int idx = blockIdx.x + it * gridDim.x;
        const int per_src = chunks * tiles_n;
        if (idx >= world * per_src)
            return false;
        // Source order: own rows first, then rank-1, rank-2, ... (the order in which
        // peers' pushes arrive, since every rank pushes to rank+1 first).  A multicast push serves all
        // peers chunk by chunk instead, so there the remote tiles are walked chunk-major: chunk 0 of
        // every source, then chunk 1 of every source, ...
        int order, chunk, tn;
        if (mc_staging != 0 && idx >= per_src) {
            const int remote = idx - per_src, per_chunk = (world - 1) * tiles_n;
            chunk = remote / per_chunk;
            const int in_chunk = remote - chunk * per_chunk;
            order = in_chunk / tiles_n + 1;
            tn = in_chunk - (order - 1) * tiles_n;
        } else {
            order = idx / per_src;
            raster(idx - order * per_src, chunks, tiles_n, group_n, chunk, tn);
        }
        const int src = (rank - order + world) % world;
        t.a_sel = src == rank ? 1 : 0;
        t.a_row = src == rank ? chunk * kRows : src * m_local + chunk * kRows;
        t.b_row = tn * COLS;
        t.k_blocks = (k + KBLK - 1) / KBLK;
        t.c_row = src * m_local + chunk * kRows;
        t.c_col = tn * COLS;
        t.rows_valid = min(kRows, m_local - chunk * kRows);
        t.cols_valid = min(COLS, n - tn * COLS);
        t.tag = src * chunks + chunk;
        return true;
    }
    __device__ __forceinline__ bool ready(const Tile &t) const {
        if (t.a_sel)
            return true;
        if (aboleth::wait_signal_status(flags + t.tag, epoch) != Status::Ok)
            return false;
        // The chunk was written by peers with generic-proxy stores; the loads that follow are TMA
        // (async proxy).  The acquire orders the generic side, this fence carries it across.
        ab::fence_proxy_async();
        return true;
    }
    __device__ __forceinline__ void store16(const Tile &t, int row, int col, const uint4 &v) const {
        *reinterpret_cast<uint4 *>(c + static_cast<std::size_t>(t.c_row + row) * ldc + t.c_col + col) = v;
    }
    __device__ __forceinline__ void tile_done(const Tile &) const {}
    __device__ __forceinline__ void finish(int, int, unsigned long long *) const {}

    // One push item = (peer, chunk, part), nearest peer first; the item that arrives last on
    // (peer, chunk) publishes the chunk.  With a multicast mapping an item is (chunk, part): its
    // stores reach every peer at once and the last part publishes the chunk to each peer in turn.
    // Called by the 128 epilogue threads together.
    __device__ __forceinline__ bool background(int thread, int nthreads) {
        if (!(phases & kPhaseProduce))
            return false;
        const bool multicast = mc_staging != 0;
        const int item = blockIdx.x + pushed * gridDim.x;
        if (item >= (multicast ? 1 : world - 1) * chunks * parts)
            return false;
        ++pushed;
        const std::size_t row_bytes = static_cast<std::size_t>(k) * ESIZE;
        const int part = item % parts;
        const int pc = item / parts;
        const int hop = pc / chunks + 1, chunk = pc - (hop - 1) * chunks;
        const int peer = (rank + hop) % world;     // unicast only
        const int rows = min(kRows, m_local - chunk * kRows);
        const int per = (rows + parts - 1) / parts;
        const int r0 = min(part * per, rows), r1 = min(r0 + per, rows);
        const std::size_t offset = (static_cast<std::size_t>(chunk) * kRows + r0) * row_bytes;
        const std::size_t shard = static_cast<std::size_t>(rank) * m_local * row_bytes;
        std::uint8_t *base = reinterpret_cast<std::uint8_t *>(multicast ? mc_staging : peer_staging[peer]);
        if (multicast)
            aboleth::detail::copy_strided_multicast(base + shard + offset, a_local + offset, (r1 - r0) * row_bytes,
                                                    thread, nthreads);
        else
            aboleth::detail::copy_strided(base + shard + offset, a_local + offset, (r1 - r0) * row_bytes, thread,
                                          nthreads);
        if constexpr (ESIZE == 1) {
            if (part == 0) {  // the chunk's scale factors: two row blocks of K / 128 atoms
                const std::size_t chunk_sf = static_cast<std::size_t>(kRows / BM) * (k / KBLK) * mx::kAtomBytes;
                std::uint8_t *sf_dst = base + staging_sfa_offset +
                                       (static_cast<std::size_t>(rank) * chunks + chunk) * chunk_sf;
                if (multicast)
                    aboleth::detail::copy_strided_multicast(sf_dst, sfa_local + chunk * chunk_sf, chunk_sf, thread,
                                                            nthreads);
                else
                    aboleth::detail::copy_strided(sf_dst, sfa_local + chunk * chunk_sf, chunk_sf, thread, nthreads);
            }
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (thread == 0) {
            aboleth::detail::fence_acq_rel_sys();
            unsigned *counter = arrivals + (multicast ? 0 : peer) * chunks + chunk;
            if (atomicAdd(counter, 1u) == static_cast<unsigned>(parts) - 1) {
                *counter = 0;  // self-cleaning
                aboleth::detail::fence_acq_rel_sys();
                for (int p = multicast ? 0 : peer; p < (multicast ? world : peer + 1); ++p) {
                    if (p == rank)
                        continue;
                    std::uint64_t *flag = reinterpret_cast<std::uint64_t *>(peer_flags[p]) + rank * chunks + chunk;
                    aboleth::detail::st_release_sys(flag, epoch);
                }
            }
        }
        return true;
    }
};

using AgGemmPolicy = AgGemmPolicyT<BN, 2, BK>;
using AgGemmMxPolicy = AgGemmPolicyT<mx::MxGeometry<kHalves>::kCols, 1, mx::kBlockK>;

__global__ void __launch_bounds__(kThreads, 1)
ag_gemm_kernel(const __grid_constant__ CUtensorMap map_staging,
               const __grid_constant__ CUtensorMap map_b,
               const __grid_constant__ CUtensorMap map_local, AgGemmPolicy params) {
    AgGemmPolicy policy = params;
    gemm_mainloop<kHalves>(policy, &map_staging, &map_b, policy.status, &map_local);
}

// The same schedule on block-scaled e4m3 operands (tcgen05.mma.kind::mxf8f6f4.block_scale): half the
// bytes cross NVLink and the product runs at the fp8 rate.
__global__ void __launch_bounds__(kThreads, 1)
ag_gemm_mx_kernel(const __grid_constant__ CUtensorMap map_staging,
                  const __grid_constant__ CUtensorMap map_b,
                  const __grid_constant__ CUtensorMap map_local, AgGemmMxPolicy params, mx::ScaleFactors sf) {
    AgGemmMxPolicy policy = params;
    mx::gemm_mx_mainloop<kHalves>(policy, &map_staging, &map_b, sf, policy.status, &map_local);
}

// ---- GEMM -> reduce-scatter -----------------------------------------------------------------

template <int COLS, int KBLK>
struct GemmRsPolicyT {
    static constexpr bool kBackground = true, kDrainedHook = true, kScaled = false;
    const std::uint64_t *peer_partials;  // [world] address of each rank's partial buffer
    const std::uint64_t *peer_flags;     // [world] address of each rank's flag array
    const __nv_bfloat16 *partials;       // local: [world, m_local, n]
    const std::uint64_t *flags;          // local: [world * tiles_local]
    __nv_bfloat16 *out;                  // [m_local, n]
    __nv_bfloat16 *stage;                // local: [gridDim.x, 256, 256] staging tiles
    unsigned long long *status;
    std::uint64_t epoch;
    int rank, world, m_local, n, k, phases;
    int tiles_n, chunks;                 // tiles per owner = chunks * tiles_n
    int group_n;                         // tile columns per raster group
    int interleave;                      // 1: owners interleaved tile by tile, owned tiles reduced in the background
    int reduced;                         // owned tiles this CTA has reduced so far (same in every thread)
    static constexpr int kSourcesInFlight = 8;

    __device__ __forceinline__ bool next(int it, Tile &t) const {
        if (!(phases & kPhaseProduce))
            return false;
        const int idx = blockIdx.x + it * gridDim.x;
        const int per_owner = chunks * tiles_n;
        if (idx >= world * per_owner)
            return false;
        // Owners in the order rank+1, rank+2, ..., rank.  Interleaved: tile j of every owner before tile
        // j + 1 of any owner, so all partials of an owner's tile j exist after about (j + 1) * world tile
        // times everywhere and the owner reduces it while the GEMM is still running; this pays when an
        // owner has several tiles per CTA to reduce.  Otherwise owner by owner: the last wave computes
        // own tiles, which need no transfer, and the reduction follows it.
        int position, order;
        if (interleave) {
            position = idx / world;
            order = idx - position * world;
        } else {
            order = idx / per_owner;
            position = idx - order * per_owner;
        }
        const int owner = (rank + 1 + order) % world;
        int chunk, tn;
        raster(position, chunks, tiles_n, group_n, chunk, tn);
        const int local = chunk * tiles_n + tn;
        t.a_sel = 0;
        t.a_row = owner * m_local + chunk * kRows;
        t.b_row = tn * COLS;
        t.k_blocks = (k + KBLK - 1) / KBLK;
        t.c_row = chunk * kRows;  // row inside the owner's block
        t.c_col = tn * COLS;
        t.rows_valid = min(kRows, m_local - chunk * kRows);
        t.cols_valid = min(COLS, n - tn * COLS);
        t.tag = owner * 65536 + local;  // owner and tile index inside the owner's block
        return true;
    }
    __device__ __forceinline__ bool ready(const Tile &) const { return true; }
    __device__ __forceinline__ void store16(const Tile &t, int row, int col, const uint4 &v) const {
        const int owner = t.tag >> 16;
        if (owner == rank) {  // own tile: straight into this rank's slot of the local partials
            __nv_bfloat16 *base = const_cast<__nv_bfloat16 *>(partials) +
                                  static_cast<std::size_t>(rank) * m_local * n;
            *reinterpret_cast<uint4 *>(base + static_cast<std::size_t>(t.c_row + row) * n + t.c_col + col) = v;
        } else {
            *reinterpret_cast<uint4 *>(stage + static_cast<std::size_t>(blockIdx.x) * (kRows * COLS) + row * COLS +
                                       col) = v;
        }
    }
    // The accumulator is free again: copy the staged tile to its owner, one 512-byte row per
    // warp instruction, eight rows' worth of loads in flight per thread.
    __device__ __forceinline__ void drained(const Tile &t, int thread, int nthreads) const {
        const int owner = t.tag >> 16;
        if (owner == rank)
            return;
        const __nv_bfloat16 *src = stage + static_cast<std::size_t>(blockIdx.x) * (kRows * COLS);
        __nv_bfloat16 *dst = reinterpret_cast<__nv_bfloat16 *>(peer_partials[owner]) +
                             static_cast<std::size_t>(rank) * m_local * n +
                             static_cast<std::size_t>(t.c_row) * n + t.c_col;
        const int vpr = t.cols_valid / 8;  // 16-byte vectors per row
        const int total = t.rows_valid * vpr;
        constexpr int kInFlight = 8;
        for (int i0 = thread; i0 < total; i0 += kInFlight * nthreads) {
            uint4 v[kInFlight];
#pragma unroll
            for (int u = 0; u < kInFlight; ++u) {
                const int i = i0 + u * nthreads;
                if (i < total) {
                    const int r = i / vpr, c = i - r * vpr;
                    v[u] = aboleth::detail::ld_stream16(src + r * COLS + c * 8);
                }
            }
#pragma unroll
            for (int u = 0; u < kInFlight; ++u) {
                const int i = i0 + u * nthreads;
                if (i < total) {
                    const int r = i / vpr, c = i - r * vpr;
                    aboleth::detail::st_stream16(dst + static_cast<std::size_t>(r) * n + c * 8, v[u]);
                }
            }
        }
    }
    // One thread, after all four epilogue warps stored the tile (bar.sync): publish it.
    __device__ __forceinline__ void tile_done(const Tile &t) const {
        const int owner = t.tag >> 16, local = t.tag & 0xffff;
        std::uint64_t *flag = reinterpret_cast<std::uint64_t *>(peer_flags[owner]) +
                              rank * (chunks * tiles_n) + local;
        aboleth::detail::fence_acq_rel_sys();
        aboleth::detail::st_relaxed_sys(flag, epoch);
    }
    // Sum the partials of owned tile `tile` over the ranks (fp32) into `out`.  All 128 epilogue threads.
    __device__ __forceinline__ void reduce_tile(int tile, int thread, int nthreads) const {
        const int chunk = tile / tiles_n, tn = tile - chunk * tiles_n;
        const int rows = min(kRows, m_local - chunk * kRows), cols = min(COLS, n - tn * COLS);
        const int vec_per_row = cols / 8;
        for (int i = thread; i < rows * vec_per_row; i += 2 * nthreads) {
            const int i2 = i + nthreads;
            const bool two = i2 < rows * vec_per_row;
            const int ra = i / vec_per_row, va = i - ra * vec_per_row;
            const int rb = two ? i2 / vec_per_row : ra, vb = two ? i2 - rb * vec_per_row : va;
            const std::size_t offa = static_cast<std::size_t>(chunk * kRows + ra) * n + tn * COLS + va * 8;
            const std::size_t offb = static_cast<std::size_t>(chunk * kRows + rb) * n + tn * COLS + vb * 8;
            float acc[2][8] = {};
            // Up to eight sources' vectors are loaded before any is added: sixteen 16-byte loads in
            // flight per thread instead of two.
            for (int s0 = 0; s0 < world; s0 += kSourcesInFlight) {
                uint4 y[kSourcesInFlight][2];
#pragma unroll
                for (int j = 0; j < kSourcesInFlight; ++j) {
                    if (s0 + j < world) {
                        const __nv_bfloat16 *base = partials + static_cast<std::size_t>(s0 + j) * m_local * n;
                        y[j][0] = aboleth::detail::ld_stream16(base + offa);
                        y[j][1] = aboleth::detail::ld_stream16(base + offb);
                    }
                }
#pragma unroll
                for (int j = 0; j < kSourcesInFlight; ++j) {
                    if (s0 + j < world) {
                        const std::uint32_t wa[4] = {y[j][0].x, y[j][0].y, y[j][0].z, y[j][0].w};
                        const std::uint32_t wb[4] = {y[j][1].x, y[j][1].y, y[j][1].z, y[j][1].w};
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            acc[0][2 * q] += __uint_as_float(wa[q] << 16);
                            acc[0][2 * q + 1] += __uint_as_float(wa[q] & 0xffff0000u);
                            acc[1][2 * q] += __uint_as_float(wb[q] << 16);
                            acc[1][2 * q + 1] += __uint_as_float(wb[q] & 0xffff0000u);
                        }
                    }
                }
            }
#pragma unroll
            for (int u = 0; u < 2; ++u) {
                if (u == 1 && !two)
                    break;
                *reinterpret_cast<uint4 *>(out + (u ? offb : offa)) = pack8_bf16(acc[u]);
            }
        }
    }

    // Background work of the epilogue warps: reduce the next owned tile if every rank's partial of it
    // has already arrived (checked without waiting).  Returns false when there is nothing to do now.
    __device__ __forceinline__ bool background(int thread, int nthreads) {
        if (!(phases & kPhaseConsume) || !interleave)
            return false;
        const int per_owner = chunks * tiles_n;
        const int position = blockIdx.x + reduced * gridDim.x;  // owned tiles in the order they are computed
        if (position >= per_owner)
            return false;
        int chunk, tn;
        raster(position, chunks, tiles_n, group_n, chunk, tn);
        const int tile = chunk * tiles_n + tn;
        __shared__ int missing;
        if (thread == 0)
            missing = 0;
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (thread < world &&
            aboleth::detail::ld_acquire_sys(flags + thread * per_owner + tile) < epoch)
            missing = 1;
        asm volatile("bar.sync 1, 128;" ::: "memory");
        const bool arrived = missing == 0;
        asm volatile("bar.sync 1, 128;" ::: "memory");  // `missing` is rewritten by the next call
        if (!arrived)
            return false;
        reduce_tile(tile, thread, nthreads);
        ++reduced;
        return true;
    }

    // After the last GEMM tile: the owned tiles that were not reduced in the background, with
    // (bounded) waits for the partials that are still on their way.
    __device__ __forceinline__ void finish(int thread, int nthreads, unsigned long long *st) {
        if (!(phases & kPhaseConsume))
            return;
        const int per_owner = chunks * tiles_n;
        for (int position = blockIdx.x + reduced * gridDim.x; position < per_owner; position += gridDim.x) {
            int chunk, tn;
            raster(position, chunks, tiles_n, group_n, chunk, tn);
            const int tile = chunk * tiles_n + tn;
            // Threads 0..world-1 wait for one source each; the named barrier publishes it.
            bool ok = true;
            if (thread < world)
                ok = aboleth::wait_signal_status(flags + thread * per_owner + tile, epoch) == Status::Ok;
            if (!ok)
                ab::set_status(st, Status::Timeout, 0x4000 + thread);
            asm volatile("bar.sync 1, 128;" ::: "memory");
            reduce_tile(tile, thread, nthreads);
            asm volatile("bar.sync 1, 128;" ::: "memory");
        }
    }
};

using GemmRsPolicy = GemmRsPolicyT<BN, BK>;
using GemmRsMxPolicy = GemmRsPolicyT<mx::MxGeometry<kHalves>::kCols, mx::kBlockK>;

__global__ void __launch_bounds__(kThreads, 1)
gemm_rs_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
               GemmRsPolicy params) {
    GemmRsPolicy policy = params;
    gemm_mainloop<kHalves>(policy, &map_a, &map_b, policy.status);
}

__global__ void __launch_bounds__(kThreads, 1)
gemm_rs_mx_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                  GemmRsMxPolicy params, mx::ScaleFactors sf) {
    GemmRsMxPolicy policy = params;
    mx::gemm_mx_mainloop<kHalves>(policy, &map_a, &map_b, sf, policy.status);
}

// Tile columns whose B panels (`cols` rows of K elements of `esize` bytes each) add up to about 48 MiB.
int raster_group(int n, int k, int cols = BN, int esize = 2) {
    const long long column_bytes = static_cast<long long>(cols) * k * esize;
    const long long tiles_n = (n + cols - 1) / cols;
    return static_cast<int>(std::max(1LL, std::min(tiles_n, (48LL << 20) / column_bytes)));
}

int sm_count() {
    static int sms = 0;
    if (sms == 0) {
        int device = 0;
        cudaGetDevice(&device);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
    }
    return sms;
}

}  // namespace

// a_local [m_local, k]; staging [world*m_local, k] (this rank's gathered-A buffer, peers write it);
// b [n, k]; c [world*m_local, n].  m_local must be a multiple of 256.  peer_staging / peer_flags:
// device int64 [world] address tables; flags: local int64 [world * m_local/256].  mc_staging: the
// multicast address of the ranks' staging buffers (all bound at the same offset of one NVLink
// multicast object), or 0 to push with one peer store per receiver.
AB_EXPORT int ab_ag_gemm_bf16(const void *a_local, const void *staging, const void *b, void *c,
                              const std::uint64_t *peer_staging, const std::uint64_t *peer_flags,
                              const std::uint64_t *flags, unsigned long long *status,
                              unsigned *arrivals, std::uint64_t epoch, int rank, int world, int m_local,
                              int n, int k, int parts, int phases, std::uint64_t mc_staging,
                              cudaStream_t stream) {
    if (world < 1 || m_local < kRows || m_local % kRows || n < 8 || n % 8 || k < 8 || k % 8 || rank < 0 ||
        rank >= world || (mc_staging & 15))
        return -1;
    CUtensorMap map_staging, map_b, map_local;
    if (!make_map_bf16(&map_staging, staging, static_cast<std::uint64_t>(world) * m_local, k, k, kRows) ||
        !make_map_bf16(&map_b, b, n, k, k, BN) || !make_map_bf16(&map_local, a_local, m_local, k, k, kRows))
        return -2;
    // The attribute belongs to the current device's context, so it is set on every call (cheap)
    // rather than remembered once per process.
    if (cudaFuncSetAttribute(ag_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem) != cudaSuccess)
        return -3;
    const int chunks = m_local / kRows;
    if (parts < 1) {  // items of about 64 KiB: short enough to slot in between accumulator polls
        const long long chunk_bytes = static_cast<long long>(kRows) * k * 2;
        parts = static_cast<int>(std::min<long long>(kRows, std::max<long long>(1, chunk_bytes / 65536)));
    }
    parts = std::min(parts, kRows);
    AgGemmPolicy p{static_cast<__nv_bfloat16 *>(c), flags, status, epoch, rank, world, m_local, n, k, n,
                   phases, (n + BN - 1) / BN, chunks, raster_group(n, k),
                   static_cast<const std::uint8_t *>(a_local), peer_staging, peer_flags, arrivals, parts, 0};
    p.mc_staging = mc_staging;
    ag_gemm_kernel<<<sm_count(), kThreads, kSmem, stream>>>(map_staging, map_b, map_local, p);
    return ab::launch_result("ag_gemm_bf16");
}

// Block-scaled e4m3 form of ab_ag_gemm_bf16.  a_local [m_local, k] e4m3 with its packed scale factors
// `sfa_local` (ab_mx_pack_scales: m_local / 128 row blocks of k / 128 atoms); b [n, k] e4m3 with packed
// `sfb`.  staging holds the gathered rows [world*m_local, k] followed by the gathered atoms
// [world * m_local / 128][k / 128][512]: ab_ag_gemm_mx_staging_bytes() bytes.  k a multiple of 128.
AB_EXPORT long long ab_ag_gemm_mx_staging_bytes(int world, int m_local, int k) {
    const long long rows = static_cast<long long>(world) * m_local;
    return rows * k + rows / BM * (k / 128) * mx::kAtomBytes;
}

AB_EXPORT int ab_ag_gemm_e4m3_mx(const void *a_local, const void *sfa_local, const void *staging, const void *b,
                                 const void *sfb, void *c, const std::uint64_t *peer_staging,
                                 const std::uint64_t *peer_flags, const std::uint64_t *flags,
                                 unsigned long long *status, unsigned *arrivals, std::uint64_t epoch, int rank,
                                 int world, int m_local, int n, int k, int parts, int phases,
                                 std::uint64_t mc_staging, cudaStream_t stream) {
    if (world < 1 || m_local < kRows || m_local % kRows || n < 8 || n % 8 || k < 128 || k % 128 || rank < 0 ||
        rank >= world || sfa_local == nullptr || sfb == nullptr || (mc_staging & 15))
        return -1;
    constexpr int kCols = mx::MxGeometry<kHalves>::kCols;
    constexpr unsigned smem = mx::MxGeometry<kHalves>::kSmemBytes;
    CUtensorMap map_staging, map_b, map_local;
    if (!make_map_e4m3(&map_staging, staging, static_cast<std::uint64_t>(world) * m_local, k, k, kRows) ||
        !make_map_e4m3(&map_b, b, n, k, k, kCols) || !make_map_e4m3(&map_local, a_local, m_local, k, k, kRows))
        return -2;
    if (cudaFuncSetAttribute(ag_gemm_mx_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
        return -3;
    const int chunks = m_local / kRows;
    if (parts < 1) {
        const long long chunk_bytes = static_cast<long long>(kRows) * k;
        parts = static_cast<int>(std::min<long long>(kRows, std::max<long long>(1, chunk_bytes / 65536)));
    }
    parts = std::min(parts, kRows);
    AgGemmMxPolicy p{static_cast<__nv_bfloat16 *>(c), flags, status, epoch, rank, world, m_local, n, k, n,
                     phases, (n + kCols - 1) / kCols, chunks, raster_group(n, k, kCols, 1),
                     static_cast<const std::uint8_t *>(a_local), peer_staging, peer_flags, arrivals, parts, 0,
                     static_cast<const std::uint8_t *>(sfa_local),
                     static_cast<std::size_t>(world) * m_local * k, mc_staging};
    const mx::ScaleFactors sf{static_cast<const std::uint8_t *>(staging) + p.staging_sfa_offset,
                              static_cast<const std::uint8_t *>(sfb), k / 128, mx::mx_granules(n),
                              static_cast<const std::uint8_t *>(sfa_local)};
    ag_gemm_mx_kernel<<<sm_count(), kThreads, smem, stream>>>(map_staging, map_b, map_local, p, sf);
    return ab::launch_result("ag_gemm_e4m3_mx");
}

// a [world*m_local, k_local]; b [n, k_local]; partials: local [world, m_local, n] (peers write it);
// out [m_local, n]; stage: local scratch of ab_gemm_rs_stage_bytes() bytes (staging tiles, one per CTA).
// m_local multiple of 256, n multiple of 8 and tiles per owner < 65536.
AB_EXPORT long long ab_gemm_rs_stage_bytes() {
    return static_cast<long long>(sm_count()) * kRows * BN * 2;
}

// Tiles per owner of the block-scaled form (192-column tiles): the flag arrays hold world times as many.
AB_EXPORT int ab_gemm_rs_mx_tiles(int m_local, int n) {
    constexpr int kCols = mx::MxGeometry<kHalves>::kCols;
    return (m_local / kRows) * ((n + kCols - 1) / kCols);
}

// Block-scaled e4m3 form of ab_gemm_rs_bf16: a [world*m_local, k_local] and b [n, k_local] are e4m3 with
// packed scale factors `sfa` / `sfb` (ab_mx_pack_scales); partials, out and stage as in the bf16 form;
// flags hold world * ab_gemm_rs_mx_tiles() entries.  k_local a multiple of 128.
AB_EXPORT int ab_gemm_rs_e4m3_mx(const void *a, const void *sfa, const void *b, const void *sfb,
                                 const void *partials, void *out, void *stage,
                                 const std::uint64_t *peer_partials, const std::uint64_t *peer_flags,
                                 const std::uint64_t *flags, unsigned long long *status, std::uint64_t epoch,
                                 int rank, int world, int m_local, int n, int k, int phases,
                                 cudaStream_t stream) {
    if (world < 1 || m_local < kRows || m_local % kRows || n < 8 || n % 8 || k < 128 || k % 128 || rank < 0 ||
        rank >= world || stage == nullptr || sfa == nullptr || sfb == nullptr)
        return -1;
    constexpr int kCols = mx::MxGeometry<kHalves>::kCols;
    constexpr unsigned smem = mx::MxGeometry<kHalves>::kSmemBytes;
    const int tiles_n = (n + kCols - 1) / kCols, chunks = m_local / kRows;
    if (tiles_n * chunks >= 65536)
        return -1;
    CUtensorMap map_a, map_b;
    if (!make_map_e4m3(&map_a, a, static_cast<std::uint64_t>(world) * m_local, k, k, kRows) ||
        !make_map_e4m3(&map_b, b, n, k, k, kCols))
        return -2;
    if (cudaFuncSetAttribute(gemm_rs_mx_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
        return -3;
    int interleave = tiles_n * chunks >= 2 * sm_count() ? 1 : 0;
    if (const char *forced = std::getenv("ABOLETH_RS_ORDER"))
        interleave = forced[0] == '1' ? 1 : 0;
    GemmRsMxPolicy p{peer_partials, peer_flags, static_cast<const __nv_bfloat16 *>(partials), flags,
                     static_cast<__nv_bfloat16 *>(out), static_cast<__nv_bfloat16 *>(stage), status, epoch, rank,
                     world, m_local, n, k, phases, tiles_n, chunks, raster_group(n, k, kCols, 1), interleave, 0};
    const mx::ScaleFactors sf{static_cast<const std::uint8_t *>(sfa), static_cast<const std::uint8_t *>(sfb),
                              k / 128, mx::mx_granules(n)};
    gemm_rs_mx_kernel<<<sm_count(), kThreads, smem, stream>>>(map_a, map_b, p, sf);
    return ab::launch_result("gemm_rs_e4m3_mx");
}

AB_EXPORT int ab_gemm_rs_bf16(const void *a, const void *b, const void *partials, void *out, void *stage,
                              const std::uint64_t *peer_partials, const std::uint64_t *peer_flags,
                              const std::uint64_t *flags, unsigned long long *status,
                              std::uint64_t epoch, int rank, int world, int m_local, int n, int k,
                              int phases, cudaStream_t stream) {
    if (world < 1 || m_local < kRows || m_local % kRows || n < 8 || n % 8 || k < 8 || k % 8 || rank < 0 ||
        rank >= world || stage == nullptr)
        return -1;
    const int tiles_n = (n + BN - 1) / BN, chunks = m_local / kRows;
    if (tiles_n * chunks >= 65536)
        return -1;
    CUtensorMap map_a, map_b;
    if (!make_map_bf16(&map_a, a, static_cast<std::uint64_t>(world) * m_local, k, k, kRows) ||
        !make_map_bf16(&map_b, b, n, k, k, BN))
        return -2;
    // The attribute belongs to the current device's context, so it is set on every call (cheap)
    // rather than remembered once per process.
    if (cudaFuncSetAttribute(gemm_rs_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem) != cudaSuccess)
        return -3;
    // Background reduction needs at least two owned tiles per CTA to pay for the transfers it moves
    // into the last wave; ABOLETH_RS_ORDER=0 / 1 forces the owner-by-owner / interleaved order.
    int interleave = tiles_n * chunks >= 2 * sm_count() ? 1 : 0;
    if (const char *forced = std::getenv("ABOLETH_RS_ORDER"))
        interleave = forced[0] == '1' ? 1 : 0;
    GemmRsPolicy p{peer_partials, peer_flags, static_cast<const __nv_bfloat16 *>(partials), flags,
                   static_cast<__nv_bfloat16 *>(out), static_cast<__nv_bfloat16 *>(stage), status, epoch, rank,
                   world, m_local, n, k, phases, tiles_n, chunks, raster_group(n, k), interleave, 0};
    gemm_rs_kernel<<<sm_count(), kThreads, kSmem, stream>>>(map_a, map_b, p);
    return ab::launch_result("gemm_rs_bf16");
}
