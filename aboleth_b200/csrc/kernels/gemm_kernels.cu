// Plain and grouped (per-expert) bf16 GEMM on tcgen05 / TMEM / TMA.
//
//   plain  : C[M, N] = A[M, K] * B[N, K]^T
//   grouped: for each expert e with rows [offsets[e], offsets[e] + counts[e]) of A:
//            C[rows, :] = A[rows, :] * W[e][N, K]^T
//
// The grouped form is the expert stage between EP dispatch and combine: A is
// the expert-contiguous activation matrix the permute kernel builds, counts and
// offsets stay on the device (no host round trip), and a CTA finds its tiles by
// walking the expert list.  The reference has no GEMM; the baseline for these
// kernels is cuBLAS through torch.matmul.
#include <algorithm>
#include <cstdlib>

#include "gemm_mx_sm100.cuh"
#include "gemm_pair_sm100.cuh"

namespace {

using namespace ab::gemm;

constexpr int kPlainHalves = 2;
constexpr int kPlainRows = BM * kPlainHalves;

struct PlainPolicy {
    static constexpr bool kBackground = false, kDrainedHook = false, kScaled = true;
    __nv_bfloat16 *c;
    int m, n, k, ldc;
    int tiles_n, tiles_total;
    int group_n;  // tile columns per raster group: their B panels stay resident in L2
    int pair;     // 1: two CTAs share a tile (worker = CTA pair), 0: one CTA per tile
    int rows;     // rows of C per tile
    int bk;       // elements of K per stage (64 for bf16, 128 for e4m3)
    float alpha;  // factor applied to the accumulator before rounding

    // Tiles are visited group by group: all row tiles of `group_n` tile columns
    // before the next group, column fastest inside a group.  B panels of one group
    // (group_n * 256 * K * 2 bytes) fit the L2, A streams once per group.
    __device__ __forceinline__ bool next(int it, Tile &t) const {
        const int idx = (blockIdx.x >> pair) + it * (gridDim.x >> pair);
        if (idx >= tiles_total)
            return false;
        const int tiles_m = tiles_total / tiles_n;
        const int per_group = group_n * tiles_m;
        const int group = idx / per_group;
        const int width = min(group_n, tiles_n - group * group_n);
        const int local = idx - group * per_group;
        const int tm = local / width, tn = group * group_n + (local - tm * width);
        t.a_row = tm * rows;
        t.b_row = tn * BN;
        t.k_blocks = (k + bk - 1) / bk;
        t.c_row = tm * rows;
        t.c_col = tn * BN;
        t.rows_valid = min(rows, m - tm * rows);
        t.cols_valid = min(BN, n - tn * BN);
        t.tag = 0;
        t.a_sel = 0;
        return true;
    }
    __device__ __forceinline__ bool ready(const Tile &) const { return true; }
    __device__ __forceinline__ void store16(const Tile &t, int row, int col, const uint4 &v) const {
        *reinterpret_cast<uint4 *>(c + static_cast<std::size_t>(t.c_row + row) * ldc + t.c_col + col) = v;
    }
    __device__ __forceinline__ void tile_done(const Tile &) const {}
    __device__ __forceinline__ void finish(int, int, unsigned long long *) const {}
};

template <int HALVES>
struct GroupedPolicy {
    static constexpr int kRows = BM * HALVES;
    static constexpr bool kBackground = false, kDrainedHook = false, kScaled = false;
    __nv_bfloat16 *c;
    const int *counts, *offsets;
    int experts, n, k, ldc, tiles_n;
    int group_n;  // tile columns per raster group (their weight panels stay in L2)
    // cursor (per thread): expert `e` starts at linear tile `base`
    int e, base;

    // Inside one expert the tiles are visited like the plain GEMM's: all row tiles of
    // `group_n` tile columns before the next group, column fastest, so an expert's weight
    // panels are read from DRAM once however many row tiles it has.
    __device__ __forceinline__ bool next(int it, Tile &t) {
        const int idx = blockIdx.x + it * gridDim.x;
        int tiles_m = 0;
        while (e < experts) {
            tiles_m = (counts[e] + kRows - 1) / kRows;
            const int tiles_e = tiles_m * tiles_n;
            if (idx < base + tiles_e)
                break;
            base += tiles_e;
            ++e;
        }
        if (e >= experts)
            return false;
        const int local = idx - base;
        const int per_group = group_n * tiles_m;
        const int group = local / per_group;
        const int width = min(group_n, tiles_n - group * group_n);
        const int in_group = local - group * per_group;
        const int tm = in_group / width, tn = group * group_n + (in_group - tm * width);
        const int row0 = offsets[e] + tm * kRows;
        t.a_row = row0;
        t.b_row = e * n + tn * BN;
        t.k_blocks = (k + BK - 1) / BK;
        t.c_row = row0;
        t.c_col = tn * BN;
        t.rows_valid = min(kRows, counts[e] - tm * kRows);
        t.cols_valid = min(BN, n - tn * BN);
        t.tag = e;
        t.a_sel = 0;
        return true;
    }
    __device__ __forceinline__ bool ready(const Tile &) const { return true; }
    __device__ __forceinline__ void store16(const Tile &t, int row, int col, const uint4 &v) const {
        *reinterpret_cast<uint4 *>(c + static_cast<std::size_t>(t.c_row + row) * ldc + t.c_col + col) = v;
    }
    __device__ __forceinline__ void tile_done(const Tile &) const {}
    __device__ __forceinline__ void finish(int, int, unsigned long long *) const {}
};

template <int HALVES, typename Policy>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a,
                    const __grid_constant__ CUtensorMap map_b, Policy params,
                    unsigned long long *status) {
    Policy policy = params;
    gemm_mainloop<HALVES>(policy, &map_a, &map_b, status);
}

template <int MH, typename Op, typename Policy>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                 Policy params, unsigned long long *status) {
    Policy policy = params;
    pair::gemm_mainloop_pair<MH, Op>(policy, &map_a, &map_b, status);
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

// ABOLETH_GEMM_PAIR: 0 = single-CTA kernels (256 x 256 tile per CTA), 1 = CTA pairs with 256 x 256
// tiles, 2 (default) = CTA pairs with 512 x 256 tiles.
int gemm_pair_mode() {
    static const int mode = [] {
        const char *v = std::getenv("ABOLETH_GEMM_PAIR");
        return v == nullptr ? 2 : std::atoi(v);
    }();
    return mode;
}

// How many 2-CTA clusters of `kernel` the device can hold at the same time.
template <typename Kernel>
int resident_pairs(Kernel kernel, unsigned smem_bytes) {
    cudaLaunchConfig_t config{};
    config.gridDim = dim3(2 * sm_count());
    config.blockDim = dim3(kThreads);
    config.dynamicSmemBytes = smem_bytes;
    cudaLaunchAttribute attribute{};
    attribute.id = cudaLaunchAttributeClusterDimension;
    attribute.val.clusterDim.x = 2;
    attribute.val.clusterDim.y = 1;
    attribute.val.clusterDim.z = 1;
    config.attrs = &attribute;
    config.numAttrs = 1;
    int clusters = 0;
    if (cudaOccupancyMaxActiveClusters(&clusters, kernel, &config) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    if (const char *v = std::getenv("ABOLETH_GEMM_PAIR_TRACE"))
        if (v[0] == '1')
            fprintf(stderr, "aboleth_b200: %d CTA pairs resident (%d SMs)\n", clusters, sm_count());
    return clusters;
}

template <typename Kernel>
bool configure(Kernel kernel, unsigned smem_bytes) {
    return cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes) ==
           cudaSuccess;
}

template <int HALVES>
int launch_grouped(const void *a, const void *w, void *c, const int *counts, const int *offsets,
                   int experts, int total_rows, int n, int k, unsigned long long *status,
                   cudaStream_t stream) {
    using Policy = GroupedPolicy<HALVES>;
    CUtensorMap map_a, map_b;
    if (!make_map_bf16(&map_a, a, total_rows, k, k, Policy::kRows) ||
        !make_map_bf16(&map_b, w, static_cast<std::uint64_t>(experts) * n, k, k, BN))
        return -2;
    constexpr unsigned smem = Geometry<HALVES>::kSmemBytes;
    if (!configure(gemm_tcgen05_kernel<HALVES, Policy>, smem))  // per device context: set on every call
        return -3;
    const int tiles_n = (n + BN - 1) / BN;
    const long long column_bytes = static_cast<long long>(BN) * k * 2;
    const int group_n = static_cast<int>(std::max(1LL, std::min<long long>(tiles_n, (48LL << 20) / column_bytes)));
    Policy p{static_cast<__nv_bfloat16 *>(c), counts, offsets, experts, n, k, n, tiles_n, group_n, 0, 0};
    gemm_tcgen05_kernel<HALVES, Policy><<<sm_count(), kThreads, smem, stream>>>(map_a, map_b, p, status);
    return ab::launch_result("grouped_gemm_bf16");
}

template <int MH, typename Op>
int launch_pair(const void *a, const void *b, PlainPolicy p, int lda, int ldb, unsigned long long *status,
                cudaStream_t stream) {
    using G = pair::PairGeometry<MH>;
    CUtensorMap map_a, map_b;
    // Each CTA of a pair loads MH * 128 rows of A and 128 rows of B per K step.
    const bool mapped = Op::kBK == 64
        ? make_map_bf16(&map_a, a, p.m, p.k, lda, G::kRowsPerCta) && make_map_bf16(&map_b, b, p.n, p.k, ldb, BN / 2)
        : make_map_e4m3(&map_a, a, p.m, p.k, lda, G::kRowsPerCta) && make_map_e4m3(&map_b, b, p.n, p.k, ldb, BN / 2);
    if (!mapped)
        return -2;
    if (!configure(gemm_pair_kernel<MH, Op, PlainPolicy>, G::kSmemBytes))  // per device context: set on every call
        return -3;
    // A persistent kernel must not launch more clusters than can be resident at once: the
    // surplus would start only after a resident one has finished all of its tiles.
    static const int resident = resident_pairs(gemm_pair_kernel<MH, Op, PlainPolicy>, G::kSmemBytes);
    if (resident < 1)
        return -3;
    p.pair = 1;
    p.rows = G::kTileRows;
    p.bk = Op::kBK;
    p.tiles_total = ((p.m + p.rows - 1) / p.rows) * p.tiles_n;
    const int pairs = std::min(p.tiles_total, resident);
    gemm_pair_kernel<MH, Op, PlainPolicy><<<2 * pairs, kThreads, G::kSmemBytes, stream>>>(map_a, map_b, p, status);
    return ab::launch_result(Op::kBK == 64 ? "gemm_bf16 (CTA pairs)" : "gemm_e4m3 (CTA pairs)");
}

// Block-scaled e4m3 GEMM, one CTA per tile of `rows` x `cols` (gemm_mx_sm100.cuh): the plain
// policy's raster order with this loop's tile shape.
struct MxPolicy {
    static constexpr bool kBackground = false, kDrainedHook = false, kScaled = false;
    __nv_bfloat16 *c;
    int m, n, k, ldc;
    int rows, cols;   // tile shape
    int tiles_n, tiles_total, group_n;

    __device__ __forceinline__ bool next(int it, Tile &t) const {
        const int idx = blockIdx.x + it * gridDim.x;
        if (idx >= tiles_total)
            return false;
        const int tiles_m = tiles_total / tiles_n;
        const int per_group = group_n * tiles_m;
        const int group = idx / per_group;
        const int width = min(group_n, tiles_n - group * group_n);
        const int local = idx - group * per_group;
        const int tm = local / width, tn = group * group_n + (local - tm * width);
        t.a_row = tm * rows;
        t.b_row = tn * cols;
        t.k_blocks = k / mx::kBlockK;
        t.c_row = tm * rows;
        t.c_col = tn * cols;
        t.rows_valid = min(rows, m - tm * rows);
        t.cols_valid = min(cols, n - tn * cols);
        t.tag = 0;
        t.a_sel = 0;
        return true;
    }
    __device__ __forceinline__ bool ready(const Tile &) const { return true; }
    __device__ __forceinline__ void store16(const Tile &t, int row, int col, const uint4 &v) const {
        *reinterpret_cast<uint4 *>(c + static_cast<std::size_t>(t.c_row + row) * ldc + t.c_col + col) = v;
    }
    __device__ __forceinline__ void tile_done(const Tile &) const {}
    __device__ __forceinline__ void finish(int, int, unsigned long long *) const {}
};

// Grouped block-scaled GEMM: GroupedPolicy's tile order with the block-scaled loop's tile shape.  An
// expert's rows must start on a multiple of 128 (a scale-factor atom covers 128 rows); a start that does
// not is reported as Malformed and ends the CTA's work.
template <int HALVES>
struct GroupedMxPolicy {
    static constexpr int kRows = BM * HALVES, kCols = mx::MxGeometry<HALVES>::kCols;
    static constexpr bool kBackground = false, kDrainedHook = false, kScaled = false;
    __nv_bfloat16 *c;
    const int *counts, *offsets;
    unsigned long long *status;
    int experts, n, k, ldc, tiles_n;
    int group_n;
    int e, base;   // cursor (per thread): expert `e` starts at linear tile `base`

    __device__ __forceinline__ bool next(int it, Tile &t) {
        const int idx = blockIdx.x + it * gridDim.x;
        int tiles_m = 0;
        while (e < experts) {
            tiles_m = (counts[e] + kRows - 1) / kRows;
            const int tiles_e = tiles_m * tiles_n;
            if (idx < base + tiles_e)
                break;
            base += tiles_e;
            ++e;
        }
        if (e >= experts)
            return false;
        if (offsets[e] & (BM - 1)) {
            ab::set_status(status, aboleth::Status::Malformed, 0x3600 + e);
            return false;
        }
        const int local = idx - base;
        const int per_group = group_n * tiles_m;
        const int group = local / per_group;
        const int width = min(group_n, tiles_n - group * group_n);
        const int in_group = local - group * per_group;
        const int tm = in_group / width, tn = group * group_n + (in_group - tm * width);
        const int row0 = offsets[e] + tm * kRows;
        t.a_row = row0;
        t.b_row = e * n + tn * kCols;
        t.k_blocks = k / mx::kBlockK;
        t.c_row = row0;
        t.c_col = tn * kCols;
        t.rows_valid = min(kRows, counts[e] - tm * kRows);
        t.cols_valid = min(kCols, n - tn * kCols);
        t.tag = e;
        t.a_sel = 0;
        return true;
    }
    __device__ __forceinline__ bool ready(const Tile &) const { return true; }
    __device__ __forceinline__ void store16(const Tile &t, int row, int col, const uint4 &v) const {
        *reinterpret_cast<uint4 *>(c + static_cast<std::size_t>(t.c_row + row) * ldc + t.c_col + col) = v;
    }
    __device__ __forceinline__ void tile_done(const Tile &) const {}
    __device__ __forceinline__ void finish(int, int, unsigned long long *) const {}
};

template <int HALVES>
__global__ void __launch_bounds__(kThreads, 1)
grouped_mx_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                  GroupedMxPolicy<HALVES> params, mx::ScaleFactors sf, unsigned long long *status) {
    GroupedMxPolicy<HALVES> policy = params;
    mx::gemm_mx_mainloop<HALVES>(policy, &map_a, &map_b, sf, status);
}

template <int HALVES>
__global__ void __launch_bounds__(kThreads, 1) gemm_mx_kernel(const __grid_constant__ CUtensorMap map_a,
                                                              const __grid_constant__ CUtensorMap map_b,
                                                              MxPolicy policy, mx::ScaleFactors sf,
                                                              unsigned long long *status) {
    mx::gemm_mx_mainloop<HALVES>(policy, &map_a, &map_b, sf, status);
}

// The exponent byte (ue8m0) of a positive power-of-two fp32; anything else is reported.
__device__ __forceinline__ unsigned ue8m0_of(float scale, unsigned long long *status, unsigned detail) {
    const unsigned bits = __float_as_uint(scale);
    if ((bits & 0x807fffffu) != 0 || (bits >> 23) == 0 || (bits >> 23) == 255)
        ab::set_status(status, aboleth::Status::Malformed, detail);
    return (bits >> 23) & 0xffu;
}

// Activation scales fp32 [rows, k_blocks] (one per row and 128 K) -> atoms [row block][K block] of 512
// bytes: byte (r % 32) * 16 + (r / 32) * 4 + s for row r of the block, the same value for s = 0..3.
__global__ void pack_scales_a_kernel(const float *scales, long long ld, std::uint32_t *out, int rows,
                                     int k_blocks, unsigned long long *status) {
    const long long row_blocks = mx::mx_row_blocks(rows);
    const long long total = row_blocks * k_blocks * 128;
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        const int r = static_cast<int>(i % 128);
        const long long atom = i / 128;           // row_block * k_blocks + kb
        const int kb = static_cast<int>(atom % k_blocks);
        const int row = static_cast<int>(atom / k_blocks) * 128 + r;
        const unsigned e = row < rows ? ue8m0_of(scales[row * ld + kb], status, 0x3500) : 127u;
        out[atom * 128 + (r % 32) * 4 + r / 32] = e * 0x01010101u;
    }
}

// Weight scales fp32 [n_blocks, k_blocks] (one per 128 x 128 block) -> atoms [K block][granule]: atom g
// holds the scales of columns [64 g, 64 g + 128), so that a tile whose first column is any multiple of 64
// (256- and 192-column tiles both) finds its two atoms at g and g + 2.  `granules` per K block.
__global__ void pack_scales_b_kernel(const float *scales, long long ld, std::uint32_t *out, int n_blocks,
                                     int granules, int k_blocks, unsigned long long *status) {
    const long long total = static_cast<long long>(k_blocks) * granules * 128;
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        const long long atom = i / 128;           // kb * granules + g
        const int w = static_cast<int>(i % 128);  // word of the atom: row (w / 4) + 32 * (w % 4)
        const int g = static_cast<int>(atom % granules);
        const int kb = static_cast<int>(atom / granules);
        const int nb = (64 * g + (w >> 2) + 32 * (w & 3)) >> 7;
        const unsigned e = nb < n_blocks ? ue8m0_of(scales[nb * ld + kb], status, 0x3501) : 127u;
        out[i] = e * 0x01010101u;
    }
}

using mx::mx_granules;
using mx::mx_row_blocks;

}  // namespace

// C[M,N] = A[M,K] * B[N,K]^T, all bf16 row-major, lda/ldb/ldc in elements.
// K and the leading dimensions must be multiples of 8 (16-byte TMA strides).
AB_EXPORT int ab_gemm_bf16(const void *a, const void *b, void *c, int m, int n, int k, int lda,
                           int ldb, int ldc, unsigned long long *status, cudaStream_t stream) {
    if (m < 1 || n < 1 || k < 1 || k % 8 || lda % 8 || ldb % 8 || ldc % 8 ||
        (reinterpret_cast<std::uintptr_t>(a) | reinterpret_cast<std::uintptr_t>(b) |
         reinterpret_cast<std::uintptr_t>(c)) & 15)
        return -1;
    PlainPolicy p{static_cast<__nv_bfloat16 *>(c), m, n, k, ldc, (n + BN - 1) / BN, 0, 0, 0, kPlainRows, BK, 1.0f};
    // About 48 MiB of B per raster group.
    const long long column_bytes = static_cast<long long>(BN) * k * 2;
    p.group_n = static_cast<int>(std::max(1LL, std::min<long long>(p.tiles_n, (48LL << 20) / column_bytes)));
    if (gemm_pair_mode() == 2)
        return launch_pair<2, OpBf16>(a, b, p, lda, ldb, status, stream);
    if (gemm_pair_mode() == 1)
        return launch_pair<1, OpBf16>(a, b, p, lda, ldb, status, stream);
    p.tiles_total = ((m + kPlainRows - 1) / kPlainRows) * p.tiles_n;
    CUtensorMap map_a, map_b;
    if (!make_map_bf16(&map_a, a, m, k, lda, kPlainRows) || !make_map_bf16(&map_b, b, n, k, ldb, BN))
        return -2;
    constexpr unsigned smem = Geometry<kPlainHalves>::kSmemBytes;
    if (!configure(gemm_tcgen05_kernel<kPlainHalves, PlainPolicy>, smem))  // per device context: set on every call
        return -3;
    const int grid = p.tiles_total < sm_count() ? p.tiles_total : sm_count();
    gemm_tcgen05_kernel<kPlainHalves, PlainPolicy><<<grid, kThreads, smem, stream>>>(map_a, map_b, p, status);
    return ab::launch_result("gemm_bf16");
}

// C[M,N] (bf16) = alpha * A[M,K] * B[N,K]^T with A and B in e4m3 (one byte per element), row-major,
// lda/ldb in elements (= bytes), ldc in bf16 elements.  K, lda and ldb must be multiples of 16.
// `alpha` carries the product of the two per-tensor scales.  CTA-pair main loop, kind::f8f6f4.
AB_EXPORT int ab_gemm_e4m3(const void *a, const void *b, void *c, int m, int n, int k, int lda, int ldb,
                           int ldc, float alpha, unsigned long long *status, cudaStream_t stream) {
    if (m < 1 || n < 1 || k < 1 || k % 16 || lda % 16 || ldb % 16 || ldc % 8 ||
        (reinterpret_cast<std::uintptr_t>(a) | reinterpret_cast<std::uintptr_t>(b) |
         reinterpret_cast<std::uintptr_t>(c)) & 15)
        return -1;
    PlainPolicy p{static_cast<__nv_bfloat16 *>(c), m, n, k, ldc, (n + BN - 1) / BN, 0, 0, 0, kPlainRows,
                  OpE4m3::kBK, alpha};
    const long long column_bytes = static_cast<long long>(BN) * k;
    p.group_n = static_cast<int>(std::max(1LL, std::min<long long>(p.tiles_n, (48LL << 20) / column_bytes)));
    return launch_pair<2, OpE4m3>(a, b, p, lda, ldb, status, stream);
}

// Grouped GEMM over `experts` problems that share N and K.  a: [total_rows, K],
// w: [experts, N, K], c: [total_rows, N]; counts/offsets: device int32 [experts].
AB_EXPORT int ab_grouped_gemm_bf16(const void *a, const void *w, void *c, const int *counts,
                                   const int *offsets, int experts, int total_rows, int n, int k,
                                   unsigned long long *status, cudaStream_t stream) {
    if (experts < 1 || total_rows < 1 || n < 1 || k < 1 || k % 8 || n % 8 ||
        (reinterpret_cast<std::uintptr_t>(a) | reinterpret_cast<std::uintptr_t>(w) |
         reinterpret_cast<std::uintptr_t>(c)) & 15)
        return -1;
    // 256-row tiles once the experts are big enough on average to fill them.
    if (total_rows / experts >= 512)
        return launch_grouped<2>(a, w, c, counts, offsets, experts, total_rows, n, k, status, stream);
    return launch_grouped<1>(a, w, c, counts, offsets, experts, total_rows, n, k, status, stream);
}

template <int HALVES>
int launch_grouped_mx(const void *a, const void *sfa, const void *w, const void *sfb, void *c, const int *counts,
                      const int *offsets, int experts, int total_rows, int n, int k,
                      unsigned long long *status, cudaStream_t stream) {
    using Policy = GroupedMxPolicy<HALVES>;
    using G = mx::MxGeometry<HALVES>;
    CUtensorMap map_a, map_b;
    if (!make_map_e4m3(&map_a, a, total_rows, k, k, Policy::kRows) ||
        !make_map_e4m3(&map_b, w, static_cast<std::uint64_t>(experts) * n, k, k, Policy::kCols))
        return -2;
    if (!configure(grouped_mx_kernel<HALVES>, G::kSmemBytes))
        return -3;
    Policy p{static_cast<__nv_bfloat16 *>(c), counts, offsets, status, experts, n, k, n,
             (n + Policy::kCols - 1) / Policy::kCols, 1, 0, 0};
    const long long column_bytes = static_cast<long long>(Policy::kCols) * k;
    p.group_n = static_cast<int>(std::max(1LL, std::min<long long>(p.tiles_n, (48LL << 20) / column_bytes)));
    const mx::ScaleFactors sf{static_cast<const std::uint8_t *>(sfa), static_cast<const std::uint8_t *>(sfb),
                              k / 128, mx_granules(experts * n)};
    // The tile count depends on counts the host never reads: a persistent grid of one CTA per SM.
    grouped_mx_kernel<HALVES><<<sm_count(), kThreads, G::kSmemBytes, stream>>>(map_a, map_b, p, sf, status);
    return ab::launch_result("grouped_gemm_e4m3_mx");
}

// Grouped block-scaled GEMM: a [total_rows, K] e4m3 in expert-contiguous order with every expert's first
// row on a multiple of 128, w [experts, N, K] e4m3, N a multiple of 64; `sfa` = ab_mx_pack_scales of the
// [total_rows, K/128] activation scales, `sfb` = of the [experts * N / 128, K/128] weight scales (the
// weights seen as one [experts * N, K] matrix).  c [total_rows, N] bf16.
AB_EXPORT int ab_grouped_gemm_e4m3_mx(const void *a, const void *sfa, const void *w, const void *sfb, void *c,
                                      const int *counts, const int *offsets, int experts, int total_rows,
                                      int n, int k, unsigned long long *status, cudaStream_t stream) {
    if (experts < 1 || total_rows < 1 || n < 64 || n % 64 || k < 128 || k % 128 || sfa == nullptr ||
        sfb == nullptr ||
        (reinterpret_cast<std::uintptr_t>(a) | reinterpret_cast<std::uintptr_t>(w) |
         reinterpret_cast<std::uintptr_t>(c) | reinterpret_cast<std::uintptr_t>(sfa) |
         reinterpret_cast<std::uintptr_t>(sfb)) & 15)
        return -1;
    if (total_rows / experts >= 256)
        return launch_grouped_mx<2>(a, sfa, w, sfb, c, counts, offsets, experts, total_rows, n, k, status, stream);
    return launch_grouped_mx<1>(a, sfa, w, sfb, c, counts, offsets, experts, total_rows, n, k, status, stream);
}

// Bytes of the packed scale factors of a block-scaled GEMM: A atoms for `m` rows, B atoms for `n` columns.
AB_EXPORT long long ab_mx_scale_bytes(int m, int n, int k, int which) {
    const long long k_blocks = (k + 127) / 128;
    if (which == 0)
        return mx_row_blocks(m) * k_blocks * 512;
    return k_blocks * mx_granules(n) * 512;
}

// fp32 power-of-two scales -> ue8m0 atoms in the order the tensor core reads them.  which = 0: activation
// scales [rows, K/128] (one per row and K block); which = 1: weight scales [ceil(rows/128), K/128].  A scale
// that is not a positive power of two is reported as Malformed in `status` (the product would be wrong).
AB_EXPORT int ab_mx_pack_scales(const float *scales, long long ld, void *out, int rows, int k, int which,
                                unsigned long long *status, cudaStream_t stream) {
    if (scales == nullptr || out == nullptr || rows < 1 || k < 128 || k % 128)
        return -1;
    const int k_blocks = k / 128;
    if (which == 0) {
        pack_scales_a_kernel<<<148, 256, 0, stream>>>(scales, ld, static_cast<std::uint32_t *>(out), rows,
                                                      k_blocks, status);
    } else {
        pack_scales_b_kernel<<<148, 256, 0, stream>>>(scales, ld, static_cast<std::uint32_t *>(out),
                                                      (rows + 127) / 128, mx_granules(rows), k_blocks, status);
    }
    return ab::launch_result("mx_pack_scales");
}

// C[M,N] (bf16) = (A * sa) (B * sb)^T for e4m3 A [M,K] and B [N,K] (row-major, lda / ldb in bytes) whose
// scales were packed by ab_mx_pack_scales: tcgen05.mma.kind::mxf8f6f4.block_scale, no expansion pass.
// K must be a multiple of 128.
AB_EXPORT int ab_gemm_e4m3_mx(const void *a, const void *b, void *c, const void *sfa, const void *sfb, int m,
                              int n, int k, int lda, int ldb, int ldc, unsigned long long *status,
                              cudaStream_t stream) {
    if (m < 1 || n < 1 || k < 128 || k % 128 || lda % 16 || ldb % 16 || ldc % 8 || sfa == nullptr ||
        sfb == nullptr ||
        (reinterpret_cast<std::uintptr_t>(a) | reinterpret_cast<std::uintptr_t>(b) |
         reinterpret_cast<std::uintptr_t>(c) | reinterpret_cast<std::uintptr_t>(sfa) |
         reinterpret_cast<std::uintptr_t>(sfb)) & 15)
        return -1;
    // 256 x 192 tiles (two row blocks share a B tile: about 5 % faster per FLOP) unless the 128 x 256
    // shape wastes less of its last wave.  ABOLETH_GEMM_MX_TILE=1 / 2 forces one / two row blocks.
    int halves = 1;
    if (m > BM) {
        const long long sms = sm_count();
        const long long tiles1 = static_cast<long long>((m + 127) / 128) * ((n + 255) / 256);
        const long long tiles2 = static_cast<long long>((m + 255) / 256) * ((n + 191) / 192);
        const long long cost1 = (tiles1 + sms - 1) / sms * (128 * 256) * 105;
        const long long cost2 = (tiles2 + sms - 1) / sms * (256 * 192) * 100;
        halves = cost2 <= cost1 ? 2 : 1;
    }
    if (const char *forced = std::getenv("ABOLETH_GEMM_MX_TILE"))
        halves = forced[0] == '1' ? 1 : 2;
    MxPolicy p{};
    p.c = static_cast<__nv_bfloat16 *>(c);
    p.m = m, p.n = n, p.k = k, p.ldc = ldc;
    p.rows = BM * halves;
    p.cols = halves == 1 ? mx::MxGeometry<1>::kCols : mx::MxGeometry<2>::kCols;
    p.tiles_n = (n + p.cols - 1) / p.cols;
    p.tiles_total = ((m + p.rows - 1) / p.rows) * p.tiles_n;
    const long long column_bytes = static_cast<long long>(p.cols) * k;
    p.group_n = static_cast<int>(std::max(1LL, std::min<long long>(p.tiles_n, (48LL << 20) / column_bytes)));
    CUtensorMap map_a, map_b;
    if (!make_map_e4m3(&map_a, a, m, k, lda, p.rows) || !make_map_e4m3(&map_b, b, n, k, ldb, p.cols))
        return -2;
    const mx::ScaleFactors sf{static_cast<const std::uint8_t *>(sfa), static_cast<const std::uint8_t *>(sfb),
                              k / 128, mx_granules(n)};
    const int grid = p.tiles_total < sm_count() ? p.tiles_total : sm_count();
    if (halves == 1) {
        if (!configure(gemm_mx_kernel<1>, mx::MxGeometry<1>::kSmemBytes))
            return -3;
        gemm_mx_kernel<1><<<grid, kThreads, mx::MxGeometry<1>::kSmemBytes, stream>>>(map_a, map_b, p, sf, status);
    } else {
        if (!configure(gemm_mx_kernel<2>, mx::MxGeometry<2>::kSmemBytes))
            return -3;
        gemm_mx_kernel<2><<<grid, kThreads, mx::MxGeometry<2>::kSmemBytes, stream>>>(map_a, map_b, p, sf, status);
    }
    return ab::launch_result("gemm_e4m3_mx");
}
