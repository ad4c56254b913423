// KV-cache page push: a producer rank stores runs of pages into a consumer rank's
// slot storage over NVLink and publishes per-(slot, consumer, source) readiness.
//
// Grid (batches, workers).  The workers of one batch split its bytes; every worker
// ends with a CTA barrier and one atomic arrival.  Batches that publish the SAME
// readiness cell (several layers and runs of one readiness group) form a group with
// one arrival counter whose target is the group's worker total: only the worker that
// arrives last IN THE GROUP performs the system fence and release-stores the epoch,
// so the cell never shows the epoch while a sibling batch is still copying - "the
// last copy worker of a consumer performs the system fence and publishes the epoch"
// (reference docs/KV_CACHE.md:46-48; kernels
// python/aboleth/frontends/triton/kv_cache.py:133-292 count per batch and then per
// consumer, and copy 8-byte words; these count once per group and copy 16-byte
// vectors, four in flight per thread).
#include "common.cuh"

namespace {

struct KvBatch {
    std::uint64_t src;     // local address of the run (contiguous pages)
    std::uint64_t dst;     // peer address of the destination slot storage
    std::uint64_t bytes;   // run length (pages * page_bytes)
    std::uint64_t ready;   // peer address of the int64 readiness cell
};

// One worker CTA: copy its slice of batch `batch`, arrive, publish if last of the group.
//   group_of == nullptr : every batch is its own group (counter `batch`, target `workers`);
//   otherwise           : counter group_of[batch], target group_target[group_of[batch]].
__device__ __forceinline__ void push_worker(const KvBatch *batches, unsigned *arrivals,
                                            const int *group_of, const unsigned *group_target,
                                            int batch, int worker, std::uint64_t epoch, int workers,
                                            unsigned long long *status) {
    const KvBatch b = batches[batch];
    // 16-byte aligned worker slices.
    const std::uint64_t per = ((b.bytes + workers - 1) / workers + 15) & ~15ull;
    const std::uint64_t begin = ab::min64(per * worker, b.bytes);
    const std::uint64_t end = ab::min64(begin + per, b.bytes);
    // A run that is not 16-byte aligned is reported and still copied (8-byte or byte path).
    if (((b.src | b.dst) & 15) != 0 && threadIdx.x == 0 && worker == 0)
        ab::set_status(status, aboleth::Status::Malformed, 0x7000 + batch);
    aboleth::detail::copy_strided(reinterpret_cast<std::uint8_t *>(b.dst + begin),
                                  reinterpret_cast<const std::uint8_t *>(b.src + begin), end - begin,
                                  threadIdx.x, blockDim.x);
    __syncthreads();
    if (threadIdx.x == 0) {
        const int counter = group_of != nullptr ? group_of[batch] : batch;
        const unsigned target = group_of != nullptr ? group_target[counter] : static_cast<unsigned>(workers);
        __threadfence();
        const unsigned old = atomicAdd(arrivals + counter, 1u);
        if (old == target - 1) {
            arrivals[counter] = 0;  // self-cleaning for the next transfer
            aboleth::detail::fence_acq_rel_sys();
            aboleth::detail::st_release_sys(reinterpret_cast<std::uint64_t *>(b.ready), epoch);
        }
    }
}

__global__ void __launch_bounds__(512) kv_push_kernel(const KvBatch *batches, unsigned *arrivals,
                                                      const int *group_of, const unsigned *group_target,
                                                      std::uint64_t epoch, int workers,
                                                      unsigned long long *status) {
    push_worker(batches, arrivals, group_of, group_target, blockIdx.x, blockIdx.y, epoch, workers, status);
}

// Self-check form: the same push plus ONE consumer CTA in the same launch (block row `count`),
// which waits (bounded) for `cell` to show `epoch` and then, at once, sums the 8-byte words of
// every batch's destination into observed[0].  A cell that is published before the data has
// landed shows up as a sum that differs from the sources'.  One launch, every CTA resident:
// nothing here waits on another launch.
__global__ void __launch_bounds__(512) kv_push_observed_kernel(
    const KvBatch *batches, unsigned *arrivals, const int *group_of, const unsigned *group_target,
    int count, std::uint64_t epoch, int workers, const std::uint64_t *cell,
    unsigned long long *observed, std::uint64_t timeout_ns, unsigned long long *status) {
    if (static_cast<int>(blockIdx.x) < count) {
        push_worker(batches, arrivals, group_of, group_target, blockIdx.x, blockIdx.y, epoch, workers, status);
        return;
    }
    if (blockIdx.y != 0)
        return;
    __shared__ int s_ok;
    __shared__ unsigned long long s_sum;
    if (threadIdx.x == 0) {
        const aboleth::Status s = aboleth::wait_signal_status(cell, epoch, timeout_ns);
        ab::set_status(status, s, 0x7300);
        s_ok = s == aboleth::Status::Ok;
        s_sum = 0;
    }
    __syncthreads();
    if (!s_ok)
        return;
    unsigned long long sum = 0;
    for (int i = 0; i < count; ++i) {
        const KvBatch b = batches[i];
        const std::uint64_t *words = reinterpret_cast<const std::uint64_t *>(b.dst);
        for (std::uint64_t w = threadIdx.x; w < b.bytes / 8; w += blockDim.x)
            sum += aboleth::detail::ld_relaxed_sys(words + w);
    }
    atomicAdd(&s_sum, sum);
    __syncthreads();
    if (threadIdx.x == 0)
        observed[0] = s_sum;
}

// Consumer side: wait (bounded) until every listed readiness cell reached `epoch`.
__global__ void kv_wait_kernel(const std::uint64_t *cells, int count, std::uint64_t epoch,
                               std::uint64_t timeout_ns, unsigned long long *status) {
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < count; i += gridDim.x * blockDim.x) {
        const aboleth::Status s = aboleth::wait_signal_status(cells + i, epoch, timeout_ns);
        ab::set_status(status, s, 0x7100 + i);
    }
}

}  // namespace

// batches: device array of `count` {src, dst, bytes, ready} records; arrivals: device u32, zeroed,
// one per batch (group_of == nullptr) or one per group.  group_of: device int [count], the group of
// each batch; group_target: device u32, arrivals that complete each group (its batches x workers).
// Batches that name the same readiness cell MUST share a group.
AB_EXPORT int ab_kv_push(const void *batches, unsigned *arrivals, const int *group_of,
                         const unsigned *group_target, int count, std::uint64_t epoch, int workers,
                         int threads, unsigned long long *status, cudaStream_t stream) {
    if (batches == nullptr || arrivals == nullptr || count < 1 || workers < 1 || workers > 65535 ||
        threads < 32 || threads > 512 || threads % 32 != 0 ||
        (group_of == nullptr) != (group_target == nullptr))
        return -1;
    kv_push_kernel<<<dim3(count, workers), threads, 0, stream>>>(
        static_cast<const KvBatch *>(batches), arrivals, group_of, group_target, epoch, workers, status);
    return ab::launch_result("kv_push");
}

// The push with a consumer CTA in the same launch (see kv_push_observed_kernel).
AB_EXPORT int ab_kv_push_observed(const void *batches, unsigned *arrivals, const int *group_of,
                                  const unsigned *group_target, int count, std::uint64_t epoch,
                                  int workers, int threads, const std::uint64_t *cell,
                                  unsigned long long *observed, std::uint64_t timeout_ns,
                                  unsigned long long *status, cudaStream_t stream) {
    if (batches == nullptr || arrivals == nullptr || cell == nullptr || observed == nullptr ||
        count < 1 || workers < 1 || workers > 64 || (count + 1) * workers > 148 || threads < 32 ||
        threads > 512 || threads % 32 != 0 || (group_of == nullptr) != (group_target == nullptr))
        return -1;  // the whole grid must be resident: at most one CTA per SM is asked for
    kv_push_observed_kernel<<<dim3(count + 1, workers), threads, 0, stream>>>(
        static_cast<const KvBatch *>(batches), arrivals, group_of, group_target, count, epoch, workers,
        cell, observed, timeout_ns, status);
    return ab::launch_result("kv_push_observed");
}

AB_EXPORT int ab_kv_wait(const std::uint64_t *cells, int count, std::uint64_t epoch,
                         std::uint64_t timeout_ns, unsigned long long *status, cudaStream_t stream) {
    if (count < 1)
        return -1;
    kv_wait_kernel<<<(count + 127) / 128, 128, 0, stream>>>(cells, count, epoch, timeout_ns, status);
    return ab::launch_result("kv_wait");
}

// Copy-engine path for few, large runs: one asynchronous copy per run (addresses may be peer
// mappings; unified addressing picks the direction).
AB_EXPORT int ab_memcpy_async(void *dst, const void *src, std::uint64_t bytes, cudaStream_t stream) {
    const cudaError_t e = cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDefault, stream);
    if (e != cudaSuccess) {
        fprintf(stderr, "aboleth_b200: asynchronous copy failed: %s\n", cudaGetErrorString(e));
        return static_cast<int>(e);
    }
    return 0;
}
