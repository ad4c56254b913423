// KV-cache page push: a producer rank stores runs of pages into a consumer rank's
// slot storage over NVLink and publishes per-(slot, consumer, source) readiness.
//
// Grid (batches, workers).  The workers of one batch split its bytes; every worker
// ends with a CTA barrier and one atomic arrival (release at GPU scope); the worker
// that arrives last performs the system fence and release-stores the readiness
// epoch on the consumer - "the last copy worker of a consumer performs the system
// fence and publishes the epoch" (reference docs/KV_CACHE.md:46-48; kernels
// python/aboleth/frontends/triton/kv_cache.py:133-292, which copy 8-byte words; these
// copy 16-byte vectors, four in flight per thread).
#include "common.cuh"

namespace {

struct KvBatch {
    std::uint64_t src;     // local address of the run (contiguous pages)
    std::uint64_t dst;     // peer address of the destination slot storage
    std::uint64_t bytes;   // run length (pages * page_bytes)
    std::uint64_t ready;   // peer address of the int64 readiness cell
};

__global__ void __launch_bounds__(512) kv_push_kernel(const KvBatch *batches, unsigned *arrivals,
                                                      std::uint64_t epoch, int workers,
                                                      unsigned long long *status) {
    const KvBatch b = batches[blockIdx.x];
    const int worker = blockIdx.y;
    // 16-byte aligned worker slices.
    const std::uint64_t per = ((b.bytes + workers - 1) / workers + 15) & ~15ull;
    const std::uint64_t begin = ab::min64(per * worker, b.bytes);
    const std::uint64_t end = ab::min64(begin + per, b.bytes);
    if (((b.src | b.dst) & 15) != 0 && threadIdx.x == 0 && worker == 0)
        ab::set_status(status, aboleth::Status::Malformed, 0x7000 + blockIdx.x);
    aboleth::detail::copy_strided(reinterpret_cast<std::uint8_t *>(b.dst + begin),
                                  reinterpret_cast<const std::uint8_t *>(b.src + begin), end - begin,
                                  threadIdx.x, blockDim.x);
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        const unsigned old = atomicAdd(arrivals + blockIdx.x, 1u);
        if (old == static_cast<unsigned>(workers) - 1) {
            arrivals[blockIdx.x] = 0;  // self-cleaning for the next transfer
            aboleth::detail::fence_acq_rel_sys();
            aboleth::detail::st_release_sys(reinterpret_cast<std::uint64_t *>(b.ready), epoch);
        }
    }
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

// batches: device array of `count` {src, dst, bytes, ready} records; arrivals: device u32 [count], zeroed.
AB_EXPORT int ab_kv_push(const void *batches, unsigned *arrivals, int count, std::uint64_t epoch,
                         int workers, int threads, unsigned long long *status, cudaStream_t stream) {
    if (count < 1 || workers < 1 || workers > 65535 || threads < 32 || threads > 512)
        return -1;
    kv_push_kernel<<<dim3(count, workers), threads, 0, stream>>>(
        static_cast<const KvBatch *>(batches), arrivals, epoch, workers, status);
    return ab::launch_result("kv_push");
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
