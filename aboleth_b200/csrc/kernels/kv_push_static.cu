// `ab_kv_push_static`: the KV page push with its arrival counters in a fixed array of
// the library image, for callers that cannot allocate device memory (see
// aboleth/kv_push_static.h for who they are and for the rules of the call).
#include <atomic>

#include "aboleth/kv_push_static.h"
#include "common.cuh"

namespace {

struct KvBatch {
    std::uint64_t src;     // local address of the run (contiguous pages)
    std::uint64_t dst;     // peer address of the destination slot storage
    std::uint64_t bytes;   // run length
    std::uint64_t ready;   // peer address of the int64 readiness cell
};

// One arrival counter per batch.  Lives in the module's global segment on every device
// that loads this library, so no call ever has to allocate it.
static __device__ __align__(256) unsigned g_kv_arrivals[AB_KV_PUSH_STATIC_MAX_BATCHES];

// Same work split and publication rule as the allocating entry point: the workers of a
// batch copy 16-byte aligned slices; each ends with a CTA barrier and one arrival; the
// last arrival fences at system scope and release-stores the epoch on the consumer.
// The counter is not reset here: the entry point clears it before every launch.
__global__ void __launch_bounds__(512) kv_push_static_kernel(const KvBatch *batches,
                                                             unsigned *arrivals, std::uint64_t epoch,
                                                             int workers, unsigned long long *status) {
    const KvBatch b = batches[blockIdx.x];
    const int worker = blockIdx.y;
    const std::uint64_t per = ((b.bytes + workers - 1) / workers + 15) & ~15ull;
    const std::uint64_t begin = ab::min64(per * worker, b.bytes);
    const std::uint64_t end = ab::min64(begin + per, b.bytes);
    if (((b.src | b.dst) & 15) != 0 && threadIdx.x == 0 && worker == 0)
        ab::set_status(status, aboleth::Status::Malformed, 0x7200 + blockIdx.x);
    aboleth::detail::copy_strided(reinterpret_cast<std::uint8_t *>(b.dst + begin),
                                  reinterpret_cast<const std::uint8_t *>(b.src + begin), end - begin,
                                  threadIdx.x, blockDim.x);
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        if (atomicAdd(arrivals + blockIdx.x, 1u) == static_cast<unsigned>(workers) - 1) {
            aboleth::detail::fence_acq_rel_sys();
            aboleth::detail::st_release_sys(reinterpret_cast<std::uint64_t *>(b.ready), epoch);
        }
    }
}

constexpr int kMaxCachedDevices = 64;
std::atomic<unsigned *> g_counter_address[kMaxCachedDevices];

// Device address of the counter array on the current device.  Looked up once per
// device; a device ordinal beyond the cache is looked up on every call.
int counter_address(unsigned **out) {
    int device = 0;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess)
        return static_cast<int>(e);
    const bool cached = device >= 0 && device < kMaxCachedDevices;
    unsigned *p = cached ? g_counter_address[device].load(std::memory_order_acquire) : nullptr;
    if (p == nullptr) {
        e = cudaGetSymbolAddress(reinterpret_cast<void **>(&p), g_kv_arrivals);
        if (e != cudaSuccess || p == nullptr) {
            fprintf(stderr, "aboleth_b200: ab_kv_push_static: no address for the counter array: %s\n",
                    cudaGetErrorString(e));
            return e != cudaSuccess ? static_cast<int>(e) : static_cast<int>(cudaErrorInvalidSymbol);
        }
        if (cached)
            g_counter_address[device].store(p, std::memory_order_release);
    }
    *out = p;
    return 0;
}

}  // namespace

AB_EXPORT int ab_kv_push_static(const void *batches, int count, std::uint64_t epoch, int workers,
                                int threads, unsigned long long *status, cudaStream_t stream) {
    if (batches == nullptr || count < 1 || workers < 1 || workers > 65535 || threads < 32 ||
        threads > 512 || threads % 32 != 0) {
        fprintf(stderr, "aboleth_b200: ab_kv_push_static: bad argument (count %d, workers %d, threads %d)\n",
                count, workers, threads);
        return AB_KV_PUSH_STATIC_BAD_ARGUMENT;
    }
    if (count > AB_KV_PUSH_STATIC_MAX_BATCHES) {
        fprintf(stderr,
                "aboleth_b200: ab_kv_push_static: %d batches exceed the built-in limit of %d; split the "
                "transfer into several calls on one stream\n",
                count, AB_KV_PUSH_STATIC_MAX_BATCHES);
        return AB_KV_PUSH_STATIC_TOO_MANY;
    }
    unsigned *arrivals = nullptr;
    if (int rc = counter_address(&arrivals))
        return rc;
    cudaError_t e = cudaMemsetAsync(arrivals, 0, sizeof(unsigned) * static_cast<size_t>(count), stream);
    if (e != cudaSuccess) {
        fprintf(stderr, "aboleth_b200: ab_kv_push_static: clearing the counters failed: %s\n",
                cudaGetErrorString(e));
        return static_cast<int>(e);
    }
    kv_push_static_kernel<<<dim3(count, workers), threads, 0, stream>>>(
        static_cast<const KvBatch *>(batches), arrivals, epoch, workers, status);
    return ab::launch_result("kv_push_static");
}
