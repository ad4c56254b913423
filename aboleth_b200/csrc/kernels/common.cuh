// Shared pieces of the hand-written sm_100a kernels: launch-error plumbing,
// bounded waits on flags and mbarriers, bulk-async (TMA) copy wrappers and the
// counter-based payload generator used by the self-checking benchmarks.
#pragma once

#include <cstdint>
#include <cstdio>
#include <cuda_runtime.h>

#include "aboleth/device.cuh"

#define AB_EXPORT extern "C" __attribute__((visibility("default")))

namespace ab {

__host__ __device__ __forceinline__ std::uint64_t min64(std::uint64_t a, std::uint64_t b) {
    return a < b ? a : b;
}

// Status word layout used by every kernel here: word 0 = first non-zero
// aboleth::Status, word 1 = a kernel-specific detail (which wait gave up).
__device__ __forceinline__ void set_status(unsigned long long *status,
                                           aboleth::Status s, unsigned long long detail) {
    if (status == nullptr || s == aboleth::Status::Ok)
        return;
    if (atomicCAS(status, 0ull, static_cast<unsigned long long>(s)) == 0ull)
        status[1] = detail;
}

inline int launch_result(const char *what) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        fprintf(stderr, "aboleth_b200: %s launch failed: %s\n", what, cudaGetErrorString(e));
        return static_cast<int>(e);
    }
    return 0;
}

__device__ __forceinline__ std::uint32_t smem_u32(const void *p) {
    return static_cast<std::uint32_t>(__cvta_generic_to_shared(p));
}

// ---- mbarrier (bounded) ---------------------------------------------------------

__device__ __forceinline__ void mbar_init(std::uint64_t *bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}

__device__ __forceinline__ void mbar_fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void mbar_expect_tx(std::uint64_t *bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
                 "r"(bytes)
                 : "memory");
}

__device__ __forceinline__ void mbar_arrive(std::uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(std::uint64_t *bar, unsigned parity) {
    unsigned ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}

// Wait for the phase with `parity` to complete.  Gives up after ~4 s of
// %globaltimer and reports false; the caller must then stop issuing work,
// record the failure and fall through to its teardown.
__device__ __forceinline__ bool mbar_wait(std::uint64_t *bar, unsigned parity) {
    for (int i = 0; i < 4096; ++i)
        if (mbar_try_wait(bar, parity))
            return true;
    const std::uint64_t start = aboleth::detail::globaltimer_ns();
    while (!mbar_try_wait(bar, parity)) {
        if (aboleth::detail::globaltimer_ns() - start > 4000000000ull)
            return false;
    }
    return true;
}

// ---- untiled bulk-async copies (16-byte aligned addresses and sizes) -----------

__device__ __forceinline__ void bulk_load(void *smem_dst, const void *gmem_src,
                                          unsigned bytes, std::uint64_t *bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::
            "r"(smem_u32(smem_dst)),
        "l"(gmem_src), "r"(bytes), "r"(smem_u32(bar))
        : "memory");
}

__device__ __forceinline__ void bulk_store(void *gmem_dst, const void *smem_src, unsigned bytes) {
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gmem_dst),
                 "r"(smem_u32(smem_src)), "r"(bytes)
                 : "memory");
}

__device__ __forceinline__ void bulk_commit() {
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}

template <int N>
__device__ __forceinline__ void bulk_wait_read() {
    asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}

template <int N>
__device__ __forceinline__ void bulk_wait_all() {
    asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}

__device__ __forceinline__ void fence_proxy_async() {
    asm volatile("fence.proxy.async;" ::: "memory");
}

// ---- seeded payload --------------------------------------------------------------

__host__ __device__ __forceinline__ std::uint64_t splitmix64(std::uint64_t x) {
    x += 0x9E3779B97F4A7C15ull;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    return x ^ (x >> 31);
}

// Eight uniform-random payload bytes for 8-byte word `word` of the slice that
// `sender` sends to `receiver`.  Both sides can regenerate it.
__host__ __device__ __forceinline__ std::uint64_t payload_word(
    std::uint64_t seed, unsigned sender, unsigned receiver, std::uint64_t word) {
    const std::uint64_t stream =
        splitmix64(seed ^ (static_cast<std::uint64_t>(sender) << 40) ^
                   (static_cast<std::uint64_t>(receiver) << 20));
    return splitmix64(stream + word);
}

}  // namespace ab
