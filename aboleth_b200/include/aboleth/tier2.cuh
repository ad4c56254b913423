// Run-time helpers of kernels emitted by the Tier-2 specializer.
//
// A Tier-2 program is SPMD over the CTA (like one Triton program): every
// thread executes every statement, single-issuer actions are predicated on
// thread 0.  What the specializer decided - where the CTA barrier goes, whether
// a system fence is needed, which store publishes - is spelled out in the
// emitted code; these helpers only hold the mechanics.
//
// The peer-memory put mirrors the reference lowering
// (compiler/lib/Target/P2P/LowerP2P.cpp:181-288,348-451): a run-time test of
// 8-byte alignment on source, destination and length; a cooperative copy by
// the whole CTA in steps of COOP_ELEMENTS 8-byte elements when the put is at
// least `coop_min` bytes; otherwise one thread copies 8-byte words, or bytes.
#pragma once

#include "aboleth/device.cuh"

namespace aboleth::t2 {

// Bytes of `requested` that lie inside the valid prefix of a region view:
// count normalised to [0, capacity], 64-bit math until the 32-bit length.
__device__ __forceinline__ std::uint32_t ab_valid_bytes(
    long long requested, long long count, long long capacity, long long item_bytes, long long at) {
    const long long n = count < 0 ? 0 : (count > capacity ? capacity : count);
    const long long left = n * item_bytes - at;
    const long long take = left < 0 ? 0 : (left < requested ? left : requested);
    return static_cast<std::uint32_t>(take);
}

// Same safety normalisation, but the padding travels: the full request, as
// long as it stays inside the region's capacity.
__device__ __forceinline__ std::uint32_t ab_checked_bytes(
    long long requested, long long count, long long capacity, long long item_bytes, long long at) {
    (void)count;
    const long long left = capacity * item_bytes - at;
    const long long take = left < 0 ? 0 : (left < requested ? left : requested);
    return static_cast<std::uint32_t>(take);
}

template <int COOP_ELEMENTS>
__device__ __forceinline__ bool put_p2p(std::uint64_t dst, std::uint64_t src, std::uint32_t bytes,
                                        std::uint32_t coop_min, bool scalar_only) {
    const bool aligned8 = ((dst | src | bytes) & 7) == 0;
    if (aligned8 && bytes >= coop_min && !scalar_only) {
        const unsigned tid = threadIdx.x, n = blockDim.x;
        const std::uint64_t step = static_cast<std::uint64_t>(COOP_ELEMENTS) * 8;
        for (std::uint64_t off = 0; off < bytes; off += step) {
            const std::uint64_t len = bytes - off < step ? bytes - off : step;
            detail::copy_strided(reinterpret_cast<std::uint8_t *>(dst + off),
                                 reinterpret_cast<const std::uint8_t *>(src + off), len, tid, n);
        }
        return true;  // cooperative: the caller's barrier follows
    }
    if (threadIdx.x == 0)
        detail::copy_strided(reinterpret_cast<std::uint8_t *>(dst),
                             reinterpret_cast<const std::uint8_t *>(src), bytes, 0, 1);
    return false;
}

template <typename T>
__device__ __forceinline__ void store_inline(std::uint64_t dst, unsigned long long value) {
    *reinterpret_cast<volatile T *>(dst) = static_cast<T>(value);
}

// 24-bit inline value: 16 + 8 bits, little endian.
__device__ __forceinline__ void store_inline24(std::uint64_t dst, unsigned long long value) {
    *reinterpret_cast<volatile std::uint16_t *>(dst) = static_cast<std::uint16_t>(value);
    *reinterpret_cast<volatile std::uint8_t *>(dst + 2) = static_cast<std::uint8_t>(value >> 16);
}

__device__ __forceinline__ void record(unsigned long long *status, Status s, unsigned detail_code) {
    if (status != nullptr && s != Status::Ok)
        if (atomicCAS(status, 0ull, static_cast<unsigned long long>(s)) == 0ull)
            status[1] = detail_code;
}

// Thread 0 waits (bounded); the CTA barrier hands the acquired view to all.
__device__ __forceinline__ void wait_signal_cta(std::uint64_t flag, std::uint64_t epoch,
                                                unsigned long long *status, unsigned detail_code) {
    if (threadIdx.x == 0)
        record(status, wait_signal_status(reinterpret_cast<const std::uint64_t *>(flag), epoch),
               detail_code);
    __syncthreads();
}

}  // namespace aboleth::t2
