// Tier 1: one-sided transport callable from any CUDA kernel (sm_100a).
//
//   aboleth::DeviceContext ctx{endpoint_handles, nullptr, status_words};
//   aboleth::put(ctx, peer, remote_row, local_row, bytes);
//   aboleth::put_inline(ctx, peer, remote_word, value);
//   aboleth::signal(ctx, peer, remote_flag, epoch);
//   aboleth::quiet(ctx, peer);
//   aboleth::wait_signal(ctx, local_flag, epoch);
//
// The call shapes are those of the reference facade
// (include/aboleth/device.cuh:40-125) and of the header its generator renders
// (python/aboleth/emit/tier1_header.py:497-813: open, put_signal, put_many,
// put_many_signal, put_many_flush, put_warp).  Addresses come from the rank's
// peer-region table (World.exchange_regions); there is no symmetric heap.
//
// What is different on purpose:
//  * This header is written by hand for NVLink peer memory.  A put is a
//    vectorised copy into the peer's mapping, a signal is one
//    `st.release.sys` that publishes every store the calling thread (or, for
//    the *_block forms, the calling CTA) made before it, and nothing else is
//    fenced: the release is the only ordering point of a chain.
//  * No wait is unbounded and nothing traps.  A wait that runs out of time
//    records Status::Timeout in `ctx.status[0]` (when given) and returns; an
//    endpoint kind this header cannot serve records Status::Malformed.
//  * The queue transports (rdma, efa, ionic, proxy) are served through the
//    host-proxy ring (aboleth/proxy_device.cuh) when the handle's kind bits
//    say so.
#pragma once

#include <cstdint>
#include <cuda_runtime.h>

#include "aboleth/abi/endpoint_abi.h"
#include "aboleth/abi/proxy_abi.h"

#ifndef ABOLETH_WAIT_TIMEOUT_NS
// Default bound of every device-side wait: two seconds of %globaltimer.
#define ABOLETH_WAIT_TIMEOUT_NS 2000000000ull
#endif

#define ABOLETH_TIER1_ABI 2
#ifndef ABOLETH_TIER1_GENERATED
// 1 in a copy published by aboleth_b200.device_library (which bakes its options in), 0 in the tree.
#define ABOLETH_TIER1_GENERATED 0
#endif
#define ABOLETH_TIER1_PUT_MANY 1
#define ABOLETH_TIER1_PUT_SIGNAL 1
#define ABOLETH_TIER1_PUT_MANY_FLUSH 1
// ABOLETH_TIER1_SPECIALIZED pins the library to ONE transport: 1 = peer memory, 2 = host-proxy ring
// (the kind bits of an endpoint handle).  A specialised library takes every handle to be of that
// kind, so the per-call test of the kind bits is gone from every operation; the other kind's
// HAS macro is 0 and asking for it at compile time (open_as<Kind>) does not compile.  Undefined:
// both kinds are served and each call dispatches on the handle (reference: docs/TIERS.md:52-66).
#ifdef ABOLETH_TIER1_SPECIALIZED
#if ABOLETH_TIER1_SPECIALIZED != 1 && ABOLETH_TIER1_SPECIALIZED != 2
#error "ABOLETH_TIER1_SPECIALIZED must be 1 (p2p) or 2 (proxy): no other transport is served directly"
#endif
#define ABOLETH_TIER1_HAS_P2P (ABOLETH_TIER1_SPECIALIZED == 1)
#define ABOLETH_TIER1_HAS_PROXY (ABOLETH_TIER1_SPECIALIZED == 2)
#else
#define ABOLETH_TIER1_HAS_P2P 1
#define ABOLETH_TIER1_HAS_PROXY 1
#endif
#define ABOLETH_TIER1_HAS_RDMA 0
#define ABOLETH_TIER1_BOUNDED_WAITS 1
#define ABOLETH_TIER1_SMALL_INLINE 1
#ifndef ABOLETH_TIER1_ENDPOINTS_PER_PEER
// Endpoints (lanes) per peer in the handle table: entry peer * N + blockIdx.x % N is used.
#define ABOLETH_TIER1_ENDPOINTS_PER_PEER 1
#endif

#ifdef ABOLETH_DEBUG_BOUNDS
#include "aboleth/debug_bounds.h"
#endif

namespace aboleth {

using abi::PutDesc;

enum class Status : std::uint32_t {
    Ok = 0,
    Timeout = 1,
    CompletionFailure = 2,
    Malformed = 3,
};

struct LocalRegion {
    std::uint64_t address;
    std::uint32_t key;
};

struct RemoteRegion {
    std::uint64_t address;
    std::uint32_t key;
};

// Kernel-argument view of one rank's endpoints.  `endpoints[peer]` is the
// handle table World.exchange_regions() returns (low three bits = kind).
// `status`, when non-null, is one 64-bit word that receives the first
// non-zero Status any call on this context produced.
struct DeviceContext {
    const std::uint64_t *endpoints;
    std::uint32_t *doorbell_locks;
    unsigned long long *status = nullptr;
#ifdef ABOLETH_DEBUG_BOUNDS
    debug::Bounds bounds;  // debug builds only: the windows this kernel may write (debug_bounds.h)
#endif
};

struct PeerRef {
    std::uint64_t handle;  // kind bits stripped
    std::uint32_t kind;
};

namespace detail {

#ifdef ABOLETH_TIER1_SPECIALIZED
inline constexpr std::uint32_t kOnlyKind = ABOLETH_TIER1_SPECIALIZED;
#else
inline constexpr std::uint32_t kOnlyKind = ~0u;  // both kinds, chosen per call
#endif

// Is this endpoint peer memory / the host ring?  Constant in a specialised library.
__device__ __forceinline__ bool is_p2p(const PeerRef &ref) {
    return kOnlyKind == ~0u ? ref.kind == abi::kKindP2P : kOnlyKind == abi::kKindP2P;
}
__device__ __forceinline__ bool is_proxy(const PeerRef &ref) {
    return kOnlyKind == ~0u ? ref.kind == abi::kKindProxy : kOnlyKind == abi::kKindProxy;
}

__device__ __forceinline__ std::uint64_t globaltimer_ns() {
    std::uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ std::uint64_t ld_acquire_sys(const std::uint64_t *p) {
    std::uint64_t v;
    asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}

__device__ __forceinline__ std::uint64_t ld_relaxed_sys(const std::uint64_t *p) {
    std::uint64_t v;
    asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}

__device__ __forceinline__ void st_release_sys(std::uint64_t *p, std::uint64_t v) {
    asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}

__device__ __forceinline__ void st_relaxed_sys(std::uint64_t *p, std::uint64_t v) {
    asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}

__device__ __forceinline__ void fence_acq_rel_sys() {
    asm volatile("fence.acq_rel.sys;" ::: "memory");
}

__device__ __forceinline__ uint4 ld_stream16(const void *p) {
    uint4 v;
    asm volatile("ld.global.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p)
                 : "memory");
    return v;
}

__device__ __forceinline__ void st_stream16(void *p, const uint4 &v) {
    asm volatile("st.global.L1::no_allocate.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p),
                 "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
                 : "memory");
}

__device__ __forceinline__ void record(const DeviceContext &ctx, Status s) {
    if (ctx.status != nullptr && s != Status::Ok)
        atomicCAS(ctx.status, 0ull, static_cast<unsigned long long>(s));
}

// Debug builds: may this context write [address, address + bytes) on a peer?  A refused
// destination is recorded (status Malformed; address, bytes and a count for the host) and
// the caller skips the access.  Release builds always answer yes and compile to nothing.
__device__ __forceinline__ bool may_write(const DeviceContext &ctx, std::uint64_t address,
                                          std::uint64_t bytes) {
#ifdef ABOLETH_DEBUG_BOUNDS
    if (!debug::inside(ctx.bounds, address, bytes)) {
        record(ctx, Status::Malformed);
        if (ctx.bounds.violation != nullptr &&
            atomicAdd(ctx.bounds.violation + 2, 1ull) == 0ull) {
            ctx.bounds.violation[0] = address;
            ctx.bounds.violation[1] = bytes;
        }
        return false;
    }
#else
    (void)ctx;
    (void)address;
    (void)bytes;
#endif
    return true;
}

// Copy `bytes` with `nthreads` cooperating threads (this thread is `tid`).
// 16-byte vectors, four in flight per thread, when everything is 16-byte
// aligned; 8-byte words when 8-byte aligned; bytes otherwise.
__device__ __forceinline__ void copy_strided(
    std::uint8_t *dst, const std::uint8_t *src, std::uint64_t bytes,
    unsigned tid, unsigned nthreads) {
    const std::uint64_t mix =
        reinterpret_cast<std::uint64_t>(dst) | reinterpret_cast<std::uint64_t>(src);
    if ((mix & 15) == 0) {
        const std::uint64_t vecs = bytes >> 4;
        std::uint64_t i = tid;
        for (; i + 3ull * nthreads < vecs; i += 4ull * nthreads) {
            uint4 a = ld_stream16(src + (i << 4));
            uint4 b = ld_stream16(src + ((i + nthreads) << 4));
            uint4 c = ld_stream16(src + ((i + 2ull * nthreads) << 4));
            uint4 d = ld_stream16(src + ((i + 3ull * nthreads) << 4));
            st_stream16(dst + (i << 4), a);
            st_stream16(dst + ((i + nthreads) << 4), b);
            st_stream16(dst + ((i + 2ull * nthreads) << 4), c);
            st_stream16(dst + ((i + 3ull * nthreads) << 4), d);
        }
        for (; i < vecs; i += nthreads)
            st_stream16(dst + (i << 4), ld_stream16(src + (i << 4)));
        for (std::uint64_t b = (vecs << 4) + tid; b < bytes; b += nthreads)
            dst[b] = src[b];
    } else if ((mix & 7) == 0) {
        const std::uint64_t words = bytes >> 3;
        for (std::uint64_t i = tid; i < words; i += nthreads)
            reinterpret_cast<std::uint64_t *>(dst)[i] =
                reinterpret_cast<const std::uint64_t *>(src)[i];
        for (std::uint64_t b = (words << 3) + tid; b < bytes; b += nthreads)
            dst[b] = src[b];
    } else {
        for (std::uint64_t b = tid; b < bytes; b += nthreads)
            dst[b] = src[b];
    }
}

// One 16-byte store to a multicast address: NVSwitch replicates it into the same offset of every
// GPU bound to the multicast object (this one included), so a broadcast leaves the GPU once.
__device__ __forceinline__ void st_multicast16(void *multicast, const uint4 &v) {
    asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(multicast),
                 "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
                 : "memory");
}

// copy_strided onto a multicast address (both 16-byte aligned, `bytes` a multiple of 16).  The
// stores are relaxed: publish with a release flag per receiver after a barrier, like any put.
__device__ __forceinline__ void copy_strided_multicast(
    std::uint8_t *multicast, const std::uint8_t *src, std::uint64_t bytes, unsigned tid, unsigned nthreads) {
    const std::uint64_t vecs = bytes >> 4;
    std::uint64_t i = tid;
    for (; i + 3ull * nthreads < vecs; i += 4ull * nthreads) {
        uint4 a = ld_stream16(src + (i << 4));
        uint4 b = ld_stream16(src + ((i + nthreads) << 4));
        uint4 c = ld_stream16(src + ((i + 2ull * nthreads) << 4));
        uint4 d = ld_stream16(src + ((i + 3ull * nthreads) << 4));
        st_multicast16(multicast + (i << 4), a);
        st_multicast16(multicast + ((i + nthreads) << 4), b);
        st_multicast16(multicast + ((i + 2ull * nthreads) << 4), c);
        st_multicast16(multicast + ((i + 3ull * nthreads) << 4), d);
    }
    for (; i < vecs; i += nthreads)
        st_multicast16(multicast + (i << 4), ld_stream16(src + (i << 4)));
}

}  // namespace detail

}  // namespace aboleth

#include "aboleth/proxy_device.cuh"

namespace aboleth {

inline constexpr int kEndpointsPerPeer = ABOLETH_TIER1_ENDPOINTS_PER_PEER;

// The handle table is peer-major with kEndpointsPerPeer entries per peer; a CTA uses the
// entry its block index selects, so CTAs spread over a peer's endpoints.
__device__ __forceinline__ PeerRef open(const DeviceContext &ctx, int peer) {
    const int slot = kEndpointsPerPeer == 1 ? 0 : static_cast<int>(blockIdx.x % kEndpointsPerPeer);
    const std::uint64_t raw = ctx.endpoints[peer * kEndpointsPerPeer + slot];
    return PeerRef{raw & ~abi::kKindMask, static_cast<std::uint32_t>(raw & abi::kKindMask)};
}

// Does this build of the library serve endpoints of `Kind`?
template <std::uint32_t Kind>
inline constexpr bool kServes = detail::kOnlyKind == ~0u ? (Kind == abi::kKindP2P || Kind == abi::kKindProxy)
                                                         : Kind == detail::kOnlyKind;

// `open` for code that is written for one transport: it does not compile against a library that
// was specialised for another.
template <std::uint32_t Kind>
__device__ __forceinline__ PeerRef open_as(const DeviceContext &ctx, int peer) {
    static_assert(kServes<Kind>, "this Tier-1 library was specialised for another transport");
    PeerRef ref = open(ctx, peer);
    ref.kind = Kind;
    return ref;
}

// ---- bounded receiver-side wait ------------------------------------------------

// Wait until *flag >= epoch (epochs are monotonic, a later one satisfies an
// earlier wait) or `timeout_ns` of %globaltimer elapsed.
__device__ __forceinline__ Status wait_signal_status(
    const std::uint64_t *flag, std::uint64_t epoch,
    std::uint64_t timeout_ns = ABOLETH_WAIT_TIMEOUT_NS) {
    if (detail::ld_acquire_sys(flag) >= epoch)
        return Status::Ok;
    // Poll with relaxed loads (cheap), then acquire once the epoch is there.
    const std::uint64_t start = detail::globaltimer_ns();
    unsigned spins = 0;
    while (detail::ld_relaxed_sys(flag) < epoch) {
        if (++spins > 64) {
            __nanosleep(32);
            if ((spins & 15) == 0 && detail::globaltimer_ns() - start > timeout_ns)
                return Status::Timeout;
        }
    }
    return detail::ld_acquire_sys(flag) >= epoch ? Status::Ok : Status::Timeout;
}

__device__ __forceinline__ void wait_signal(
    const DeviceContext &ctx, const std::uint64_t *flag, std::uint64_t epoch) {
    detail::record(ctx, wait_signal_status(flag, epoch));
}

// ---- single-thread forms (the Tier-1 contract: any one thread may call) --------

__device__ __forceinline__ void put(
    const DeviceContext &ctx, const PeerRef &ref, const RemoteRegion &dst,
    const LocalRegion &src, std::uint32_t bytes) {
    if (detail::is_p2p(ref)) {
        if (!detail::may_write(ctx, dst.address, bytes))
            return;
        detail::copy_strided(reinterpret_cast<std::uint8_t *>(dst.address),
                             reinterpret_cast<const std::uint8_t *>(src.address),
                             bytes, 0, 1);
    } else if (detail::is_proxy(ref)) {
        abi::ProxyCommand cmd{src.address, dst.address, bytes, src.key, dst.key,
                              abi::kProxyCommandWrite};
        detail::record(ctx, proxy::submit(ref.handle, &cmd, 1, nullptr));
    } else {
        detail::record(ctx, Status::Malformed);
    }
}

__device__ __forceinline__ void put(
    const DeviceContext &ctx, int peer, const RemoteRegion &dst,
    const LocalRegion &src, std::uint32_t bytes) {
    put(ctx, open(ctx, peer), dst, src, bytes);
}

// Eight bytes straight out of a register.
__device__ __forceinline__ void put_inline(
    const DeviceContext &ctx, const PeerRef &ref, const RemoteRegion &dst,
    std::uint64_t value) {
    if (detail::is_p2p(ref)) {
        if (!detail::may_write(ctx, dst.address, 8))
            return;
        detail::st_relaxed_sys(reinterpret_cast<std::uint64_t *>(dst.address), value);
    } else if (detail::is_proxy(ref)) {
        // The ring carries an 8-byte inline value as a weak signal command.
        abi::ProxyCommand cmd{value, dst.address, 8, 0, dst.key,
                              abi::kProxyCommandWeakSignal};
        detail::record(ctx, proxy::submit(ref.handle, &cmd, 1, nullptr));
    } else {
        detail::record(ctx, Status::Malformed);
    }
}

__device__ __forceinline__ void put_inline(
    const DeviceContext &ctx, int peer, const RemoteRegion &dst, std::uint64_t value) {
    put_inline(ctx, open(ctx, peer), dst, value);
}

// The low `bytes` (1, 2, 3, 4 or 8) of `value`, little endian.  Peer memory takes any of
// them as plain stores; the ring carries only whole 8-byte values.
__device__ __forceinline__ void put_inline_small(
    const DeviceContext &ctx, const PeerRef &ref, const RemoteRegion &dst,
    std::uint64_t value, int bytes) {
    if (bytes == 8) {
        put_inline(ctx, ref, dst, value);
    } else if (detail::is_p2p(ref) && bytes >= 1 && bytes <= 4) {
        volatile std::uint8_t *out = reinterpret_cast<volatile std::uint8_t *>(dst.address);
        for (int i = 0; i < bytes; ++i)
            out[i] = static_cast<std::uint8_t>(value >> (8 * i));
    } else {
        detail::record(ctx, Status::Malformed);
    }
}

// Strong publication: a peer that observes `epoch` in `flag` observes every
// store this thread made to that peer before the call.
__device__ __forceinline__ void signal(
    const DeviceContext &ctx, const PeerRef &ref, const RemoteRegion &flag,
    std::uint64_t epoch) {
    if (detail::is_p2p(ref)) {
        if (!detail::may_write(ctx, flag.address, 8))
            return;
        detail::st_release_sys(reinterpret_cast<std::uint64_t *>(flag.address), epoch);
    } else if (detail::is_proxy(ref)) {
        abi::ProxyCommand cmd{epoch, flag.address, 8, 0, flag.key,
                              abi::kProxyCommandStrongSignal};
        detail::record(ctx, proxy::submit(ref.handle, &cmd, 1, nullptr));
    } else {
        detail::record(ctx, Status::Malformed);
    }
}

__device__ __forceinline__ void signal(
    const DeviceContext &ctx, int peer, const RemoteRegion &flag, std::uint64_t epoch) {
    signal(ctx, open(ctx, peer), flag, epoch);
}

// put then signal as ONE chain: one release (p2p) or one two-command batch
// with a single reservation and a single ready store (proxy).
__device__ __forceinline__ void put_signal(
    const DeviceContext &ctx, const PeerRef &ref, const RemoteRegion &dst,
    const LocalRegion &src, std::uint32_t bytes, const RemoteRegion &flag,
    std::uint64_t epoch) {
    if (detail::is_p2p(ref)) {
        if (!detail::may_write(ctx, dst.address, bytes) || !detail::may_write(ctx, flag.address, 8))
            return;
        detail::copy_strided(reinterpret_cast<std::uint8_t *>(dst.address),
                             reinterpret_cast<const std::uint8_t *>(src.address),
                             bytes, 0, 1);
        detail::st_release_sys(reinterpret_cast<std::uint64_t *>(flag.address), epoch);
    } else if (detail::is_proxy(ref)) {
        abi::ProxyCommand cmds[2] = {
            {src.address, dst.address, bytes, src.key, dst.key, abi::kProxyCommandWrite},
            {epoch, flag.address, 8, 0, flag.key, abi::kProxyCommandStrongSignal}};
        detail::record(ctx, proxy::submit(ref.handle, cmds, 2, nullptr));
    } else {
        detail::record(ctx, Status::Malformed);
    }
}

__device__ __forceinline__ void put_signal(
    const DeviceContext &ctx, int peer, const RemoteRegion &dst,
    const LocalRegion &src, std::uint32_t bytes, const RemoteRegion &flag,
    std::uint64_t epoch) {
    put_signal(ctx, open(ctx, peer), dst, src, bytes, flag, epoch);
}

// `count` puts as one batch; nothing is published.
__device__ __forceinline__ void put_many(
    const DeviceContext &ctx, const PeerRef &ref, const PutDesc *descs, int count) {
    if (detail::is_p2p(ref)) {
        for (int i = 0; i < count; ++i)
            detail::copy_strided(reinterpret_cast<std::uint8_t *>(descs[i].dst),
                                 reinterpret_cast<const std::uint8_t *>(descs[i].src),
                                 descs[i].bytes, 0, 1);
    } else if (detail::is_proxy(ref)) {
        detail::record(ctx, proxy::submit_puts(ref.handle, descs, count, nullptr, 0, nullptr));
    } else {
        detail::record(ctx, Status::Malformed);
    }
}

// `count` puts closed by ONE signal: the chain pays one release / one
// reservation, however long it is.
__device__ __forceinline__ void put_many_signal(
    const DeviceContext &ctx, const PeerRef &ref, const PutDesc *descs, int count,
    const RemoteRegion &flag, std::uint64_t epoch) {
    if (detail::is_p2p(ref)) {
        for (int i = 0; i < count; ++i)
            detail::copy_strided(reinterpret_cast<std::uint8_t *>(descs[i].dst),
                                 reinterpret_cast<const std::uint8_t *>(descs[i].src),
                                 descs[i].bytes, 0, 1);
        detail::st_release_sys(reinterpret_cast<std::uint64_t *>(flag.address), epoch);
    } else if (detail::is_proxy(ref)) {
        detail::record(ctx, proxy::submit_puts(ref.handle, descs, count, &flag, epoch, nullptr));
    } else {
        detail::record(ctx, Status::Malformed);
    }
}

// Sender-side completion of everything posted to the peer so far.  Peer
// stores read their source when they issue, so on p2p the source is already
// reusable and this is a no-op; on the ring it waits for the host to retire
// the last batch this endpoint reserved.
__device__ __forceinline__ void quiet(const DeviceContext &ctx, const PeerRef &ref) {
    if (detail::is_proxy(ref))
        detail::record(ctx, proxy::drain(ref.handle));
    else if (!detail::is_p2p(ref))
        detail::record(ctx, Status::Malformed);
}

__device__ __forceinline__ void quiet(const DeviceContext &ctx, int peer) {
    quiet(ctx, open(ctx, peer));
}

__device__ __forceinline__ void put_many_flush(
    const DeviceContext &ctx, const PeerRef &ref, const PutDesc *descs, int count) {
    put_many(ctx, ref, descs, count);
    quiet(ctx, ref);
}

// ---- cooperative forms (p2p only) -----------------------------------------------

// One full warp copies; ends with a warp barrier and a system fence so the
// bytes are placed when the call returns (no signal has to follow).
__device__ __forceinline__ void put_warp(
    const DeviceContext &ctx, const PeerRef &ref, const RemoteRegion &dst,
    const LocalRegion &src, std::uint32_t bytes) {
    if (!detail::is_p2p(ref)) {
        if ((threadIdx.x & 31) == 0)
            put(ctx, ref, dst, src, bytes);
        __syncwarp();
        return;
    }
    if (detail::may_write(ctx, dst.address, bytes))  // warp-uniform: every lane sees the same arguments
        detail::copy_strided(reinterpret_cast<std::uint8_t *>(dst.address),
                             reinterpret_cast<const std::uint8_t *>(src.address), bytes,
                             threadIdx.x & 31, 32);
    __syncwarp();
    detail::fence_acq_rel_sys();
}

// The whole CTA copies.  No fence: a following signal_block publishes it.
__device__ __forceinline__ void put_block(
    const RemoteRegion &dst, const LocalRegion &src, std::uint64_t bytes) {
    const unsigned tid = threadIdx.x + blockDim.x * (threadIdx.y + blockDim.y * threadIdx.z);
    const unsigned n = blockDim.x * blockDim.y * blockDim.z;
    detail::copy_strided(reinterpret_cast<std::uint8_t *>(dst.address),
                         reinterpret_cast<const std::uint8_t *>(src.address), bytes, tid, n);
}

// CTA barrier, then one thread's fence + release store: every thread's earlier
// peer stores are visible to whoever acquires `epoch` from `flag`.  The CTA
// barrier orders the CTA's stores before thread 0 (CTA-scope causality), and
// the system-scope fence makes that order cumulative for the remote observer.
__device__ __forceinline__ void signal_block(const RemoteRegion &flag, std::uint64_t epoch) {
    __syncthreads();
    if (threadIdx.x == 0 && threadIdx.y == 0 && threadIdx.z == 0) {
        detail::fence_acq_rel_sys();
        detail::st_relaxed_sys(reinterpret_cast<std::uint64_t *>(flag.address), epoch);
    }
}

// ---- compile-time peer forms ---------------------------------------------------------------

template <int Peer>
__device__ __forceinline__ void put(const DeviceContext &ctx, const RemoteRegion &dst,
                                    const LocalRegion &src, std::uint32_t bytes) {
    put(ctx, open(ctx, Peer), dst, src, bytes);
}

template <int Peer>
__device__ __forceinline__ void signal(const DeviceContext &ctx, const RemoteRegion &flag,
                                       std::uint64_t epoch) {
    signal(ctx, open(ctx, Peer), flag, epoch);
}

template <int Peer>
__device__ __forceinline__ void put_signal(const DeviceContext &ctx, const RemoteRegion &dst,
                                           const LocalRegion &src, std::uint32_t bytes,
                                           const RemoteRegion &flag, std::uint64_t epoch) {
    put_signal(ctx, open(ctx, Peer), dst, src, bytes, flag, epoch);
}

template <int Peer>
__device__ __forceinline__ void quiet(const DeviceContext &ctx) {
    quiet(ctx, open(ctx, Peer));
}

}  // namespace aboleth
