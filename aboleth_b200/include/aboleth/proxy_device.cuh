// Device side of the host-proxy ring (layouts: aboleth/abi/proxy_abi.h).
//
// One batch = one sequence reservation, `count` 32-byte commands written as
// four 64-bit stores each, one `st.release.sys` of ready_sequence.  The
// protocol is the reference's (docs/PROXY_ABI.md:53-69,
// include/aboleth/Target/ProxyDevice.cuh:49-189); unlike it, a wait that runs
// out of time returns Status::Timeout instead of printing and trapping.
#pragma once

#include <cstdint>

#include "aboleth/abi/proxy_abi.h"

namespace aboleth {

struct RemoteRegion;
enum class Status : std::uint32_t;

namespace proxy {

__device__ __forceinline__ const abi::ProxyEndpointDescriptor &descriptor(std::uint64_t handle) {
    return *reinterpret_cast<const abi::ProxyEndpointDescriptor *>(handle);
}

__device__ __forceinline__ std::uint64_t timeout_ns(const abi::ProxyEndpointDescriptor &d) {
    // The descriptor states cycles; at ~2 GHz a cycle is about half a
    // nanosecond.  Zero means the build default.
    return d.completion_timeout_cycles == 0 ? ABOLETH_WAIT_TIMEOUT_NS
                                            : (d.completion_timeout_cycles >> 1) + 1;
}

// Wait until the host retired sequence `target - 1` (completed >= target).
__device__ __forceinline__ Status wait_completed(
    const abi::ProxyEndpointDescriptor &d, std::uint64_t target) {
    auto *state = reinterpret_cast<abi::ProxyQueueState *>(d.queue_state);
    const std::uint64_t limit = timeout_ns(d);
    const std::uint64_t start = detail::globaltimer_ns();
    while (true) {
        if (detail::ld_acquire_sys(&state->completed_sequence) >= target) {
            return detail::ld_relaxed_sys(&state->status) == 0 ? Status(0) : Status(2);
        }
        __nanosleep(128);
        if (detail::globaltimer_ns() - start > limit)
            return Status(1);
    }
}

// Reserve one sequence and wait until its slot is free.
__device__ __forceinline__ Status reserve(
    const abi::ProxyEndpointDescriptor &d, std::uint64_t *sequence) {
    auto *producer = reinterpret_cast<unsigned long long *>(d.producer_index_address);
    const std::uint64_t seq = atomicAdd(producer, 1ull);
    *sequence = seq;
    if (seq < d.slot_count)
        return Status(0);
    return wait_completed(d, seq + 1 - d.slot_count);
}

__device__ __forceinline__ abi::ProxyBatchSlot *slot_of(
    const abi::ProxyEndpointDescriptor &d, std::uint64_t seq) {
    return reinterpret_cast<abi::ProxyBatchSlot *>(
        d.queue_state + offsetof(abi::ProxyQueueState, slots) +
        (seq % d.slot_count) * static_cast<std::uint64_t>(d.slot_stride));
}

__device__ __forceinline__ void write_command(
    abi::ProxyBatchSlot *slot, int index, const abi::ProxyCommand &c) {
    auto *w = reinterpret_cast<std::uint64_t *>(&slot->commands[index]);
    detail::st_relaxed_sys(w + 0, c.source_address);
    detail::st_relaxed_sys(w + 1, c.destination_address);
    detail::st_relaxed_sys(w + 2, static_cast<std::uint64_t>(c.bytes) |
                                      (static_cast<std::uint64_t>(c.source_key) << 32));
    detail::st_relaxed_sys(w + 3, static_cast<std::uint64_t>(c.destination_key) |
                                      (static_cast<std::uint64_t>(c.opcode) << 32));
}

__device__ __forceinline__ void publish(abi::ProxyBatchSlot *slot, std::uint64_t seq, int count) {
    detail::st_relaxed_sys(reinterpret_cast<std::uint64_t *>(&slot->command_count),
                           static_cast<std::uint64_t>(static_cast<std::uint32_t>(count)));
    detail::st_release_sys(&slot->ready_sequence, seq + 1);
}

// Submit `count` prepared commands as one batch.  `last`, when non-null,
// receives the batch's sequence so the caller can poll for exactly it.
__device__ __forceinline__ Status submit(
    std::uint64_t handle, const abi::ProxyCommand *cmds, int count, std::uint64_t *last) {
    const auto &d = descriptor(handle);
    if (d.abi_version != abi::kProxyEndpointVersion || count < 1 ||
        count > static_cast<int>(d.maximum_commands))
        return Status(3);
    std::uint64_t seq;
    const Status s = reserve(d, &seq);
    if (last != nullptr)
        *last = seq;
    if (s != Status(0))
        return s;
    abi::ProxyBatchSlot *slot = slot_of(d, seq);
    for (int i = 0; i < count; ++i)
        write_command(slot, i, cmds[i]);
    publish(slot, seq, count);
    return Status(0);
}

// `count` puts, optionally closed by one strong signal, as one batch.
__device__ __forceinline__ Status submit_puts(
    std::uint64_t handle, const abi::PutDesc *descs, int count,
    const RemoteRegion *flag, std::uint64_t epoch, std::uint64_t *last);

// Wait until every batch reserved so far on this endpoint has retired.
__device__ __forceinline__ Status drain(std::uint64_t handle) {
    const auto &d = descriptor(handle);
    auto *producer = reinterpret_cast<std::uint64_t *>(d.producer_index_address);
    const std::uint64_t reserved = detail::ld_relaxed_sys(producer);
    if (reserved == 0)
        return Status(0);
    return wait_completed(d, reserved);
}

// Wait until the batch with sequence `seq` retired.
__device__ __forceinline__ Status poll(std::uint64_t handle, std::uint64_t seq) {
    return wait_completed(descriptor(handle), seq + 1);
}

}  // namespace proxy
}  // namespace aboleth

// submit_puts needs the complete RemoteRegion, which device.cuh defines before
// it includes this header.
namespace aboleth::proxy {
__device__ __forceinline__ Status submit_puts(
    std::uint64_t handle, const abi::PutDesc *descs, int count,
    const RemoteRegion *flag, std::uint64_t epoch, std::uint64_t *last) {
    const auto &d = descriptor(handle);
    const int total = count + (flag != nullptr ? 1 : 0);
    if (d.abi_version != abi::kProxyEndpointVersion || total < 1 ||
        total > static_cast<int>(d.maximum_commands))
        return Status(3);
    std::uint64_t seq;
    const Status s = reserve(d, &seq);
    if (last != nullptr)
        *last = seq;
    if (s != Status(0))
        return s;
    abi::ProxyBatchSlot *slot = slot_of(d, seq);
    for (int i = 0; i < count; ++i) {
        abi::ProxyCommand c{descs[i].src, descs[i].dst, descs[i].bytes, descs[i].src_key,
                            descs[i].dst_key, abi::kProxyCommandWrite};
        write_command(slot, i, c);
    }
    if (flag != nullptr) {
        abi::ProxyCommand c{epoch, flag->address, 8, 0, flag->key,
                            abi::kProxyCommandStrongSignal};
        write_command(slot, count, c);
    }
    publish(slot, seq, total);
    return Status(0);
}
}  // namespace aboleth::proxy
