// Host-proxy ring ABI.
//
// A GPU producer reserves one sequence number per batch, writes up to 256
// 32-byte commands into slot `sequence % 64` of a host-pinned queue, and
// release-stores `ready_sequence`.  A host progress thread consumes slots
// strictly in sequence order and release-publishes `completed_sequence`
// (also after a failure, so device waiters terminate).  Sizes and offsets are
// those of the reference project (include/aboleth/Target/ProxyAbi.h:9-89).
#pragma once

#include <cstddef>
#include <cstdint>
#include <type_traits>

namespace aboleth::abi {

inline constexpr std::uint32_t kProxyEndpointVersion = 8;
inline constexpr std::uint32_t kProxySlotCount = 64;
inline constexpr std::uint32_t kProxyMaximumCommands = 256;

inline constexpr std::uint32_t kProxyCommandNop = 0;
inline constexpr std::uint32_t kProxyCommandWrite = 1;
inline constexpr std::uint32_t kProxyCommandWeakSignal = 2;
inline constexpr std::uint32_t kProxyCommandStrongSignal = 3;

// Endpoint status word.  An endpoint is discarded after a non-zero status.
inline constexpr std::uint64_t kEndpointStatusOk = 0;
inline constexpr std::uint64_t kEndpointStatusTimeout = 1;
inline constexpr std::uint64_t kEndpointStatusCompletionFailure = 2;
inline constexpr std::uint64_t kEndpointStatusMalformed = 3;

struct alignas(8) ProxyCommand {
    std::uint64_t source_address;       // signals carry their value here
    std::uint64_t destination_address;
    std::uint32_t bytes;
    std::uint32_t source_key;
    std::uint32_t destination_key;
    std::uint32_t opcode;
};

struct alignas(8) ProxyBatchSlot {
    std::uint64_t ready_sequence;  // sequence + 1 once the slot is complete
    std::uint32_t command_count;
    std::uint32_t reserved;
    ProxyCommand commands[kProxyMaximumCommands];
};

struct alignas(8) ProxyQueueState {
    std::uint64_t completed_sequence;
    std::uint64_t status;
    ProxyBatchSlot slots[kProxySlotCount];
};

struct alignas(8) ProxyEndpointDescriptor {
    std::uint64_t queue_state;              // device-visible address of ProxyQueueState
    std::uint64_t producer_index_address;   // GPU-resident 64-bit reservation counter
    std::uint64_t completion_timeout_cycles;
    std::uint32_t slot_count;
    std::uint32_t slot_stride;
    std::uint32_t maximum_commands;
    std::uint32_t abi_version;
};

#define AB_LAYOUT(T, SIZE)                           \
    static_assert(std::is_standard_layout_v<T>);     \
    static_assert(std::is_trivially_copyable_v<T>);  \
    static_assert(alignof(T) == 8);                  \
    static_assert(sizeof(T) == SIZE)

AB_LAYOUT(ProxyCommand, 32);
AB_LAYOUT(ProxyBatchSlot, 8208);
AB_LAYOUT(ProxyQueueState, 525328);
AB_LAYOUT(ProxyEndpointDescriptor, 40);
#undef AB_LAYOUT

static_assert(offsetof(ProxyCommand, bytes) == 16);
static_assert(offsetof(ProxyCommand, opcode) == 28);
static_assert(offsetof(ProxyBatchSlot, command_count) == 8);
static_assert(offsetof(ProxyBatchSlot, commands) == 16);
static_assert(offsetof(ProxyQueueState, status) == 8);
static_assert(offsetof(ProxyQueueState, slots) == 16);
static_assert(offsetof(ProxyEndpointDescriptor, producer_index_address) == 8);
static_assert(offsetof(ProxyEndpointDescriptor, completion_timeout_cycles) == 16);
static_assert(offsetof(ProxyEndpointDescriptor, slot_count) == 24);
static_assert(offsetof(ProxyEndpointDescriptor, abi_version) == 36);

}  // namespace aboleth::abi
