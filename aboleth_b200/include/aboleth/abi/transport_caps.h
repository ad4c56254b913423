// Transport capability registry.
//
// Planning code never asks "which transport is this"; it asks what the
// transport can do.  Each row answers the fourteen questions the planners
// and the emitters need.  The rows and field meanings match the table in the
// reference project (include/aboleth/Target/TransportCaps.h:46-187) so that
// plans computed here agree with plans computed there.
//
// On a B200 NVSwitch box only the `p2p` row is a product path.  `proxy` is the
// host-thread fallback that makes the queue-transport names usable without a
// NIC; `rdma`, `efa` and `ionic` rows exist so that programs written against
// those names still plan, emit and (through the proxy) run.
#pragma once

#include <cstddef>
#include <cstdint>

#if defined(__CUDACC__)
#define AB_HD __host__ __device__
#else
#define AB_HD
#endif

namespace aboleth::abi {

enum class TransportCompletionModel : std::uint32_t {
    None = 0,            // program order is completion (peer memory)
    OrderedCounter = 1,  // one completion retires everything before it
    UnorderedCount = 2,  // a batch retires after N completions were counted
};

enum class TransportDoorbellModel : std::uint32_t {
    None = 0,
    BlueFlame = 1,  // one ordered 64-bit MMIO store
    HostRing = 2,   // host progress thread consumes a ring
    Doorbell = 3,   // doorbell register after the queue entries
};

struct TransportCaps {
    const char *name;
    bool gpu_initiated;            // the kernel itself submits
    bool load_store_addressable;   // remote memory is ld/st reachable: no queue
    bool ordered_delivery;         // one endpoint delivers in submission order
    bool native_atomics;           // remote compare-and-swap exists
    bool fenced_write;             // a write may wait for all earlier commands
    bool imm_data;                 // write-with-immediate exists
    bool queue_capacity_limited;   // outstanding work bounded by a queue
    bool selective_completion;     // one completion can cover a batch
    std::uint32_t max_inline_bytes;
    std::uint32_t default_completion_interval;  // 0: whole phase retires once
    TransportCompletionModel completion_model;
    TransportDoorbellModel doorbell_model;
    std::uint32_t path_mtu;
    std::uint32_t max_data_queues;
};

using CM = TransportCompletionModel;
using DM = TransportDoorbellModel;

inline constexpr TransportCaps kTransportCaps[] = {
    //  name    gpu    ld/st  order  atom   fence  imm    qcap   selc  inl ivl  completion          doorbell       mtu  q
    {"p2p",    true,  true,  true,  true,  false, false, false, true,  0,  0,  CM::None,           DM::None,      0,    0},
    {"proxy",  false, false, true,  true,  false, false, false, true,  8,  8,  CM::OrderedCounter, DM::HostRing,  4096, 0},
    {"rdma",   true,  false, true,  true,  true,  false, true,  true,  28, 16, CM::OrderedCounter, DM::BlueFlame, 4096, 0},
    {"ionic",  true,  false, true,  false, true,  false, true,  false, 16, 8,  CM::OrderedCounter, DM::Doorbell,  4096, 0},
    {"efa",    true,  false, false, false, false, true,  true,  false, 0,  16, CM::UnorderedCount, DM::Doorbell,  4096, 0},
};

inline constexpr std::size_t kTransportCapsCount =
    sizeof(kTransportCaps) / sizeof(kTransportCaps[0]);

// `name` need not be NUL terminated: `length` bytes are compared and the
// table entry must end exactly there.
AB_HD inline constexpr const TransportCaps *lookup_transport_caps(
    const char *name, std::size_t length) {
    for (std::size_t row = 0; row < kTransportCapsCount; ++row) {
        const char *candidate = kTransportCaps[row].name;
        std::size_t i = 0;
        while (i < length && candidate[i] != '\0' && candidate[i] == name[i])
            ++i;
        if (i == length && candidate[i] == '\0')
            return &kTransportCaps[row];
    }
    return nullptr;
}

AB_HD inline constexpr const TransportCaps *lookup_transport_caps(
    const char *name) {
    std::size_t length = 0;
    while (name[length] != '\0')
        ++length;
    return lookup_transport_caps(name, length);
}

struct TransportCostParams {
    std::uint32_t path_mtu;
    std::uint32_t completion_units_per_command;  // 0 with selective completion
    std::uint32_t max_data_queues;
};

AB_HD inline constexpr TransportCostParams transport_cost_params(
    const TransportCaps &caps) {
    return {caps.path_mtu, caps.selective_completion ? 0u : 1u,
            caps.max_data_queues};
}

AB_HD inline constexpr TransportCostParams default_transport_cost_params() {
    return transport_cost_params(*lookup_transport_caps("rdma"));
}

static_assert(kTransportCapsCount == 5);
static_assert(lookup_transport_caps("p2p")->load_store_addressable);
static_assert(!lookup_transport_caps("p2p")->queue_capacity_limited);
static_assert(lookup_transport_caps("proxy")->max_inline_bytes == 8);
static_assert(lookup_transport_caps("rdma")->max_inline_bytes == 28);
static_assert(!lookup_transport_caps("efa")->ordered_delivery);
static_assert(lookup_transport_caps("efa")->imm_data);
static_assert(lookup_transport_caps("nvshmem") == nullptr);
static_assert(lookup_transport_caps("rdm", 3) == nullptr);
static_assert(lookup_transport_caps("rdmaX", 4) == lookup_transport_caps("rdma"));
static_assert(default_transport_cost_params().path_mtu == 4096);

}  // namespace aboleth::abi
