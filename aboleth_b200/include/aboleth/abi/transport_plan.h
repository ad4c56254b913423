// Publication modes, phase deadlines and the 112-byte phase-plan record.
//
// Field order, sizes and enumerator values follow the reference project
// (include/aboleth/Target/TransportPlan.h:16-227) so a plan blob written by
// either side can be read by the other.
#pragma once

#include <cstdint>
#include <type_traits>

#include "aboleth/abi/transport_caps.h"

namespace aboleth::abi {

inline constexpr std::uint32_t kTransportPhasePlanVersion = 4;
inline constexpr std::uint32_t kTransportNoPhase = 0xffffffffu;

enum class TransportTopologyKind : std::uint32_t { AllNIC = 0, Mixed = 1, AllP2P = 2 };
enum class TransportQp0Role : std::uint32_t { Data = 0, Control = 1 };

// How a strong publication makes payload visible before its epoch.
enum class TransportPublicationMode : std::uint32_t {
    SameQueueStrong = 0,       // responder atomic behind the payload on one queue
    P2PRelease = 1,            // release store orders the prior peer stores
    GinSignal = 2,
    FenceThenSignal = 3,       // retire payload completions, then signal
    ImmCounting = 4,           // receiver counts write-with-immediate arrivals
    SameQueueFencedWrite = 5,  // fenced write; needs strictly ordered registrations
};

enum class TransportBarrierKind : std::uint32_t { None = 0, Transport = 1, NativeP2P = 2 };

enum class TransportEffectPhase : std::uint32_t {
    Dispatch = 0, Experts = 1, Combine = 2, NextPack = 3, Count = 4,
};

inline constexpr std::uint32_t kTransportPlanFirstUse = 1u << 0;
inline constexpr std::uint32_t kTransportPlanReuseSafe = 1u << 1;
inline constexpr std::uint32_t kTransportPlanQpExclusive = 1u << 2;
inline constexpr std::uint32_t kTransportPlanDrainAtEpilogue = 1u << 3;
inline constexpr std::uint32_t kTransportPlanGroupedCompletion = 1u << 4;
inline constexpr std::uint32_t kTransportPlanCompletionLeader = 1u << 5;

// The strongest-necessary publication a transport can perform, derived from
// its capability row alone.
AB_HD inline constexpr TransportPublicationMode legal_strong_publication(
    const TransportCaps &caps, bool prefer_imm,
    bool strict_registrations = false) {
    if (caps.load_store_addressable)
        return TransportPublicationMode::P2PRelease;
    if (!caps.ordered_delivery)
        return (prefer_imm && caps.imm_data)
                   ? TransportPublicationMode::ImmCounting
                   : TransportPublicationMode::FenceThenSignal;
    if (strict_registrations && caps.fenced_write)
        return TransportPublicationMode::SameQueueFencedWrite;
    return caps.native_atomics ? TransportPublicationMode::SameQueueStrong
                               : TransportPublicationMode::FenceThenSignal;
}

// Only a remote compare-and-swap can verify the predecessor epoch.
AB_HD inline constexpr bool publication_is_checked(const TransportCaps &caps) {
    return caps.native_atomics && !caps.load_store_addressable;
}

// Is a deadline stated as "before phase P, `delta` iterations later" due when
// the program enters `phase` at 1-based iteration `iteration`?
AB_HD inline constexpr bool transport_deadline_due(
    TransportEffectPhase phase, std::uint64_t iteration,
    std::uint32_t before_phase, std::uint32_t iteration_delta) {
    if (before_phase == kTransportNoPhase ||
        before_phase != static_cast<std::uint32_t>(phase))
        return false;
    return iteration_delta == 0 || iteration > iteration_delta;
}

struct alignas(8) TransportPhasePlan {
    std::uint32_t abi_version;
    std::uint32_t byte_size;
    std::uint32_t active_qps;
    std::uint32_t data_qps;
    std::uint32_t data_wqe_bound;
    std::uint32_t data_reclaim_interval;
    std::uint32_t control_wqe_bound;
    std::uint32_t control_reclaim_interval;
    std::uint32_t topology_kind;
    std::uint32_t qp0_role;
    std::uint32_t publication_mode;
    std::uint32_t prologue_barrier_kind;
    std::uint32_t epilogue_barrier_kind;
    std::uint32_t flags;
    std::uint32_t publication_before_phase;
    std::uint32_t publication_iteration_delta;
    std::uint32_t completion_before_phase;
    std::uint32_t completion_iteration_delta;
    std::uint32_t first_overwrite_phase;
    std::uint32_t first_overwrite_iteration_delta;
    std::uint32_t reclaim_before_phase;
    std::uint32_t reclaim_iteration_delta;
    std::uint32_t payload_bytes;
    std::uint32_t path_mtu;
    std::uint32_t completion_interval;
    std::uint32_t buffer_slots;
    std::uint32_t payload_commit_tokens;
    std::uint32_t reserved;
};

static_assert(std::is_standard_layout_v<TransportPhasePlan>);
static_assert(std::is_trivially_copyable_v<TransportPhasePlan>);
static_assert(sizeof(TransportPhasePlan) == 112);

static_assert(legal_strong_publication(*lookup_transport_caps("p2p"), true) ==
              TransportPublicationMode::P2PRelease);
static_assert(legal_strong_publication(*lookup_transport_caps("rdma"), false) ==
              TransportPublicationMode::SameQueueStrong);
static_assert(legal_strong_publication(*lookup_transport_caps("rdma"), false, true) ==
              TransportPublicationMode::SameQueueFencedWrite);
static_assert(legal_strong_publication(*lookup_transport_caps("proxy"), false, true) ==
              TransportPublicationMode::SameQueueStrong);
static_assert(legal_strong_publication(*lookup_transport_caps("ionic"), false) ==
              TransportPublicationMode::FenceThenSignal);
static_assert(legal_strong_publication(*lookup_transport_caps("efa"), false) ==
              TransportPublicationMode::FenceThenSignal);
static_assert(legal_strong_publication(*lookup_transport_caps("efa"), true) ==
              TransportPublicationMode::ImmCounting);
static_assert(publication_is_checked(*lookup_transport_caps("rdma")));
static_assert(!publication_is_checked(*lookup_transport_caps("p2p")));
static_assert(transport_deadline_due(TransportEffectPhase::NextPack, 1, 3, 0));
static_assert(!transport_deadline_due(TransportEffectPhase::Experts, 1, 1, 1));
static_assert(transport_deadline_due(TransportEffectPhase::Experts, 2, 1, 1));

}  // namespace aboleth::abi
