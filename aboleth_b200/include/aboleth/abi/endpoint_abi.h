// Endpoint-level records that travel between ranks or between host and device.
//
// * RdmaEndpointDescriptor — 96-byte device view of an mlx5 queue pair.  No
//   NIC path is built here, but the record is kept so that tools which parse
//   descriptor tables keep working (reference: include/aboleth/Target/RdmaAbi.h:61-99).
// * AbolethConnectionInfo — 128-byte record a rank publishes for each non-P2P
//   endpoint during connect_all (reference: include/aboleth/runtime_c.h:31-54).
// * AbolethEndpointConfig — 96-byte knob block versioned by `struct_size`
//   (reference: include/aboleth/runtime_c.h:63-108).
// * Tier-1 put descriptor and endpoint-handle kind bits
//   (reference: python/aboleth/emit/tier1_header.py:23-31,497-560).
#pragma once

#include <cstddef>
#include <cstdint>
#include <type_traits>

namespace aboleth::abi {

inline constexpr std::uint32_t kRdmaEndpointVersion = 3;
inline constexpr std::uint64_t kMaxInlinePayloadBytes = 972;
inline constexpr std::uint64_t kSingleBlockInlinePayloadBytes = 28;

struct alignas(8) RdmaEndpointDescriptor {
    std::uint64_t send_queue;
    std::uint64_t send_dbrec;
    std::uint64_t blueflame;
    std::uint64_t completion_queue;
    std::uint64_t completion_dbrec;
    std::uint64_t producer_index_address;
    std::uint64_t completion_consumer_address;
    std::uint64_t completion_timeout_cycles;
    std::uint32_t send_stride;
    std::uint32_t send_wqe_count;
    std::uint32_t qpn;
    std::uint32_t completion_entry_size;
    std::uint32_t completion_entry_count;
    std::uint32_t abi_version;
    std::uint32_t atomic_result_lkey;
    std::uint32_t reserved1;
};
static_assert(std::is_standard_layout_v<RdmaEndpointDescriptor>);
static_assert(sizeof(RdmaEndpointDescriptor) == 96);
static_assert(offsetof(RdmaEndpointDescriptor, completion_timeout_cycles) == 56);
static_assert(offsetof(RdmaEndpointDescriptor, send_stride) == 64);
static_assert(offsetof(RdmaEndpointDescriptor, abi_version) == 84);

// Words of the per-endpoint completion-state block.
inline constexpr int kCompletionWordConsumer = 0;
inline constexpr int kCompletionWordCompletedHead = 1;
inline constexpr int kCompletionWordReadyHead = 2;
inline constexpr int kCompletionWordStatus = 3;
inline constexpr int kCompletionWordAtomicResult = 4;

// Low three bits of a device endpoint handle say which transport serves it.
// These are *device kind bits*; the bootstrap wire codes and the native
// connection codes below are two different numberings.
inline constexpr std::uint64_t kKindMask = 7;
inline constexpr std::uint64_t kKindRdma = 0;
inline constexpr std::uint64_t kKindP2P = 1;
inline constexpr std::uint64_t kKindProxy = 2;
inline constexpr std::uint64_t kKindEfa = 3;
inline constexpr std::uint64_t kKindIonic = 4;

// One entry of a put_many batch.
struct alignas(8) PutDesc {
    std::uint64_t dst;
    std::uint64_t src;
    std::uint32_t bytes;
    std::uint32_t dst_key;
    std::uint32_t src_key;
    std::uint32_t pad;
};
static_assert(sizeof(PutDesc) == 32);

}  // namespace aboleth::abi

// ---- C-level records (global namespace, as in the reference C ABI) ---------

constexpr std::uint32_t kAbolethConnectionInfoVersion = 2;
constexpr std::uint32_t kAbolethTransportDirect = 1;
constexpr std::uint32_t kAbolethTransportProxy = 2;
constexpr std::uint32_t kAbolethTransportEfa = 3;
constexpr std::uint32_t kAbolethTransportIonic = 4;
constexpr std::uint32_t kAbolethProxyProviderVerbsRc = 1;
constexpr std::uint32_t kAbolethProxyProviderEfaOfi = 2;
// The NIC-less provider of this build: the proxy thread moves bytes with CUDA
// peer copies.  Not a reference value; chosen outside its range.
constexpr std::uint32_t kAbolethProxyProviderCudaCopy = 16;
constexpr std::size_t kAbolethConnectionAddressBytes = 64;

constexpr std::uint32_t kAbolethProviderVerbs = 1u << 0;
constexpr std::uint32_t kAbolethProviderMlx5 = 1u << 1;
constexpr std::uint32_t kAbolethProviderEfa = 1u << 2;
constexpr std::uint32_t kAbolethProviderLibfabric = 1u << 3;
constexpr std::uint32_t kAbolethProviderCuda = 1u << 4;
constexpr std::uint32_t kAbolethProviderHip = 1u << 5;
constexpr std::uint32_t kAbolethProviderIonic = 1u << 6;

struct AbolethConnectionInfo {
    std::uint32_t abi_version;
    std::uint32_t transport;
    std::uint32_t qpn;
    std::uint32_t psn;
    std::uint32_t gid_index;
    std::uint32_t path_mtu;
    std::uint16_t lid;
    std::uint8_t port_num;
    std::uint8_t link_layer;
    std::uint8_t gid[16];
    std::uint32_t provider;
    std::uint32_t address_format;
    std::uint32_t address_length;
    std::uint32_t reserved0;
    std::uint8_t address[kAbolethConnectionAddressBytes];
    std::uint8_t reserved[4];
};
static_assert(sizeof(AbolethConnectionInfo) == 128);
static_assert(offsetof(AbolethConnectionInfo, gid) == 28);
static_assert(offsetof(AbolethConnectionInfo, address) == 60);

// `struct_size` is sizeof() as the caller's header declares it: smaller is
// accepted (trailing fields default), larger is refused.
struct AbolethEndpointConfig {
    std::uint32_t struct_size;
    std::uint32_t qp_type;        // 0 only
    std::uint32_t qp_depth;       // 0 = runtime default
    std::uint32_t max_inline;     // 0 = environment / default
    std::uint32_t qps_per_peer;   // 0 or 1
    std::uint32_t sm_map_policy;  // 0 only
    std::int32_t port;            // 0 = the runtime's port
    std::int32_t gid_index;       // -1 = the runtime's GID entry
    char hca[64];                 // empty = the runtime's device
};
static_assert(sizeof(AbolethEndpointConfig) == 96);
static_assert(offsetof(AbolethEndpointConfig, hca) == 32);
