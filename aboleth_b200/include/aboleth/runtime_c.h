// C ABI of the native host runtime (libab200_runtime.so).
//
// The entry points that exist in the reference C ABI keep their names and
// argument lists (include/aboleth/runtime_c.h:110-307) so a ctypes or C client
// written against it links here: last_error, provider_caps, create/destroy,
// register/unregister buffer and accessors, create/connect/destroy local
// endpoint and its state/capacity/max_inline/submit_mode queries.  What the
// reference implements with ibverbs is implemented here with CUDA: a
// registration is an entry in the runtime's key table (plus a CUDA IPC export
// on request), and every queue transport is served by the host-proxy ring.
// Adapter / GID / port selection is answered from sysfs rather than through a
// verbs context; endpoint pairs over mlx5/EFA report "unavailable" through
// last_error.
#pragma once

#include <cstddef>
#include <cstdint>

#include "aboleth/abi/endpoint_abi.h"
#include "aboleth/abi/proxy_abi.h"

extern "C" {

const char *aboleth_runtime_last_error();
std::uint32_t aboleth_runtime_provider_caps();

void *aboleth_runtime_create();
void *aboleth_runtime_create_for_device(int gpu_index, const char *hca_name);
const char *aboleth_runtime_hca_name(void *runtime);
int aboleth_runtime_gpu_index(void *runtime);
int aboleth_runtime_port(void *runtime);
int aboleth_runtime_gid_index(void *runtime);
int aboleth_runtime_link_layer(void *runtime);
int aboleth_runtime_lid(void *runtime);
int aboleth_runtime_destroy(void *runtime);

// Adapter, GID and port selection without a runtime, answered from sysfs
// (csrc/host/providers.cpp): the mlx5 adapter sharing the deepest PCI path with
// CUDA ordinal `gpu_index` (ABOLETH_HCA overrides; negative = first adapter), the
// GID index a verbs client would address the fabric through (InfiniBand 0, RoCE
// prefers a v2 entry, ABOLETH_GID_INDEX overrides; port 0 = ABOLETH_PORT or 1), and
// the local address of an RC path (link layer 1 InfiniBand / 2 Ethernet, path MTU
// as an ibv_mtu enumerator, honouring ABOLETH_PATH_MTU).  Each returns -1 with
// aboleth_runtime_last_error() when the machine presents no such adapter.
int aboleth_runtime_select_device(int gpu_index, char *name_out, std::size_t name_capacity);
int aboleth_runtime_select_gid_index(const char *device_name, int port);
int aboleth_runtime_query_port_address(const char *device_name, int port, std::uint16_t *lid_out,
                                       std::uint8_t *link_layer_out, std::uint8_t *gid_out16,
                                       int *gid_index_out, std::uint32_t *path_mtu_out);

void *aboleth_runtime_register_buffer(void *runtime, int gpu_index, void *address,
                                      std::size_t bytes, std::uint64_t generation);
int aboleth_runtime_unregister_buffer(void *buffer);
std::uint64_t aboleth_runtime_buffer_address(void *buffer);
std::uint64_t aboleth_runtime_buffer_length(void *buffer);
std::uint32_t aboleth_runtime_buffer_lkey(void *buffer);
std::uint32_t aboleth_runtime_buffer_rkey(void *buffer);
int aboleth_runtime_buffer_device(void *buffer);
std::uint64_t aboleth_runtime_buffer_generation(void *buffer);
int aboleth_runtime_buffer_strictly_ordered(void *buffer);

// transport: kAbolethTransportProxy, or Direct/Efa/Ionic which this build
// serves through the same ring.  gpu_index < 0 selects host-memory mode: the
// queue lives in ordinary memory and the worker moves bytes with memcpy, which
// is how the ring is tested without a GPU.  `descriptor_device` receives the
// 40-byte ProxyEndpointDescriptor (device memory when gpu_index >= 0).
void *aboleth_runtime_create_local_endpoint(void *runtime, std::uint32_t transport, int gpu_index,
                                            void *descriptor_device, std::size_t descriptor_bytes,
                                            const AbolethEndpointConfig *config);
int aboleth_runtime_local_endpoint_connection_info(void *endpoint, AbolethConnectionInfo *info);
int aboleth_runtime_connect_local_endpoint(void *endpoint, const AbolethConnectionInfo *remote);
int aboleth_runtime_local_endpoint_state(void *endpoint, std::uint64_t *producer,
                                         std::uint64_t *consumer, std::uint64_t *status);
int aboleth_runtime_local_endpoint_capacity(void *endpoint, std::uint32_t *capacity);
int aboleth_runtime_local_endpoint_max_inline(void *endpoint, std::uint32_t *max_inline_bytes);
int aboleth_runtime_local_endpoint_submit_mode(void *endpoint, std::uint32_t *submit_mode);
int aboleth_runtime_local_endpoint_gpu_resident_queues(void *endpoint, std::uint32_t *resident);
int aboleth_runtime_destroy_local_endpoint(void *endpoint);

// ---- additions of this build (no counterpart in the reference C ABI) --------

// What the machine presents, whether or not this build has a code path for it:
// a kAbolethProvider* bit is set when the provider's library resolves through
// dlopen (never a link-time dependency) and a device for it is listed.
// aboleth_runtime_provider_caps() is this mask restricted to the providers this
// build can drive (CUDA).
std::uint32_t ab200_probe_providers();
void ab200_set_last_error(const char *message);

// CUDA IPC plumbing for World.register / exchange_regions.
int ab200_ipc_export(const void *address, void *handle64, std::uint64_t *base,
                     std::uint64_t *allocation_size);
int ab200_ipc_open(const void *handle64, void **mapped_base);
int ab200_ipc_close(void *mapped_base);
int ab200_enable_peer_access(int device, int peer_device);

// Host-side twin of the device producer (aboleth/proxy_device.cuh): reserve,
// write `count` commands, release ready_sequence.  Lets a CPU thread stand in
// for the GPU.  Returns the batch sequence, or ~0 on a malformed request.
std::uint64_t ab200_proxy_host_submit(const aboleth::abi::ProxyEndpointDescriptor *descriptor,
                                      const aboleth::abi::ProxyCommand *commands, int count,
                                      double timeout_seconds);
// Wait until `sequence` retired.  Returns the endpoint status, or 1 on timeout.
std::uint64_t ab200_proxy_host_poll(const aboleth::abi::ProxyEndpointDescriptor *descriptor,
                                    std::uint64_t sequence, double timeout_seconds);
// Host copy of the descriptor the endpoint wrote to `descriptor_device`.
int ab200_endpoint_descriptor(void *endpoint, aboleth::abi::ProxyEndpointDescriptor *out);
// Fault injection (host side only): the next `batches` batches retire with
// `status` instead of being executed.
int ab200_endpoint_inject_failure(void *endpoint, std::uint64_t status, int batches);
// Counters: batches consumed, commands executed, bytes moved, signals written.
int ab200_endpoint_stats(void *endpoint, std::uint64_t *four_words);
// Submission-queue snapshot for differential tests (the reference's pair_snapshot_sq,
// include/aboleth/runtime_c.h:299-305): `batches` retired batches from sequence `first`, each as a
// 32-bit command count followed by its 32-byte commands.  Returns bytes written or -1.
long long ab200_endpoint_snapshot(void *endpoint, std::uint64_t first, int batches, void *out,
                                  std::size_t capacity);

}  // extern "C"
