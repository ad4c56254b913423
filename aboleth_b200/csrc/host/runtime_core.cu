// Native host runtime: error reporting, provider capabilities, the key table
// of registered buffers, CUDA IPC export/import, and the host-proxy progress
// thread that serves every queue transport on a machine without a NIC.
//
// This file is host C++ compiled by nvcc (it contains no kernels), like the
// reference's src/runtime/core/*.cu.  The proxy follows the protocol of the
// reference's src/runtime/proxy/aboleth_proxy.cu:387-520 (consume strictly by
// sequence, always publish completed_sequence, status 0..3) with a CUDA copy
// provider in place of verbs.
#include <atomic>
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

#include <unistd.h>

#include <cuda_runtime.h>

#include "aboleth/runtime_c.h"

namespace {

using aboleth::abi::ProxyBatchSlot;
using aboleth::abi::ProxyCommand;
using aboleth::abi::ProxyEndpointDescriptor;
using aboleth::abi::ProxyQueueState;
namespace abi = aboleth::abi;

thread_local std::string g_error;

int fail(const std::string &message) {
    g_error = message;
    return -1;
}

template <typename T>
T *fail_ptr(const std::string &message) {
    g_error = message;
    return nullptr;
}

bool cuda_ok(cudaError_t e, const char *what) {
    if (e == cudaSuccess)
        return true;
    g_error = std::string(what) + ": " + cudaGetErrorString(e);
    return false;
}

int visible_gpus() {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    return n;
}

struct Buffer;

struct Runtime {
    int device = -1;
    std::mutex mutex;
    std::uint32_t next_key = 0x1000;
    std::map<std::uint32_t, Buffer *> keys;
};

struct Buffer {
    Runtime *runtime;
    std::uint64_t address, length, generation;
    std::uint32_t key;
    int device;
};

// ---- proxy endpoint --------------------------------------------------------------

struct Endpoint {
    Runtime *runtime = nullptr;
    std::uint32_t transport = 0;
    int device = -1;  // < 0: host-memory mode
    ProxyQueueState *queue = nullptr;          // host view
    std::uint64_t queue_device_address = 0;    // what the GPU dereferences
    std::uint64_t *producer = nullptr;         // device (or host) reservation counter
    ProxyEndpointDescriptor descriptor{};
    std::thread worker;
    std::atomic<bool> stop{false};
    std::atomic<bool> connected{false};
    std::atomic<std::uint64_t> inject_status{0};
    std::atomic<int> inject_batches{0};
    std::atomic<std::uint64_t> stats[4];
    cudaStream_t stream = nullptr;
    std::uint64_t *staging = nullptr;  // pinned words for signal values
    bool strict_keys = false;
};

bool key_covers(Runtime *rt, std::uint32_t key, std::uint64_t address, std::uint64_t bytes) {
    if (key == 0)
        return true;  // unchecked
    std::lock_guard<std::mutex> lock(rt->mutex);
    auto it = rt->keys.find(key);
    if (it == rt->keys.end())
        return false;
    const Buffer *b = it->second;
    return address >= b->address && address + bytes <= b->address + b->length;
}

// Execute one command.  Returns an endpoint status (0 ok).
std::uint64_t execute(Endpoint *ep, const ProxyCommand &c, int staging_slot) {
    switch (c.opcode) {
    case abi::kProxyCommandNop:
        return abi::kEndpointStatusOk;
    case abi::kProxyCommandWrite: {
        if (!key_covers(ep->runtime, c.source_key, c.source_address, c.bytes) ||
            !key_covers(ep->runtime, c.destination_key, c.destination_address, c.bytes))
            return abi::kEndpointStatusCompletionFailure;
        if (c.bytes == 0)
            return abi::kEndpointStatusOk;
        if (ep->device < 0) {
            std::memcpy(reinterpret_cast<void *>(c.destination_address),
                        reinterpret_cast<const void *>(c.source_address), c.bytes);
        } else if (cudaMemcpyAsync(reinterpret_cast<void *>(c.destination_address),
                                   reinterpret_cast<const void *>(c.source_address), c.bytes,
                                   cudaMemcpyDefault, ep->stream) != cudaSuccess) {
            cudaGetLastError();
            return abi::kEndpointStatusCompletionFailure;
        }
        ep->stats[2] += c.bytes;
        return abi::kEndpointStatusOk;
    }
    case abi::kProxyCommandWeakSignal:
    case abi::kProxyCommandStrongSignal: {
        if (!key_covers(ep->runtime, c.destination_key, c.destination_address, 8))
            return abi::kEndpointStatusCompletionFailure;
        if (ep->device < 0) {
            // Host mode: memcpy above already completed; release publishes it.
            __atomic_store_n(reinterpret_cast<std::uint64_t *>(c.destination_address),
                             c.source_address, __ATOMIC_RELEASE);
        } else {
            // Strong: the payload copies queued before it on this stream are
            // placed before the 8-byte write because the stream is in order;
            // weak signals take the same path (ordering costs nothing here).
            ep->staging[staging_slot] = c.source_address;
            if (cudaMemcpyAsync(reinterpret_cast<void *>(c.destination_address),
                                &ep->staging[staging_slot], 8, cudaMemcpyDefault,
                                ep->stream) != cudaSuccess) {
                cudaGetLastError();
                return abi::kEndpointStatusCompletionFailure;
            }
        }
        ep->stats[3] += 1;
        return abi::kEndpointStatusOk;
    }
    default:
        return abi::kEndpointStatusMalformed;
    }
}

void worker_main(Endpoint *ep) {
    if (ep->device >= 0) {
        cudaSetDevice(ep->device);
        cudaStreamCreateWithFlags(&ep->stream, cudaStreamNonBlocking);
    }
    ProxyQueueState *q = ep->queue;
    std::uint64_t next = 0;
    unsigned idle = 0;
    while (!ep->stop.load(std::memory_order_acquire)) {
        ProxyBatchSlot &slot = q->slots[next % abi::kProxySlotCount];
        if (__atomic_load_n(&slot.ready_sequence, __ATOMIC_ACQUIRE) != next + 1) {
            if (++idle > 2000)
                std::this_thread::sleep_for(std::chrono::microseconds(20));
            continue;
        }
        idle = 0;
        std::uint64_t status = __atomic_load_n(&q->status, __ATOMIC_RELAXED);
        const std::uint32_t count = slot.command_count;
        if (status == abi::kEndpointStatusOk) {
            if (ep->inject_batches.load() > 0) {
                ep->inject_batches.fetch_sub(1);
                status = ep->inject_status.load();
            } else if (count == 0 || count > abi::kProxyMaximumCommands) {
                status = abi::kEndpointStatusMalformed;
            } else {
                for (std::uint32_t i = 0; i < count && status == abi::kEndpointStatusOk; ++i) {
                    status = execute(ep, slot.commands[i], static_cast<int>(i % 256));
                    ep->stats[1] += 1;
                }
                if (ep->device >= 0 && cudaStreamSynchronize(ep->stream) != cudaSuccess) {
                    cudaGetLastError();
                    status = abi::kEndpointStatusCompletionFailure;
                }
            }
            if (status != abi::kEndpointStatusOk)
                __atomic_store_n(&q->status, status, __ATOMIC_RELEASE);
        }
        // A failed endpoint still retires its batches so that waiters end.
        ep->stats[0] += 1;
        ++next;
        __atomic_store_n(&q->completed_sequence, next, __ATOMIC_RELEASE);
    }
    if (ep->stream != nullptr) {
        cudaStreamSynchronize(ep->stream);
        cudaStreamDestroy(ep->stream);
        ep->stream = nullptr;
    }
}

bool host_wait_completed(const ProxyQueueState *q, std::uint64_t target, double timeout_seconds) {
    const auto deadline = std::chrono::steady_clock::now() +
                          std::chrono::duration<double>(timeout_seconds);
    unsigned spins = 0;
    while (__atomic_load_n(&q->completed_sequence, __ATOMIC_ACQUIRE) < target) {
        if (++spins > 1000) {
            std::this_thread::sleep_for(std::chrono::microseconds(10));
            if (std::chrono::steady_clock::now() > deadline)
                return false;
        }
    }
    return true;
}

}  // namespace

extern "C" {

const char *aboleth_runtime_last_error() { return g_error.c_str(); }

// Lets the runtime's other translation units report through the same thread-local string.
void ab200_set_last_error(const char *message) { g_error = message ? message : ""; }

std::uint32_t aboleth_runtime_provider_caps() {
    // No verbs, mlx5, EFA, libfabric, HIP or Ionic provider is compiled in.
    return visible_gpus() > 0 ? kAbolethProviderCuda : 0u;
}

void *aboleth_runtime_create() { return aboleth_runtime_create_for_device(-1, nullptr); }

void *aboleth_runtime_create_for_device(int gpu_index, const char *hca_name) {
    if (hca_name != nullptr && hca_name[0] != '\0')
        return fail_ptr<void>("no HCA can be opened: this build has no verbs provider");
    if (gpu_index >= 0 && gpu_index >= visible_gpus())
        return fail_ptr<void>("CUDA ordinal " + std::to_string(gpu_index) + " is not visible");
    auto *rt = new Runtime();
    rt->device = gpu_index;
    return rt;
}

const char *aboleth_runtime_hca_name(void *) { return ""; }
int aboleth_runtime_gpu_index(void *runtime) { return static_cast<Runtime *>(runtime)->device; }
int aboleth_runtime_port(void *) { return 0; }
int aboleth_runtime_gid_index(void *) { return -1; }
int aboleth_runtime_link_layer(void *) { return 0; }
int aboleth_runtime_lid(void *) { return 0; }

int aboleth_runtime_destroy(void *runtime) {
    auto *rt = static_cast<Runtime *>(runtime);
    if (rt == nullptr)
        return fail("null runtime");
    {
        std::lock_guard<std::mutex> lock(rt->mutex);
        if (!rt->keys.empty())
            return fail("runtime still holds registered buffers");
    }
    delete rt;
    return 0;
}

void *aboleth_runtime_register_buffer(void *runtime, int gpu_index, void *address,
                                      std::size_t bytes, std::uint64_t generation) {
    auto *rt = static_cast<Runtime *>(runtime);
    if (rt == nullptr)
        return fail_ptr<void>("null runtime");
    if (address == nullptr || bytes == 0)
        return fail_ptr<void>("cannot register an empty buffer");
    auto *b = new Buffer{rt, reinterpret_cast<std::uint64_t>(address), bytes, generation, 0, gpu_index};
    std::lock_guard<std::mutex> lock(rt->mutex);
    b->key = rt->next_key++;
    rt->keys[b->key] = b;
    return b;
}

int aboleth_runtime_unregister_buffer(void *buffer) {
    auto *b = static_cast<Buffer *>(buffer);
    if (b == nullptr)
        return fail("null buffer");
    {
        std::lock_guard<std::mutex> lock(b->runtime->mutex);
        b->runtime->keys.erase(b->key);
    }
    delete b;
    return 0;
}

std::uint64_t aboleth_runtime_buffer_address(void *b) { return static_cast<Buffer *>(b)->address; }
std::uint64_t aboleth_runtime_buffer_length(void *b) { return static_cast<Buffer *>(b)->length; }
std::uint32_t aboleth_runtime_buffer_lkey(void *b) { return static_cast<Buffer *>(b)->key; }
std::uint32_t aboleth_runtime_buffer_rkey(void *b) { return static_cast<Buffer *>(b)->key; }
int aboleth_runtime_buffer_device(void *b) { return static_cast<Buffer *>(b)->device; }
std::uint64_t aboleth_runtime_buffer_generation(void *b) { return static_cast<Buffer *>(b)->generation; }
// A CUDA copy stream places bytes in order: every registration is strict.
int aboleth_runtime_buffer_strictly_ordered(void *) { return 1; }

void *aboleth_runtime_create_local_endpoint(void *runtime, std::uint32_t transport, int gpu_index,
                                            void *descriptor_device, std::size_t descriptor_bytes,
                                            const AbolethEndpointConfig *config) {
    auto *rt = static_cast<Runtime *>(runtime);
    if (rt == nullptr)
        return fail_ptr<void>("null runtime");
    if (transport < kAbolethTransportDirect || transport > kAbolethTransportIonic)
        return fail_ptr<void>("unknown endpoint transport " + std::to_string(transport));
    if (descriptor_device == nullptr || descriptor_bytes < sizeof(ProxyEndpointDescriptor))
        return fail_ptr<void>("endpoint descriptor storage is smaller than 40 bytes");
    AbolethEndpointConfig cfg{};
    cfg.gid_index = -1;
    if (config != nullptr) {
        if (config->struct_size > sizeof(AbolethEndpointConfig))
            return fail_ptr<void>("AbolethEndpointConfig.struct_size is larger than this runtime knows");
        if (config->struct_size < sizeof(std::uint32_t))
            return fail_ptr<void>("AbolethEndpointConfig.struct_size is too small");
        std::memcpy(&cfg, config, config->struct_size);
        if (cfg.qp_type != 0)
            return fail_ptr<void>("qp_type must be 0 (reliable connected)");
        if (cfg.qps_per_peer > 1)
            return fail_ptr<void>("qps_per_peer must be 0 or 1");
        if (cfg.sm_map_policy != 0)
            return fail_ptr<void>("sm_map_policy must be 0");
        if (config->struct_size >= 28 && cfg.port != 0)
            return fail_ptr<void>("port must be 0: no adapter port exists");
        if (config->struct_size >= 32 && cfg.gid_index != -1)
            return fail_ptr<void>("gid_index must be -1: no GID table exists");
        if (config->struct_size >= 33 && cfg.hca[0] != '\0')
            return fail_ptr<void>("hca must be empty: no HCA exists");
    }
    auto *ep = new Endpoint();
    ep->runtime = rt;
    ep->transport = transport;
    ep->device = gpu_index;
    for (auto &s : ep->stats)
        s = 0;
    const char *strict = std::getenv("ABOLETH_PROXY_STRICT_KEYS");
    ep->strict_keys = strict != nullptr && strict[0] == '1';
    if (gpu_index < 0) {
        ep->queue = static_cast<ProxyQueueState *>(std::calloc(1, sizeof(ProxyQueueState)));
        ep->producer = static_cast<std::uint64_t *>(std::calloc(1, 8));
        ep->queue_device_address = reinterpret_cast<std::uint64_t>(ep->queue);
    } else {
        if (!cuda_ok(cudaSetDevice(gpu_index), "cudaSetDevice")) {
            delete ep;
            return nullptr;
        }
        void *host = nullptr, *dev = nullptr;
        if (!cuda_ok(cudaHostAlloc(&host, sizeof(ProxyQueueState), cudaHostAllocMapped | cudaHostAllocPortable),
                     "cudaHostAlloc(queue)") ||
            !cuda_ok(cudaHostGetDevicePointer(&dev, host, 0), "cudaHostGetDevicePointer")) {
            delete ep;
            return nullptr;
        }
        std::memset(host, 0, sizeof(ProxyQueueState));
        ep->queue = static_cast<ProxyQueueState *>(host);
        ep->queue_device_address = reinterpret_cast<std::uint64_t>(dev);
        void *producer = nullptr, *staging = nullptr;
        if (!cuda_ok(cudaMalloc(&producer, 8), "cudaMalloc(producer)") ||
            !cuda_ok(cudaMemset(producer, 0, 8), "cudaMemset(producer)") ||
            !cuda_ok(cudaHostAlloc(&staging, 256 * 8, cudaHostAllocPortable), "cudaHostAlloc(staging)")) {
            delete ep;
            return nullptr;
        }
        ep->producer = static_cast<std::uint64_t *>(producer);
        ep->staging = static_cast<std::uint64_t *>(staging);
    }
    ep->descriptor.queue_state = ep->queue_device_address;
    ep->descriptor.producer_index_address = reinterpret_cast<std::uint64_t>(ep->producer);
    const char *timeout = std::getenv("ABOLETH_COMPLETION_TIMEOUT_CYCLES");
    ep->descriptor.completion_timeout_cycles = timeout ? std::strtoull(timeout, nullptr, 0) : 0;
    ep->descriptor.slot_count = abi::kProxySlotCount;
    ep->descriptor.slot_stride = sizeof(ProxyBatchSlot);
    ep->descriptor.maximum_commands = abi::kProxyMaximumCommands;
    ep->descriptor.abi_version = abi::kProxyEndpointVersion;
    if (gpu_index < 0) {
        std::memcpy(descriptor_device, &ep->descriptor, sizeof(ep->descriptor));
    } else if (!cuda_ok(cudaMemcpy(descriptor_device, &ep->descriptor, sizeof(ep->descriptor),
                                   cudaMemcpyHostToDevice),
                        "cudaMemcpy(descriptor)")) {
        delete ep;
        return nullptr;
    }
    ep->worker = std::thread(worker_main, ep);
    return ep;
}

int aboleth_runtime_local_endpoint_connection_info(void *endpoint, AbolethConnectionInfo *info) {
    auto *ep = static_cast<Endpoint *>(endpoint);
    if (ep == nullptr || info == nullptr)
        return fail("null endpoint or connection info");
    std::memset(info, 0, sizeof(*info));
    info->abi_version = kAbolethConnectionInfoVersion;
    info->transport = ep->transport;
    info->provider = kAbolethProxyProviderCudaCopy;
    info->path_mtu = 4096;
    // The "address" of a CUDA-copy endpoint is (pid, device): enough for a
    // peer to recognise that both ends live on one node.
    const std::uint64_t pid = static_cast<std::uint64_t>(getpid());
    const std::int64_t device = ep->device;
    info->address_format = 1;
    info->address_length = 16;
    std::memcpy(info->address, &pid, 8);
    std::memcpy(info->address + 8, &device, 8);
    return 0;
}

int aboleth_runtime_connect_local_endpoint(void *endpoint, const AbolethConnectionInfo *remote) {
    auto *ep = static_cast<Endpoint *>(endpoint);
    if (ep == nullptr || remote == nullptr)
        return fail("null endpoint or connection info");
    if (remote->abi_version != kAbolethConnectionInfoVersion)
        return fail("connection info version " + std::to_string(remote->abi_version) +
                    " is not " + std::to_string(kAbolethConnectionInfoVersion));
    if (remote->transport != ep->transport)
        return fail("peer endpoint was opened for a different transport");
    if (remote->provider != kAbolethProxyProviderCudaCopy)
        return fail("peer endpoint uses a provider this build does not have");
    ep->connected = true;
    return 0;
}

int aboleth_runtime_local_endpoint_state(void *endpoint, std::uint64_t *producer,
                                         std::uint64_t *consumer, std::uint64_t *status) {
    auto *ep = static_cast<Endpoint *>(endpoint);
    if (ep == nullptr)
        return fail("null endpoint");
    std::uint64_t reserved = 0;
    if (ep->device < 0) {
        reserved = __atomic_load_n(ep->producer, __ATOMIC_ACQUIRE);
    } else if (!cuda_ok(cudaMemcpy(&reserved, ep->producer, 8, cudaMemcpyDeviceToHost),
                        "cudaMemcpy(producer)")) {
        return -1;
    }
    if (producer)
        *producer = reserved;
    if (consumer)
        *consumer = __atomic_load_n(&ep->queue->completed_sequence, __ATOMIC_ACQUIRE);
    if (status)
        *status = __atomic_load_n(&ep->queue->status, __ATOMIC_ACQUIRE);
    return 0;
}

int aboleth_runtime_local_endpoint_capacity(void *endpoint, std::uint32_t *capacity) {
    if (endpoint == nullptr || capacity == nullptr)
        return fail("null endpoint");
    *capacity = abi::kProxySlotCount * abi::kProxyMaximumCommands;
    return 0;
}

int aboleth_runtime_local_endpoint_max_inline(void *endpoint, std::uint32_t *max_inline_bytes) {
    if (endpoint == nullptr || max_inline_bytes == nullptr)
        return fail("null endpoint");
    *max_inline_bytes = 8;
    return 0;
}

int aboleth_runtime_local_endpoint_submit_mode(void *endpoint, std::uint32_t *submit_mode) {
    if (endpoint == nullptr || submit_mode == nullptr)
        return fail("null endpoint");
    *submit_mode = 2;  // command proxy: the host builds and posts the work
    return 0;
}

int aboleth_runtime_local_endpoint_gpu_resident_queues(void *endpoint, std::uint32_t *resident) {
    if (endpoint == nullptr || resident == nullptr)
        return fail("null endpoint");
    *resident = 0;
    return 0;
}

int aboleth_runtime_destroy_local_endpoint(void *endpoint) {
    auto *ep = static_cast<Endpoint *>(endpoint);
    if (ep == nullptr)
        return fail("null endpoint");
    ep->stop.store(true, std::memory_order_release);
    if (ep->worker.joinable())
        ep->worker.join();
    if (ep->device < 0) {
        std::free(ep->queue);
        std::free(ep->producer);
    } else {
        cudaSetDevice(ep->device);
        cudaFreeHost(ep->queue);
        cudaFree(ep->producer);
        cudaFreeHost(ep->staging);
    }
    delete ep;
    return 0;
}

// ---- CUDA IPC ----------------------------------------------------------------------

int ab200_ipc_export(const void *address, void *handle64, std::uint64_t *base,
                     std::uint64_t *allocation_size) {
    static_assert(sizeof(cudaIpcMemHandle_t) == 64);
    using RangeFn = int (*)(unsigned long long *, std::size_t *, unsigned long long);
    static RangeFn range = nullptr;
    if (range == nullptr) {
        void *fn = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (!cuda_ok(cudaGetDriverEntryPoint("cuMemGetAddressRange", &fn, cudaEnableDefault, &q),
                     "cudaGetDriverEntryPoint(cuMemGetAddressRange)") ||
            fn == nullptr)
            return fail("cuMemGetAddressRange is unavailable");
        range = reinterpret_cast<RangeFn>(fn);
    }
    unsigned long long lo = 0;
    std::size_t size = 0;
    const int rc = range(&lo, &size, reinterpret_cast<unsigned long long>(address));
    if (rc != 0)
        return fail("cuMemGetAddressRange failed with CUresult " + std::to_string(rc));
    cudaIpcMemHandle_t h;
    if (!cuda_ok(cudaIpcGetMemHandle(&h, reinterpret_cast<void *>(lo)), "cudaIpcGetMemHandle"))
        return -1;
    std::memcpy(handle64, &h, 64);
    *base = lo;
    *allocation_size = size;
    return 0;
}

int ab200_ipc_open(const void *handle64, void **mapped_base) {
    cudaIpcMemHandle_t h;
    std::memcpy(&h, handle64, 64);
    if (!cuda_ok(cudaIpcOpenMemHandle(mapped_base, h, cudaIpcMemLazyEnablePeerAccess),
                 "cudaIpcOpenMemHandle"))
        return -1;
    return 0;
}

int ab200_ipc_close(void *mapped_base) {
    return cuda_ok(cudaIpcCloseMemHandle(mapped_base), "cudaIpcCloseMemHandle") ? 0 : -1;
}

int ab200_enable_peer_access(int device, int peer_device) {
    if (device == peer_device)
        return 0;
    int can = 0;
    if (!cuda_ok(cudaDeviceCanAccessPeer(&can, device, peer_device), "cudaDeviceCanAccessPeer"))
        return -1;
    if (!can)
        return fail("device " + std::to_string(device) + " cannot reach device " +
                    std::to_string(peer_device) + " over peer memory");
    int previous = 0;
    cudaGetDevice(&previous);
    cudaSetDevice(device);
    cudaError_t e = cudaDeviceEnablePeerAccess(peer_device, 0);
    cudaSetDevice(previous);
    if (e == cudaErrorPeerAccessAlreadyEnabled) {
        cudaGetLastError();
        return 0;
    }
    return cuda_ok(e, "cudaDeviceEnablePeerAccess") ? 0 : -1;
}

// ---- host twin of the device producer ------------------------------------------------

std::uint64_t ab200_proxy_host_submit(const ProxyEndpointDescriptor *d, const ProxyCommand *commands,
                                      int count, double timeout_seconds) {
    if (d == nullptr || d->abi_version != abi::kProxyEndpointVersion || count < 1 ||
        count > static_cast<int>(d->maximum_commands)) {
        fail("malformed proxy batch");
        return ~0ull;
    }
    auto *q = reinterpret_cast<ProxyQueueState *>(d->queue_state);
    auto *producer = reinterpret_cast<std::uint64_t *>(d->producer_index_address);
    const std::uint64_t seq = __atomic_fetch_add(producer, 1, __ATOMIC_RELAXED);
    if (seq >= d->slot_count && !host_wait_completed(q, seq + 1 - d->slot_count, timeout_seconds)) {
        fail("proxy ring stayed full");
        return ~0ull;
    }
    ProxyBatchSlot &slot = q->slots[seq % d->slot_count];
    for (int i = 0; i < count; ++i)
        slot.commands[i] = commands[i];
    slot.command_count = static_cast<std::uint32_t>(count);
    __atomic_store_n(&slot.ready_sequence, seq + 1, __ATOMIC_RELEASE);
    return seq;
}

std::uint64_t ab200_proxy_host_poll(const ProxyEndpointDescriptor *d, std::uint64_t sequence,
                                    double timeout_seconds) {
    auto *q = reinterpret_cast<ProxyQueueState *>(d->queue_state);
    if (!host_wait_completed(q, sequence + 1, timeout_seconds))
        return abi::kEndpointStatusTimeout;
    return __atomic_load_n(&q->status, __ATOMIC_ACQUIRE);
}

int ab200_endpoint_descriptor(void *endpoint, ProxyEndpointDescriptor *out) {
    auto *ep = static_cast<Endpoint *>(endpoint);
    if (ep == nullptr || out == nullptr)
        return fail("null endpoint");
    *out = ep->descriptor;
    if (ep->device >= 0)
        out->queue_state = reinterpret_cast<std::uint64_t>(ep->queue);  // host view
    return 0;
}

int ab200_endpoint_inject_failure(void *endpoint, std::uint64_t status, int batches) {
    auto *ep = static_cast<Endpoint *>(endpoint);
    if (ep == nullptr)
        return fail("null endpoint");
    ep->inject_status = status;
    ep->inject_batches = batches;
    return 0;
}

int ab200_endpoint_stats(void *endpoint, std::uint64_t *four_words) {
    auto *ep = static_cast<Endpoint *>(endpoint);
    if (ep == nullptr)
        return fail("null endpoint");
    for (int i = 0; i < 4; ++i)
        four_words[i] = ep->stats[i].load();
    return 0;
}

// Snapshot of the submission queue: for each of `batches` batches starting at sequence `first`, a
// 32-bit command count followed by that many 32-byte commands, as the producer wrote them.  A slot
// keeps its contents after the worker retired it (until the ring wraps), so the last 64 batches can
// be read at rest.  Returns the bytes written, or -1 (batch not produced yet, out of the ring's
// window, or `capacity` too small).
long long ab200_endpoint_snapshot(void *endpoint, std::uint64_t first, int batches, void *out,
                                  std::size_t capacity) {
    auto *ep = static_cast<Endpoint *>(endpoint);
    if (ep == nullptr || out == nullptr || batches < 0)
        return fail("snapshot: null endpoint or buffer");
    const std::uint64_t completed = __atomic_load_n(&ep->queue->completed_sequence, __ATOMIC_ACQUIRE);
    if (first + static_cast<std::uint64_t>(batches) > completed)
        return fail("snapshot: batches that were not retired yet");
    if (completed - first > abi::kProxySlotCount)
        return fail("snapshot: batches already overwritten by the ring");
    auto *cursor = static_cast<unsigned char *>(out);
    std::size_t used = 0;
    for (int b = 0; b < batches; ++b) {
        const abi::ProxyBatchSlot &slot = ep->queue->slots[(first + b) % abi::kProxySlotCount];
        const std::uint32_t count = slot.command_count;
        const std::size_t bytes = sizeof(std::uint32_t) + count * sizeof(abi::ProxyCommand);
        if (count > abi::kProxyMaximumCommands || used + bytes > capacity)
            return fail("snapshot: buffer too small or slot damaged");
        std::memcpy(cursor + used, &count, sizeof(count));
        std::memcpy(cursor + used + sizeof(count), slot.commands, count * sizeof(abi::ProxyCommand));
        used += bytes;
    }
    return static_cast<long long>(used);
}

}  // extern "C"
