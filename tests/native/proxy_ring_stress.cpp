// Many producers against the host-proxy ring, in host-memory mode (no GPU).
//
// Built with -fsanitize=thread by tests/test_sanitizers.py together with the
// runtime's own source.  Several threads per endpoint reserve, fill and release
// batches through the host twin of the device producer while the worker thread
// consumes them, another thread registers and unregisters buffers (the key table
// the worker consults), and a last one reads endpoint state and counters.  Every
// payload is checked after its batch retires.  Exit code 0 means every batch
// retired with status 0, every byte and every flag arrived, and the injected
// failure was reported as status 2 without stalling later batches; the sanitizer
// reports a data race by itself.
#include <atomic>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <thread>
#include <vector>

#include "aboleth/runtime_c.h"

namespace abi = aboleth::abi;

namespace {

constexpr int kEndpoints = 2;
constexpr int kProducersPerEndpoint = 3;
constexpr int kBatchesPerProducer = 4000;  // 12000 batches per endpoint: the 64-slot ring wraps many times
constexpr int kPayloadBytes = 256;

std::atomic<int> g_failures{0};

void expect(bool ok, const char *what) {
    if (!ok) {
        std::fprintf(stderr, "proxy_ring_stress: %s\n", what);
        g_failures.fetch_add(1);
    }
}

struct Lane {
    std::vector<std::uint8_t> source, destination;
    std::uint64_t flag = 0;
};

void producer(const abi::ProxyEndpointDescriptor *descriptor, Lane *lane, std::uint32_t source_key, int salt) {
    for (int b = 0; b < kBatchesPerProducer; ++b) {
        for (int i = 0; i < kPayloadBytes; ++i)
            lane->source[i] = static_cast<std::uint8_t>(((i * 17 + 3) & 0xff) ^ salt ^ b);
        abi::ProxyCommand commands[2]{};
        commands[0].source_address = reinterpret_cast<std::uint64_t>(lane->source.data());
        commands[0].destination_address = reinterpret_cast<std::uint64_t>(lane->destination.data());
        commands[0].bytes = kPayloadBytes;
        commands[0].source_key = source_key;
        commands[0].opcode = abi::kProxyCommandWrite;
        commands[1].source_address = static_cast<std::uint64_t>(b + 1);  // the flag's value
        commands[1].destination_address = reinterpret_cast<std::uint64_t>(&lane->flag);
        commands[1].bytes = 8;
        commands[1].opcode = abi::kProxyCommandStrongSignal;
        const std::uint64_t sequence = ab200_proxy_host_submit(descriptor, commands, 2, 20.0);
        expect(sequence != ~0ull, "a submission was refused");
        expect(ab200_proxy_host_poll(descriptor, sequence, 20.0) == abi::kEndpointStatusOk,
               "a batch did not retire with status 0");
        expect(__atomic_load_n(&lane->flag, __ATOMIC_ACQUIRE) == static_cast<std::uint64_t>(b + 1),
               "the flag does not hold this batch's epoch");
        expect(std::memcmp(lane->source.data(), lane->destination.data(), kPayloadBytes) == 0,
               "the payload differs after its batch retired");
    }
}

}  // namespace

int main() {
    void *runtime = aboleth_runtime_create_for_device(-1, nullptr);
    if (runtime == nullptr) {
        std::fprintf(stderr, "runtime: %s\n", aboleth_runtime_last_error());
        return 2;
    }
    void *endpoints[kEndpoints];
    abi::ProxyEndpointDescriptor descriptors[kEndpoints];
    for (int e = 0; e < kEndpoints; ++e) {
        endpoints[e] = aboleth_runtime_create_local_endpoint(runtime, kAbolethTransportProxy, -1, &descriptors[e],
                                                             sizeof(descriptors[e]), nullptr);
        if (endpoints[e] == nullptr) {
            std::fprintf(stderr, "endpoint: %s\n", aboleth_runtime_last_error());
            return 2;
        }
    }

    std::vector<Lane> lanes(kEndpoints * kProducersPerEndpoint);
    std::vector<void *> registrations;
    for (Lane &lane : lanes) {
        lane.source.assign(kPayloadBytes, 0);
        lane.destination.assign(kPayloadBytes, 0);
        registrations.push_back(
            aboleth_runtime_register_buffer(runtime, -1, lane.source.data(), lane.source.size(), 1));
    }

    std::atomic<bool> done{false};
    // Churn in the key table while the workers look keys up.
    std::thread registrar([&] {
        std::vector<std::uint8_t> scratch(4096);
        while (!done.load(std::memory_order_acquire)) {
            void *r = aboleth_runtime_register_buffer(runtime, -1, scratch.data(), scratch.size(), 7);
            expect(r != nullptr && aboleth_runtime_buffer_length(r) == scratch.size(), "scratch registration failed");
            aboleth_runtime_unregister_buffer(r);
        }
    });
    // A reader of state and counters, as a monitoring thread would be.
    std::thread observer([&] {
        while (!done.load(std::memory_order_acquire)) {
            for (int e = 0; e < kEndpoints; ++e) {
                std::uint64_t producer_index = 0, consumer = 0, status = 0, stats[4];
                aboleth_runtime_local_endpoint_state(endpoints[e], &producer_index, &consumer, &status);
                ab200_endpoint_stats(endpoints[e], stats);
                expect(status == abi::kEndpointStatusOk, "an endpoint failed during the stress");
            }
            std::this_thread::yield();
        }
    });

    std::vector<std::thread> producers;
    for (int e = 0; e < kEndpoints; ++e)
        for (int p = 0; p < kProducersPerEndpoint; ++p) {
            const int lane = e * kProducersPerEndpoint + p;
            producers.emplace_back(producer, &descriptors[e], &lanes[lane],
                                   aboleth_runtime_buffer_lkey(registrations[lane]), 31 * lane + 5);
        }
    for (std::thread &t : producers)
        t.join();
    done.store(true, std::memory_order_release);
    registrar.join();
    observer.join();

    for (int e = 0; e < kEndpoints; ++e) {
        std::uint64_t stats[4];
        ab200_endpoint_stats(endpoints[e], stats);
        const std::uint64_t batches = static_cast<std::uint64_t>(kProducersPerEndpoint) * kBatchesPerProducer;
        expect(stats[0] == batches && stats[1] == 2 * batches && stats[2] == batches * kPayloadBytes &&
                   stats[3] == batches,
               "the endpoint's counters do not add up");
    }

    // Host-side fault injection: the next batch retires with status 2, and so does
    // the one after it (a failed endpoint keeps retiring without executing).
    ab200_endpoint_inject_failure(endpoints[0], abi::kEndpointStatusCompletionFailure, 1);
    abi::ProxyCommand nop{};
    nop.opcode = abi::kProxyCommandNop;
    for (int i = 0; i < 2; ++i) {
        const std::uint64_t sequence = ab200_proxy_host_submit(&descriptors[0], &nop, 1, 5.0);
        expect(ab200_proxy_host_poll(&descriptors[0], sequence, 5.0) == abi::kEndpointStatusCompletionFailure,
               "the injected failure was not reported");
    }

    for (int e = 0; e < kEndpoints; ++e)
        expect(aboleth_runtime_destroy_local_endpoint(endpoints[e]) == 0, "destroying an endpoint failed");
    for (void *r : registrations)
        aboleth_runtime_unregister_buffer(r);
    expect(aboleth_runtime_destroy(runtime) == 0, "the runtime still held registrations");
    std::printf("batches per endpoint: %d, failures: %d\n", kProducersPerEndpoint * kBatchesPerProducer,
                g_failures.load());
    return g_failures.load() == 0 ? 0 : 1;
}
