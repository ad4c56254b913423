// Standalone C++ arm of the Tier-1 ladder: ping-pong latency, windowed put bandwidth and all-to-all
// rounds written against aboleth/device.cuh only (no Python, no PyTorch).  One process drives every
// GPU it is given: rank r lives on GPU r, peers are reached through CUDA peer access, and a rank's
// kernel is launched on its own GPU, so kernels that wait on one another never share a GPU.  With one
// GPU every benchmark runs in loopback (the rank's only peer is itself, one kernel, no partner).
//
// Same measurements as the reference's C++ arms (experiments/bench/bench_tier1_aboleth.cu,
// bench_tier1_arms.cuh: option parsing, run loops, JSON; bench_common.h:31-57,131-223: %globaltimer
// stamps, pattern fill / check, quantiles), restated for peer memory on one node.
//
//   bench_tier1 [--gpus N] [--bench pingpong|window|alltoall|all] [--bytes B] [--iters I]
//               [--warmup W] [--window K] [--ctas C] [--threads T]
//
// Prints one JSON object per benchmark on its own line; exits 1 if a wait timed out or a payload
// byte is wrong.  Every device wait is bounded (aboleth::wait_signal gives up after
// ABOLETH_WAIT_TIMEOUT_NS and records Status::Timeout in the rank's status word).
#include <algorithm>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include <cuda_runtime.h>

#include "aboleth/device.cuh"

namespace {

#define CHECK_CUDA(expr)                                                                          \
    do {                                                                                          \
        cudaError_t err__ = (expr);                                                               \
        if (err__ != cudaSuccess) {                                                               \
            std::fprintf(stderr, "%s:%d: %s: %s\n", __FILE__, __LINE__, #expr,                    \
                         cudaGetErrorString(err__));                                              \
            std::exit(2);                                                                         \
        }                                                                                         \
    } while (0)

using aboleth::DeviceContext;
using aboleth::LocalRegion;
using aboleth::RemoteRegion;

__device__ __forceinline__ std::uint64_t now_ns() {
    std::uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__host__ __device__ inline std::uint8_t pattern_byte(std::uint64_t i, std::uint32_t salt) {
    return static_cast<std::uint8_t>(((i * 17 + 3) & 0xFF) ^ (salt & 0xFF));
}

__global__ void fill_pattern(std::uint8_t *buf, std::uint64_t bytes, std::uint32_t salt) {
    for (std::uint64_t i = blockIdx.x * blockDim.x + threadIdx.x; i < bytes;
         i += static_cast<std::uint64_t>(gridDim.x) * blockDim.x)
        buf[i] = pattern_byte(i, salt);
}

__global__ void check_pattern(const std::uint8_t *buf, std::uint64_t bytes, std::uint32_t salt,
                              unsigned long long *wrong) {
    unsigned long long bad = 0;
    for (std::uint64_t i = blockIdx.x * blockDim.x + threadIdx.x; i < bytes;
         i += static_cast<std::uint64_t>(gridDim.x) * blockDim.x)
        bad += buf[i] != pattern_byte(i, salt);
    if (bad)
        atomicAdd(wrong, bad);
}

// What one rank's kernels need: addresses are valid on the rank's own GPU (peer pointers included).
struct RankView {
    const std::uint64_t *endpoints;  // [world] handle table, kKindP2P entries
    unsigned long long *status;      // first non-zero Status of any call
    std::uint64_t send;              // [world][stride] payloads, slot p goes to peer p
    std::uint64_t recv;              // [world][stride] slot s is written by rank s
    std::uint64_t flags;             // [world] u64, flag s is written by rank s
    std::uint64_t peer_recv[8];      // recv base of every rank
    std::uint64_t peer_flags[8];     // flag base of every rank
    std::uint64_t *times;            // [iters] ns per iteration (thread 0 of CTA 0)
    std::uint64_t stride;
    int rank, world;
};

// CTA barrier that also tells every thread whether this rank has recorded a failure (a wait that
// timed out): the loops below stop at the first one instead of timing out once per iteration.
__device__ __forceinline__ bool barrier_failed(const RankView &v) {
    return __syncthreads_or(threadIdx.x == 0 && *reinterpret_cast<volatile unsigned long long *>(v.status) != 0);
}

// Ping-pong between `rank` and `peer`: the initiator puts `bytes`, signals, and waits for the echo.
// Loopback (peer == rank): one kernel plays both parts on its own flag.
__global__ void pingpong_kernel(RankView v, int peer, int initiator, std::uint32_t bytes, int iters,
                                int warmup, std::uint64_t epoch0) {
    DeviceContext ctx{v.endpoints, nullptr, v.status};
    const RemoteRegion dst{v.peer_recv[peer] + v.rank * v.stride, 0};
    const LocalRegion src{v.send + peer * v.stride, 0};
    const RemoteRegion peer_flag{v.peer_flags[peer] + v.rank * 8, 0};
    const std::uint64_t *my_flag = reinterpret_cast<const std::uint64_t *>(v.flags) + peer;
    const bool loopback = peer == v.rank;
    for (int it = 0; it < warmup + iters; ++it) {
        const std::uint64_t epoch = epoch0 + it + 1;
        const std::uint64_t t0 = now_ns();
        if (initiator || loopback) {
            aboleth::put_block(dst, src, bytes);
            aboleth::signal_block(peer_flag, epoch);
            if (threadIdx.x == 0)
                aboleth::wait_signal(ctx, my_flag, epoch);
        } else {
            if (threadIdx.x == 0)
                aboleth::wait_signal(ctx, my_flag, epoch);
            __syncthreads();
            aboleth::put_block(dst, src, bytes);
            aboleth::signal_block(peer_flag, epoch);
        }
        if (barrier_failed(v))
            break;
        if (threadIdx.x == 0 && it >= warmup)
            v.times[it - warmup] = now_ns() - t0;
    }
}

// Windowed puts: every CTA sends `window` chunks per iteration and closes them with one signal; the
// receiver side of the same kernel (CTA c of the partner, or of this rank in loopback) waits for
// the window's signal.  The time of thread 0 of CTA 0 over all iterations gives the bandwidth.
__global__ void window_kernel(RankView v, int peer, std::uint32_t bytes, int window, int iters, int warmup,
                              std::uint64_t epoch0) {
    DeviceContext ctx{v.endpoints, nullptr, v.status};
    const std::uint64_t slot = static_cast<std::uint64_t>(blockIdx.x) * window * bytes;
    const RemoteRegion peer_flag{v.peer_flags[peer] + (v.world + blockIdx.x) * 8, 0};
    const std::uint64_t *my_flag = reinterpret_cast<const std::uint64_t *>(v.flags) + v.world + blockIdx.x;
    std::uint64_t t0 = 0;
    for (int it = 0; it < warmup + iters; ++it) {
        if (it == warmup) {
            __syncthreads();
            t0 = now_ns();
        }
        for (int w = 0; w < window; ++w) {
            const std::uint64_t off = slot + static_cast<std::uint64_t>(w) * bytes;
            aboleth::put_block(RemoteRegion{v.peer_recv[peer] + off, 0}, LocalRegion{v.send + off, 0}, bytes);
        }
        aboleth::signal_block(peer_flag, epoch0 + it + 1);
        if (threadIdx.x == 0)
            aboleth::wait_signal(ctx, my_flag, epoch0 + it + 1);  // the partner's window of the same iteration
        if (barrier_failed(v))
            break;
    }
    if (threadIdx.x == 0 && blockIdx.x == 0)
        v.times[0] = now_ns() - t0;
}

// All-to-all rounds: CTA p sends slot p to peer p, signals, and waits for peer p's slot of this round.
__global__ void alltoall_kernel(RankView v, std::uint32_t bytes, int rounds, int warmup, std::uint64_t epoch0) {
    DeviceContext ctx{v.endpoints, nullptr, v.status};
    const int peer = blockIdx.x;
    const RemoteRegion dst{v.peer_recv[peer] + v.rank * v.stride, 0};
    const LocalRegion src{v.send + peer * v.stride, 0};
    const RemoteRegion peer_flag{v.peer_flags[peer] + v.rank * 8, 0};
    const std::uint64_t *my_flag = reinterpret_cast<const std::uint64_t *>(v.flags) + peer;
    std::uint64_t t0 = 0;
    for (int it = 0; it < warmup + rounds; ++it) {
        if (it == warmup)
            t0 = now_ns();
        aboleth::put_block(dst, src, bytes);
        aboleth::signal_block(peer_flag, epoch0 + it + 1);
        if (threadIdx.x == 0)
            aboleth::wait_signal(ctx, my_flag, epoch0 + it + 1);
        if (barrier_failed(v))
            break;
    }
    if (threadIdx.x == 0)
        v.times[peer] = now_ns() - t0;
}

struct Options {
    int gpus = 0;  // 0: every visible GPU, at most 8
    std::string bench = "all";
    std::uint32_t bytes = 4096;
    int iters = 200, warmup = 20, window = 8, ctas = 8, threads = 256;
};

void usage() {
    std::puts("bench_tier1 [--gpus N] [--bench pingpong|window|alltoall|all] [--bytes B] [--iters I]\n"
              "            [--warmup W] [--window K] [--ctas C] [--threads T]");
}

Options parse(int argc, char **argv) {
    Options o;
    for (int i = 1; i < argc; ++i) {
        const std::string a = argv[i];
        auto value = [&]() -> const char * {
            if (i + 1 >= argc) {
                usage();
                std::exit(2);
            }
            return argv[++i];
        };
        if (a == "--gpus") o.gpus = std::atoi(value());
        else if (a == "--bench") o.bench = value();
        else if (a == "--bytes") o.bytes = static_cast<std::uint32_t>(std::strtoul(value(), nullptr, 10));
        else if (a == "--iters") o.iters = std::atoi(value());
        else if (a == "--warmup") o.warmup = std::atoi(value());
        else if (a == "--window") o.window = std::atoi(value());
        else if (a == "--ctas") o.ctas = std::atoi(value());
        else if (a == "--threads") o.threads = std::atoi(value());
        else {
            usage();
            std::exit(a == "--help" || a == "-h" ? 0 : 2);
        }
    }
    if (o.bytes < 16 || o.bytes % 16 || o.iters < 1 || o.warmup < 0 || o.window < 1 || o.ctas < 1 ||
        o.threads < 32 || o.threads > 1024 || o.threads % 32) {
        std::fputs("bytes must be a positive multiple of 16; threads a multiple of 32 up to 1024\n", stderr);
        std::exit(2);
    }
    return o;
}

struct Rank {
    int device = 0;
    cudaStream_t stream = nullptr;
    std::uint8_t *arena = nullptr;  // send | recv | flags
    std::uint64_t *endpoints = nullptr;
    unsigned long long *status = nullptr, *wrong = nullptr;
    std::uint64_t *times = nullptr;
    RankView view{};
};

double quantile(std::vector<double> v, double q) {
    std::sort(v.begin(), v.end());
    const double pos = q * (v.size() - 1);
    const std::size_t lo = static_cast<std::size_t>(pos);
    const std::size_t hi = std::min(lo + 1, v.size() - 1);
    return v[lo] + (v[hi] - v[lo]) * (pos - lo);
}

}  // namespace

int main(int argc, char **argv) {
    const Options opt = parse(argc, argv);
    int visible = 0;
    if (cudaGetDeviceCount(&visible) != cudaSuccess || visible < 1) {
        std::fputs("no CUDA device\n", stderr);
        return 77;  // "requirement not met" for gated runners
    }
    const int world = opt.gpus > 0 ? opt.gpus : std::min(visible, 8);
    if (world > visible || world > 8) {
        std::fprintf(stderr, "%d ranks need %d GPUs (one rank per GPU), %d visible\n", world, world, visible);
        return 77;
    }
    // One slot per peer for ping-pong / all-to-all, one window per CTA for the windowed puts.
    const std::uint64_t per_peer = std::max<std::uint64_t>(
        opt.bytes, (static_cast<std::uint64_t>(opt.ctas) * opt.window * opt.bytes + world - 1) / world);
    const std::uint64_t stride = (per_peer + 255) / 256 * 256;
    const std::uint64_t flag_words = world + opt.ctas;
    const std::uint64_t arena_bytes = 2 * world * stride + flag_words * 8;
    const int time_words = std::max(opt.iters, 8);

    std::vector<Rank> ranks(world);
    for (int r = 0; r < world; ++r) {
        Rank &k = ranks[r];
        k.device = r;
        CHECK_CUDA(cudaSetDevice(r));
        for (int p = 0; p < world; ++p) {
            if (p == r)
                continue;
            int can = 0;
            CHECK_CUDA(cudaDeviceCanAccessPeer(&can, r, p));
            if (!can) {
                std::fprintf(stderr, "GPU %d cannot map GPU %d\n", r, p);
                return 77;
            }
            const cudaError_t e = cudaDeviceEnablePeerAccess(p, 0);
            if (e != cudaSuccess && e != cudaErrorPeerAccessAlreadyEnabled)
                CHECK_CUDA(e);
            (void)cudaGetLastError();
        }
        CHECK_CUDA(cudaStreamCreate(&k.stream));
        CHECK_CUDA(cudaMalloc(&k.arena, arena_bytes));
        CHECK_CUDA(cudaMemset(k.arena, 0, arena_bytes));
        CHECK_CUDA(cudaMalloc(&k.endpoints, world * 8));
        CHECK_CUDA(cudaMalloc(&k.status, 8));
        CHECK_CUDA(cudaMalloc(&k.wrong, 8));
        CHECK_CUDA(cudaMalloc(&k.times, time_words * 8));
        CHECK_CUDA(cudaMemset(k.status, 0, 8));
        CHECK_CUDA(cudaMemset(k.wrong, 0, 8));
        std::vector<std::uint64_t> table(world, aboleth::abi::kKindP2P);
        CHECK_CUDA(cudaMemcpy(k.endpoints, table.data(), world * 8, cudaMemcpyHostToDevice));
        for (int p = 0; p < world; ++p)  // slot p carries the pattern salted by (sender, receiver)
            fill_pattern<<<64, 256>>>(k.arena + p * stride, stride, r * world + p);
        CHECK_CUDA(cudaDeviceSynchronize());
    }
    for (int r = 0; r < world; ++r) {
        RankView &v = ranks[r].view;
        v.endpoints = ranks[r].endpoints;
        v.status = ranks[r].status;
        v.send = reinterpret_cast<std::uint64_t>(ranks[r].arena);
        v.recv = v.send + world * stride;
        v.flags = v.send + 2 * world * stride;
        v.times = ranks[r].times;
        v.stride = stride;
        v.rank = r;
        v.world = world;
        for (int p = 0; p < world; ++p) {
            v.peer_recv[p] = reinterpret_cast<std::uint64_t>(ranks[p].arena) + world * stride;
            v.peer_flags[p] = reinterpret_cast<std::uint64_t>(ranks[p].arena) + 2 * world * stride;
        }
    }
    auto sync_all = [&]() {
        for (Rank &k : ranks) {
            CHECK_CUDA(cudaSetDevice(k.device));
            CHECK_CUDA(cudaStreamSynchronize(k.stream));
        }
    };
    auto read_times = [&](const Rank &k, int n) {
        std::vector<std::uint64_t> host(n);
        CHECK_CUDA(cudaSetDevice(k.device));
        CHECK_CUDA(cudaMemcpy(host.data(), k.times, n * 8, cudaMemcpyDeviceToHost));
        return host;
    };
    std::uint64_t epoch = 0;  // flags only grow; every benchmark starts above the last one's epochs
    const bool all = opt.bench == "all";
    const int partner = world > 1 ? 1 : 0;

    if (all || opt.bench == "pingpong") {
        // Rank 0 initiates; the responder is launched first so that it is already waiting.
        if (world > 1) {
            CHECK_CUDA(cudaSetDevice(ranks[1].device));
            pingpong_kernel<<<1, opt.threads, 0, ranks[1].stream>>>(ranks[1].view, 0, 0, opt.bytes, opt.iters,
                                                                     opt.warmup, epoch);
        }
        CHECK_CUDA(cudaSetDevice(ranks[0].device));
        pingpong_kernel<<<1, opt.threads, 0, ranks[0].stream>>>(ranks[0].view, partner, 1, opt.bytes, opt.iters,
                                                                 opt.warmup, epoch);
        CHECK_CUDA(cudaGetLastError());
        sync_all();
        epoch += opt.warmup + opt.iters;
        std::vector<double> us;
        for (std::uint64_t t : read_times(ranks[0], opt.iters))
            us.push_back(t * 1e-3);
        std::printf("{\"bench\": \"pingpong\", \"transport\": \"p2p\", \"gpus\": %d, \"loopback\": %s, \"bytes\": %u, "
                    "\"iters\": %d, \"round_trip_us\": {\"p50\": %.3f, \"p90\": %.3f, \"p99\": %.3f, \"min\": %.3f}}\n",
                    world, world > 1 ? "false" : "true", opt.bytes, opt.iters, quantile(us, 0.5), quantile(us, 0.9),
                    quantile(us, 0.99), quantile(us, 0.0));
    }
    if (all || opt.bench == "window") {
        const int senders = world > 1 ? 2 : 1;  // both directions at once with a partner
        for (int r = senders - 1; r >= 0; --r) {
            CHECK_CUDA(cudaSetDevice(ranks[r].device));
            window_kernel<<<opt.ctas, opt.threads, 0, ranks[r].stream>>>(
                ranks[r].view, world > 1 ? 1 - r : 0, opt.bytes, opt.window, opt.iters, opt.warmup, epoch);
        }
        CHECK_CUDA(cudaGetLastError());
        sync_all();
        epoch += opt.warmup + opt.iters;
        const double ns = static_cast<double>(read_times(ranks[0], 1)[0]);
        const double moved = static_cast<double>(opt.iters) * opt.ctas * opt.window * opt.bytes;
        std::printf("{\"bench\": \"window\", \"transport\": \"p2p\", \"gpus\": %d, \"loopback\": %s, \"bytes\": %u, "
                    "\"window\": %d, \"ctas\": %d, \"iters\": %d, \"gbs_per_direction\": %.2f, \"us_per_window\": %.3f}\n",
                    world, world > 1 ? "false" : "true", opt.bytes, opt.window, opt.ctas, opt.iters, moved / ns,
                    ns * 1e-3 / opt.iters);
    }
    if (all || opt.bench == "alltoall") {
        for (int r = world - 1; r >= 0; --r) {
            CHECK_CUDA(cudaSetDevice(ranks[r].device));
            alltoall_kernel<<<world, opt.threads, 0, ranks[r].stream>>>(ranks[r].view, opt.bytes, opt.iters,
                                                                        opt.warmup, epoch);
        }
        CHECK_CUDA(cudaGetLastError());
        sync_all();
        epoch += opt.warmup + opt.iters;
        double slowest = 0;
        for (const Rank &k : ranks)
            for (std::uint64_t t : read_times(k, world))
                slowest = std::max(slowest, static_cast<double>(t));
        unsigned long long wrong_total = 0;
        for (int r = 0; r < world; ++r) {
            CHECK_CUDA(cudaSetDevice(ranks[r].device));
            for (int s = 0; s < world; ++s)  // slot s must hold sender s's payload for this receiver
                check_pattern<<<64, 256>>>(ranks[r].arena + (world + s) * stride, opt.bytes, s * world + r,
                                           ranks[r].wrong);
            unsigned long long wrong = 0;
            CHECK_CUDA(cudaMemcpy(&wrong, ranks[r].wrong, 8, cudaMemcpyDeviceToHost));
            wrong_total += wrong;
        }
        const double round_ns = slowest / opt.iters;
        std::printf("{\"bench\": \"alltoall\", \"transport\": \"p2p\", \"gpus\": %d, \"bytes_per_peer\": %u, \"rounds\": %d, "
                    "\"round_us\": %.3f, \"busbw_gbs\": %.3f, \"wrong_bytes\": %llu}\n",
                    world, opt.bytes, opt.iters, round_ns * 1e-3,
                    world > 1 ? (world - 1) * static_cast<double>(opt.bytes) / round_ns : 0.0, wrong_total);
        if (wrong_total)
            return 1;
    }
    int failed = 0;
    for (Rank &k : ranks) {
        unsigned long long status = 0;
        CHECK_CUDA(cudaSetDevice(k.device));
        CHECK_CUDA(cudaMemcpy(&status, k.status, 8, cudaMemcpyDeviceToHost));
        if (status) {
            std::fprintf(stderr, "rank %d: transport status %llu\n", k.device, status);
            failed = 1;
        }
        cudaFree(k.arena);
        cudaFree(k.endpoints);
        cudaFree(k.status);
        cudaFree(k.wrong);
        cudaFree(k.times);
        cudaStreamDestroy(k.stream);
    }
    return failed;
}
