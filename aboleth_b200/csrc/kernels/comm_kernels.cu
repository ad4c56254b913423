// All-to-all, put/signal chain, ping-pong and calibration kernels over NVLink
// peer memory, built on the Tier-1 device library.
//
// What the reference measures with one thread (or one warp) per peer
// (experiments/bench/kernels/bench_kernels.cuh:461-528) is measured here with
// `lanes` CTAs per peer, because on NVLink 5 a single CTA cannot fill a link:
// CTA (p, lane) owns slice `lane` of the message to peer p, publishes it with
// ONE release store however many puts the slice was split into, and waits for
// the same slice from that peer.  Flags are int64 epochs indexed
// [source_rank * lanes + lane], as in the reference's record transport
// (python/aboleth/records.py:13-85).
#include <cstdio>

#include "common.cuh"

namespace {

using aboleth::LocalRegion;
using aboleth::RemoteRegion;
using aboleth::Status;

struct AllToAllParams {
    const std::uint8_t *send;            // [world][stride] this rank's outgoing slices
    const std::uint64_t *peer_recv;      // [world] address of each peer's receive base
    const std::uint64_t *peer_flags;     // [world] address of each peer's flag array
    const std::uint64_t *my_flags;       // this rank's flag array [world * lanes]
    unsigned long long *status;          // 2 words
    std::uint64_t stride;                // bytes between per-peer slices
    std::uint64_t bytes;                 // payload bytes per peer
    std::uint64_t epoch0;                // epoch of round 0 is epoch0 + 1
    int rank, world, lanes, chain, batched, rounds, include_self, wait;
};

__device__ __forceinline__ std::uint64_t align_down16(std::uint64_t x) { return x & ~15ull; }

// Slice [begin, end) of `bytes` owned by `lane`, 16-byte aligned cuts.
__device__ __forceinline__ void lane_slice(std::uint64_t bytes, int lane, int lanes,
                                           std::uint64_t &begin, std::uint64_t &end) {
    const std::uint64_t per = align_down16((bytes + lanes - 1) / lanes + 15);
    begin = min(static_cast<std::uint64_t>(lane) * per, bytes);
    end = min(begin + per, bytes);
}

// MODE 0: vectorised ld/st by the whole CTA.  MODE 1: bulk-async (TMA) ring
// driven by one thread: global -> shared -> peer global, never multicast.
template <int MODE>
__global__ void __launch_bounds__(1024) alltoall_kernel(AllToAllParams p) {
    constexpr int kStages = 4;
    constexpr unsigned kChunk = 16384;
    extern __shared__ __align__(128) std::uint8_t smem[];
    __shared__ __align__(8) std::uint64_t bars[kStages];
    __shared__ int failed;

    const int peers = p.include_self ? p.world : p.world - 1;
    const int slot = blockIdx.x / p.lanes;
    const int lane = blockIdx.x % p.lanes;
    if (slot >= peers)
        return;
    const int peer = p.include_self ? slot : slot + (slot >= p.rank ? 1 : 0);

    std::uint64_t begin, end;
    lane_slice(p.bytes, lane, p.lanes, begin, end);
    const std::uint8_t *src = p.send + static_cast<std::uint64_t>(peer) * p.stride;
    std::uint8_t *dst = reinterpret_cast<std::uint8_t *>(p.peer_recv[peer]) +
                        static_cast<std::uint64_t>(p.rank) * p.stride;
    std::uint64_t *remote_flag = reinterpret_cast<std::uint64_t *>(p.peer_flags[peer]) +
                                 static_cast<std::uint64_t>(p.rank) * p.lanes + lane;
    const std::uint64_t *local_flag =
        p.my_flags + static_cast<std::uint64_t>(peer) * p.lanes + lane;

    unsigned bar_phase = 0;  // MODE 1: bit s = parity of stage s
    if (MODE == 1) {
        if (threadIdx.x == 0) {
            for (int s = 0; s < kStages; ++s)
                ab::mbar_init(&bars[s], 1);
            ab::mbar_fence_init();
            failed = 0;
        }
        __syncthreads();
    }

    // The slice is issued as `chain` puts.  Batched: one signal closes the
    // chain.  Unbatched: every put is followed by its own signal.
    const std::uint64_t span = end - begin;
    const std::uint64_t piece = align_down16((span + p.chain - 1) / p.chain + 15);

    for (int round = 0; round < p.rounds; ++round) {
        const std::uint64_t epoch = p.epoch0 + 1 + round;
        for (int c = 0; c < p.chain; ++c) {
            const std::uint64_t b = begin + min(static_cast<std::uint64_t>(c) * piece, span);
            const std::uint64_t e = begin + min(static_cast<std::uint64_t>(c + 1) * piece, span);
            if (MODE == 0) {
                aboleth::put_block(RemoteRegion{reinterpret_cast<std::uint64_t>(dst + b), 0},
                                   LocalRegion{reinterpret_cast<std::uint64_t>(src + b), 0}, e - b);
            } else if (threadIdx.x == 0 && !failed) {
                const std::uint64_t n = e - b;
                const std::uint64_t chunks = (n + kChunk - 1) / kChunk;
                const std::uint64_t ahead = chunks < kStages ? chunks : kStages;
                for (std::uint64_t i = 0; i < ahead; ++i) {
                    const unsigned len = static_cast<unsigned>(ab::min64(kChunk, n - i * kChunk));
                    ab::mbar_expect_tx(&bars[i], len);
                    ab::bulk_load(smem + i * kChunk, src + b + i * kChunk, len, &bars[i]);
                }
                for (std::uint64_t i = 0; i < chunks; ++i) {
                    const int s = static_cast<int>(i % kStages);
                    const unsigned len = static_cast<unsigned>(ab::min64(kChunk, n - i * kChunk));
                    if (!ab::mbar_wait(&bars[s], (bar_phase >> s) & 1u)) {
                        failed = 1;
                        ab::set_status(p.status, Status::Timeout, 0x100 + s);
                        break;
                    }
                    bar_phase ^= 1u << s;
                    ab::bulk_store(dst + b + i * kChunk, smem + s * kChunk, len);
                    ab::bulk_commit();
                    if (i + kStages < chunks) {
                        // The stage is reloaded once the store has read it.
                        ab::bulk_wait_read<0>();
                        const std::uint64_t j = i + kStages;
                        const unsigned len2 = static_cast<unsigned>(ab::min64(kChunk, n - j * kChunk));
                        ab::mbar_expect_tx(&bars[s], len2);
                        ab::bulk_load(smem + s * kChunk, src + b + j * kChunk, len2, &bars[s]);
                    }
                }
                // Writes placed and visible to this thread before any signal.
                ab::bulk_wait_all<0>();
            }
            if (!p.batched && c + 1 < p.chain)
                aboleth::signal_block(RemoteRegion{reinterpret_cast<std::uint64_t>(remote_flag), 0},
                                      epoch);
        }
        aboleth::signal_block(RemoteRegion{reinterpret_cast<std::uint64_t>(remote_flag), 0}, epoch);
        if (p.wait && threadIdx.x == 0) {
            const Status s = aboleth::wait_signal_status(local_flag, epoch);
            ab::set_status(p.status, s, 0x200 + peer);
        }
        __syncthreads();
    }
}

// Fill / check of the seeded payload.  `check` adds the number of wrong 8-byte
// words to *errors.
__global__ void fill_payload_kernel(std::uint64_t *buf, std::uint64_t words, std::uint64_t seed,
                                    unsigned sender, unsigned receiver) {
    for (std::uint64_t i = blockIdx.x * static_cast<std::uint64_t>(blockDim.x) + threadIdx.x;
         i < words; i += static_cast<std::uint64_t>(gridDim.x) * blockDim.x)
        buf[i] = ab::payload_word(seed, sender, receiver, i);
}

__global__ void check_payload_kernel(const std::uint64_t *buf, std::uint64_t words,
                                     std::uint64_t seed, unsigned sender, unsigned receiver,
                                     unsigned long long *errors) {
    unsigned long long bad = 0;
    for (std::uint64_t i = blockIdx.x * static_cast<std::uint64_t>(blockDim.x) + threadIdx.x;
         i < words; i += static_cast<std::uint64_t>(gridDim.x) * blockDim.x)
        bad += buf[i] != ab::payload_word(seed, sender, receiver, i);
    if (bad)
        atomicAdd(errors, bad);
}

// Ping-pong: the leader sends `chain` puts closed by one signal and waits for
// the echo; the follower waits and echoes.  One CTA.  samples[r] = round
// trip of round r in ns (leader only).
struct PingPongParams {
    const std::uint8_t *src;
    std::uint64_t peer_dst;      // peer's receive buffer
    std::uint64_t peer_flag;     // peer's flag word
    const std::uint64_t *my_flag;
    unsigned long long *status;
    std::uint64_t *samples;
    std::uint64_t bytes, epoch0;
    int leader, chain, rounds, batched;
};

__global__ void __launch_bounds__(1024) pingpong_kernel(PingPongParams p) {
    const std::uint64_t piece = ((p.bytes + p.chain - 1) / p.chain + 15) & ~15ull;
    for (int round = 0; round < p.rounds; ++round) {
        const std::uint64_t epoch = p.epoch0 + 1 + round;
        std::uint64_t t0 = 0;
        if (!p.leader) {
            if (threadIdx.x == 0)
                ab::set_status(p.status, aboleth::wait_signal_status(p.my_flag, epoch), 0x300);
            __syncthreads();
        } else if (threadIdx.x == 0) {
            t0 = aboleth::detail::globaltimer_ns();
        }
        for (int c = 0; c < p.chain; ++c) {
            const std::uint64_t b = min(static_cast<std::uint64_t>(c) * piece, p.bytes);
            const std::uint64_t e = min(static_cast<std::uint64_t>(c + 1) * piece, p.bytes);
            aboleth::put_block(RemoteRegion{p.peer_dst + b, 0},
                               LocalRegion{reinterpret_cast<std::uint64_t>(p.src + b), 0}, e - b);
            if (!p.batched && c + 1 < p.chain)
                aboleth::signal_block(RemoteRegion{p.peer_flag, 0}, epoch);
        }
        aboleth::signal_block(RemoteRegion{p.peer_flag, 0}, epoch);
        if (p.leader) {
            if (threadIdx.x == 0) {
                ab::set_status(p.status, aboleth::wait_signal_status(p.my_flag, epoch), 0x301);
                if (p.samples != nullptr)
                    p.samples[round] = aboleth::detail::globaltimer_ns() - t0;
            }
            __syncthreads();
        }
    }
}

// Single-thread Tier-1 exercise used by the unit tests: thread 0 of block 0
// performs put, put_inline, put_many_signal and a bounded wait through the
// public facade against an endpoint-handle table.
struct Tier1Params {
    const std::uint64_t *endpoints;
    unsigned long long *status;
    std::uint64_t dst, src, flag, inline_dst, wait_flag;
    std::uint64_t epoch, wait_epoch, timeout_ns;
    std::uint32_t bytes;
    int peer, pieces;
};

__global__ void tier1_exercise_kernel(Tier1Params p) {
    if (blockIdx.x != 0)
        return;
    aboleth::DeviceContext ctx{p.endpoints, nullptr, p.status};
    if (threadIdx.x == 0) {
        const aboleth::PeerRef ref = aboleth::open(ctx, p.peer);
        aboleth::put_inline(ctx, ref, RemoteRegion{p.inline_dst, 0}, p.epoch * 3 + 1);
        if (p.pieces <= 1) {
            aboleth::put_signal(ctx, ref, RemoteRegion{p.dst, 0}, LocalRegion{p.src, 0}, p.bytes,
                                RemoteRegion{p.flag, 0}, p.epoch);
        } else {
            aboleth::PutDesc descs[8];
            const int n = p.pieces > 8 ? 8 : p.pieces;
            const std::uint32_t piece = ((p.bytes + n - 1) / n + 15) & ~15u;
            for (int i = 0; i < n; ++i) {
                const std::uint32_t b = min(i * piece, p.bytes), e = min((i + 1) * piece, p.bytes);
                descs[i] = aboleth::PutDesc{p.dst + b, p.src + b, e - b, 0, 0, 0};
            }
            aboleth::put_many_signal(ctx, ref, descs, n, RemoteRegion{p.flag, 0}, p.epoch);
        }
        aboleth::quiet(ctx, ref);
        if (p.wait_flag != 0) {
            const Status s = aboleth::wait_signal_status(
                reinterpret_cast<const std::uint64_t *>(p.wait_flag), p.wait_epoch, p.timeout_ns);
            ab::set_status(p.status, s, 0x400);
        }
    }
}

// ---- endpoint probe -----------------------------------------------------------------
// One CTA per lane.  Per iteration: the CTA copies the lane's slice to the partner and
// publishes one epoch in the lane's flag there; "sender completed" on peer memory is the
// release store itself, so there is nothing further to wait for.  Nothing here waits on
// another rank.  (Role of the reference's probe kernel, python/aboleth/endpoint_probe.py:32-45.)
__global__ void __launch_bounds__(1024) probe_send_kernel(const std::uint8_t *payload,
                                                          std::uint64_t peer_receive,
                                                          std::uint64_t peer_flags,
                                                          const std::uint64_t *starts,
                                                          std::uint64_t chunk, int iterations) {
    const int lane = blockIdx.x;
    const std::uint64_t offset = chunk * lane;
    const std::uint64_t first = starts[lane];
    const aboleth::RemoteRegion dst{peer_receive + offset, 0};
    const aboleth::LocalRegion src{reinterpret_cast<std::uint64_t>(payload) + offset, 0};
    const aboleth::RemoteRegion flag{peer_flags + 8ull * lane, 0};
    for (int i = 0; i < iterations; ++i) {
        aboleth::put_block(dst, src, chunk);
        aboleth::signal_block(flag, first + i + 1);
    }
}

}  // namespace

AB_EXPORT int ab_alltoall(const void *send, const std::uint64_t *peer_recv,
                          const std::uint64_t *peer_flags, const std::uint64_t *my_flags,
                          unsigned long long *status, std::uint64_t stride, std::uint64_t bytes,
                          std::uint64_t epoch0, int rank, int world, int lanes, int chain,
                          int batched, int rounds, int include_self, int wait, int mode,
                          int threads, cudaStream_t stream) {
    if (world < 1 || lanes < 1 || chain < 1 || rounds < 1 || threads < 32 || threads > 1024)
        return -1;
    AllToAllParams p{static_cast<const std::uint8_t *>(send), peer_recv, peer_flags, my_flags,
                     status, stride, bytes, epoch0, rank, world, lanes, chain, batched, rounds,
                     include_self, wait};
    const int peers = include_self ? world : world - 1;
    if (peers == 0)
        return 0;
    if (mode == 1 && (bytes % 16 != 0 || stride % 16 != 0))
        return -2;  // bulk-async copies move whole 16-byte units
    const dim3 grid(peers * lanes);
    if (mode == 1) {
        const int smem = 4 * 16384;
        // Per device context, so set on every call rather than once per process.
        if (cudaFuncSetAttribute(alltoall_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) !=
            cudaSuccess)
            return -3;
        alltoall_kernel<1><<<grid, 32, smem, stream>>>(p);
    } else {
        alltoall_kernel<0><<<grid, threads, 0, stream>>>(p);
    }
    return ab::launch_result("alltoall");
}

AB_EXPORT int ab_fill_payload(void *buf, std::uint64_t bytes, std::uint64_t seed, unsigned sender,
                              unsigned receiver, cudaStream_t stream) {
    const std::uint64_t words = bytes / 8;
    if (words == 0)
        return 0;
    const int blocks = static_cast<int>(ab::min64((words + 255) / 256, 148 * 8));
    fill_payload_kernel<<<blocks, 256, 0, stream>>>(static_cast<std::uint64_t *>(buf), words, seed,
                                                    sender, receiver);
    return ab::launch_result("fill_payload");
}

AB_EXPORT int ab_check_payload(const void *buf, std::uint64_t bytes, std::uint64_t seed,
                               unsigned sender, unsigned receiver, unsigned long long *errors,
                               cudaStream_t stream) {
    const std::uint64_t words = bytes / 8;
    if (words == 0)
        return 0;
    const int blocks = static_cast<int>(ab::min64((words + 255) / 256, 148 * 8));
    check_payload_kernel<<<blocks, 256, 0, stream>>>(static_cast<const std::uint64_t *>(buf), words,
                                                     seed, sender, receiver, errors);
    return ab::launch_result("check_payload");
}

AB_EXPORT int ab_pingpong(const void *src, std::uint64_t peer_dst, std::uint64_t peer_flag,
                          const std::uint64_t *my_flag, unsigned long long *status,
                          std::uint64_t *samples, std::uint64_t bytes, std::uint64_t epoch0,
                          int leader, int chain, int rounds, int batched, int threads,
                          cudaStream_t stream) {
    if (chain < 1 || rounds < 1 || threads < 32 || threads > 1024)
        return -1;
    PingPongParams p{static_cast<const std::uint8_t *>(src), peer_dst, peer_flag, my_flag, status,
                     samples, bytes, epoch0, leader, chain, rounds, batched};
    pingpong_kernel<<<1, threads, 0, stream>>>(p);
    return ab::launch_result("pingpong");
}

AB_EXPORT int ab_tier1_exercise(const std::uint64_t *endpoints, unsigned long long *status,
                                std::uint64_t dst, std::uint64_t src, std::uint64_t flag,
                                std::uint64_t inline_dst, std::uint64_t wait_flag,
                                std::uint64_t epoch, std::uint64_t wait_epoch,
                                std::uint64_t timeout_ns, std::uint32_t bytes, int peer, int pieces,
                                cudaStream_t stream) {
    Tier1Params p{endpoints, status, dst, src, flag, inline_dst, wait_flag,
                  epoch, wait_epoch, timeout_ns, bytes, peer, pieces};
    tier1_exercise_kernel<<<1, 32, 0, stream>>>(p);
    return ab::launch_result("tier1_exercise");
}

// payload: local bytes; peer_receive / peer_flags: the partner's mapped addresses; starts: device
// u64 [lanes] with every lane's current epoch.  chunk must be a multiple of 16.
AB_EXPORT int ab_probe_send(const void *payload, std::uint64_t peer_receive, std::uint64_t peer_flags,
                            const std::uint64_t *starts, std::uint64_t chunk, int lanes, int warps,
                            int iterations, cudaStream_t stream) {
    if (lanes < 1 || lanes > 1024 || warps < 1 || warps > 32 || iterations < 0 || chunk % 16 ||
        (reinterpret_cast<std::uintptr_t>(payload) | peer_receive) % 16)
        return -1;
    probe_send_kernel<<<lanes, warps * 32, 0, stream>>>(static_cast<const std::uint8_t *>(payload),
                                                        peer_receive, peer_flags, starts, chunk,
                                                        iterations);
    return ab::launch_result("probe_send");
}
