// NCCL host-API arm of the all-to-all ladder: the baseline the Tier-1 numbers are read against.
//
// One process drives every GPU (rank r on GPU r, ncclCommInitAll).  A round is one grouped
// exchange: every rank sends `bytes` to every other rank and receives as much, posted as
// ncclSend / ncclRecv pairs inside one ncclGroupStart / ncclGroupEnd.  This is how the reference
// measures its NCCL host baseline (experiments/bench/bench_tier1_nccl_host.cu:40-54 for the
// exchange, :160-189 for the loop); here it is timed with CUDA events on each rank's stream,
// after warm-up, and the slowest rank's time per round is reported with the same bus-bandwidth
// formula as the other arms: (n - 1) * bytes / round time.
//
//   bench_nccl_host [--gpus N] [--bytes B] [--iters I] [--warmup W]
//
// Prints one JSON line; exits 77 when fewer than two GPUs are visible.
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include <cuda_runtime.h>
#include <nccl.h>

#define CHECK_CUDA(call)                                                                       \
    do {                                                                                       \
        cudaError_t e_ = (call);                                                               \
        if (e_ != cudaSuccess) {                                                               \
            std::fprintf(stderr, "%s: %s\n", #call, cudaGetErrorString(e_));                   \
            return 1;                                                                          \
        }                                                                                      \
    } while (0)
#define CHECK_NCCL(call)                                                                       \
    do {                                                                                       \
        ncclResult_t r_ = (call);                                                              \
        if (r_ != ncclSuccess) {                                                               \
            std::fprintf(stderr, "%s: %s\n", #call, ncclGetErrorString(r_));                   \
            return 1;                                                                          \
        }                                                                                      \
    } while (0)

int main(int argc, char **argv) {
    int gpus = 0, iters = 200, warmup = 20;
    long long bytes = 65536;
    for (int i = 1; i + 1 < argc; i += 2) {
        const std::string key = argv[i];
        if (key == "--gpus")
            gpus = std::atoi(argv[i + 1]);
        else if (key == "--bytes")
            bytes = std::atoll(argv[i + 1]);
        else if (key == "--iters")
            iters = std::atoi(argv[i + 1]);
        else if (key == "--warmup")
            warmup = std::atoi(argv[i + 1]);
        else {
            std::fprintf(stderr, "unknown option %s\n", argv[i]);
            return 2;
        }
    }
    int visible = 0;
    if (cudaGetDeviceCount(&visible) != cudaSuccess)
        visible = 0;
    if (gpus == 0)
        gpus = visible;
    if (visible < 2 || gpus < 2 || gpus > visible) {
        std::fprintf(stderr, "needs at least two visible GPUs (visible %d, asked %d)\n", visible, gpus);
        return 77;
    }
    if (bytes < 1 || iters < 1 || warmup < 3) {
        std::fprintf(stderr, "need bytes >= 1, iters >= 1, warmup >= 3\n");
        return 2;
    }

    std::vector<int> devices(gpus);
    for (int r = 0; r < gpus; ++r)
        devices[r] = r;
    std::vector<ncclComm_t> comms(gpus);
    CHECK_NCCL(ncclCommInitAll(comms.data(), gpus, devices.data()));
    std::vector<cudaStream_t> streams(gpus);
    std::vector<char *> send(gpus), recv(gpus);
    std::vector<cudaEvent_t> begin(gpus), end(gpus);
    const size_t slab = static_cast<size_t>(bytes) * gpus;
    for (int r = 0; r < gpus; ++r) {
        CHECK_CUDA(cudaSetDevice(r));
        CHECK_CUDA(cudaStreamCreateWithFlags(&streams[r], cudaStreamNonBlocking));
        CHECK_CUDA(cudaMalloc(&send[r], slab));
        CHECK_CUDA(cudaMalloc(&recv[r], slab));
        CHECK_CUDA(cudaMemset(send[r], r + 1, slab));
        CHECK_CUDA(cudaMemset(recv[r], 0, slab));
        CHECK_CUDA(cudaEventCreate(&begin[r]));
        CHECK_CUDA(cudaEventCreate(&end[r]));
    }

    const auto exchange = [&]() -> int {
        CHECK_NCCL(ncclGroupStart());
        for (int r = 0; r < gpus; ++r)
            for (int p = 0; p < gpus; ++p) {
                if (p == r)
                    continue;
                CHECK_NCCL(ncclSend(send[r] + static_cast<size_t>(p) * bytes, bytes, ncclChar, p, comms[r], streams[r]));
                CHECK_NCCL(ncclRecv(recv[r] + static_cast<size_t>(p) * bytes, bytes, ncclChar, p, comms[r], streams[r]));
            }
        CHECK_NCCL(ncclGroupEnd());
        return 0;
    };

    for (int i = 0; i < warmup; ++i)
        if (exchange() != 0)
            return 1;
    for (int r = 0; r < gpus; ++r) {
        CHECK_CUDA(cudaSetDevice(r));
        CHECK_CUDA(cudaStreamSynchronize(streams[r]));
    }
    for (int r = 0; r < gpus; ++r) {
        CHECK_CUDA(cudaSetDevice(r));
        CHECK_CUDA(cudaEventRecord(begin[r], streams[r]));
    }
    for (int i = 0; i < iters; ++i)
        if (exchange() != 0)
            return 1;
    float slowest_ms = 0.f;
    for (int r = 0; r < gpus; ++r) {
        CHECK_CUDA(cudaSetDevice(r));
        CHECK_CUDA(cudaEventRecord(end[r], streams[r]));
    }
    for (int r = 0; r < gpus; ++r) {
        CHECK_CUDA(cudaSetDevice(r));
        CHECK_CUDA(cudaEventSynchronize(end[r]));
        float ms = 0.f;
        CHECK_CUDA(cudaEventElapsedTime(&ms, begin[r], end[r]));
        slowest_ms = ms > slowest_ms ? ms : slowest_ms;
    }

    // Self-check: rank r's slot p holds what rank p sent (bytes of value p + 1).
    long long wrong = 0;
    std::vector<char> host(static_cast<size_t>(bytes));
    for (int r = 0; r < gpus; ++r) {
        CHECK_CUDA(cudaSetDevice(r));
        for (int p = 0; p < gpus; ++p) {
            if (p == r)
                continue;
            CHECK_CUDA(cudaMemcpy(host.data(), recv[r] + static_cast<size_t>(p) * bytes, bytes, cudaMemcpyDeviceToHost));
            for (long long i = 0; i < bytes; ++i)
                wrong += host[i] != static_cast<char>(p + 1);
        }
    }
    const double round_us = slowest_ms * 1e3 / iters;
    std::printf("{\"bench\": \"alltoall\", \"arm\": \"nccl_host\", \"n_gpus\": %d, \"bytes_per_peer\": %lld, "
                "\"iters\": %d, \"warmup\": %d, \"round_us\": %.3f, \"busbw_gbs\": %.3f, \"wrong_bytes\": %lld}\n",
                gpus, bytes, iters, warmup, round_us, (gpus - 1) * static_cast<double>(bytes) / round_us / 1e3, wrong);
    for (int r = 0; r < gpus; ++r) {
        cudaSetDevice(r);
        cudaFree(send[r]);
        cudaFree(recv[r]);
        cudaEventDestroy(begin[r]);
        cudaEventDestroy(end[r]);
        cudaStreamDestroy(streams[r]);
        ncclCommDestroy(comms[r]);
    }
    return wrong == 0 ? 0 : 1;
}
