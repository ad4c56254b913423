// A user kernel written against the Tier-1 header: every CTA puts its slice to the peer with the
// whole CTA copying, publishes it with one release, and waits (bounded) for the peer's slice.
// `endpoints` is the handle table a World (or Runtime.create_local_endpoint) provides.
#include "aboleth/device.cuh"

extern "C" __global__ void exchange_slices(const std::uint64_t *endpoints, unsigned long long *status,
                                           unsigned long long peer_recv, unsigned long long peer_flags,
                                           unsigned long long send, unsigned long long my_flags,
                                           unsigned long long slice_bytes, unsigned long long epoch) {
    aboleth::DeviceContext ctx{endpoints, nullptr, status};
    const unsigned long long offset = blockIdx.x * slice_bytes;
    aboleth::put_block(aboleth::RemoteRegion{peer_recv + offset, 0}, aboleth::LocalRegion{send + offset, 0},
                       slice_bytes);
    aboleth::signal_block(aboleth::RemoteRegion{peer_flags + blockIdx.x * 8, 0}, epoch);
    if (threadIdx.x == 0) {
        aboleth::wait_signal(ctx, reinterpret_cast<const std::uint64_t *>(my_flags) + blockIdx.x, epoch);
        // A small control word travels out of a register.
        aboleth::put_inline(ctx, 0, aboleth::RemoteRegion{peer_flags + (gridDim.x + blockIdx.x) * 8, 0},
                            epoch * 1000 + blockIdx.x);
    }
}
