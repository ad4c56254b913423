// Destination checks for debug builds of Tier-1 device code.
//
// compute-sanitizer style tools are not always available where these kernels run, and a
// peer store to a wrong address corrupts ANOTHER process's memory.  A kernel compiled
// with -DABOLETH_DEBUG_BOUNDS therefore carries, in its DeviceContext, the list of
// windows it may write (the peers' registered regions, as the host knows them from
// World.exchange_regions) and checks the destination of every put, put_inline and
// signal against it.  A destination outside every window is not written: the call
// records Status::Malformed in the context's status word and stores the offending
// (address, bytes, count of violations) in three 64-bit words the host reads after the
// launch.  Nothing traps.  Release builds (the macro undefined) carry none of this.
//
// This header is plain C++ (no PTX) so that the rule itself is unit-tested on the host.
// The reference has no counterpart: it relies on verifiers and differential tests.
#pragma once

#include <cstdint>

#if defined(__CUDACC__)
#define ABOLETH_BOUNDS_FN __host__ __device__ inline
#else
#define ABOLETH_BOUNDS_FN inline
#endif

namespace aboleth {
namespace debug {

struct Window {
    std::uint64_t base;
    std::uint64_t bytes;
};

struct Bounds {
    const Window *windows = nullptr;  // null or count 0: nothing is checked
    std::uint32_t count = 0;
    unsigned long long *violation = nullptr;  // [0] address, [1] bytes, [2] number of violations
};

// Is [address, address + bytes) inside one window?  An empty access is always fine; a
// range that wraps around the address space never is.
ABOLETH_BOUNDS_FN bool inside(const Bounds &bounds, std::uint64_t address, std::uint64_t bytes) {
    if (bounds.windows == nullptr || bounds.count == 0 || bytes == 0)
        return true;
    const std::uint64_t end = address + bytes;
    if (end < address)
        return false;
    for (std::uint32_t i = 0; i < bounds.count; ++i) {
        const Window &w = bounds.windows[i];
        if (address >= w.base && end <= w.base + w.bytes && w.base + w.bytes >= w.base)
            return true;
    }
    return false;
}

}  // namespace debug
}  // namespace aboleth
