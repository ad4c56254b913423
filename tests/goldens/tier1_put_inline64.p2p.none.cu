// Emitted by the aboleth_b200 Tier-2 specializer.  Program 'tier1_put_inline64', transport p2p.
#include "aboleth/tier2.cuh"

extern "C" __global__ void tier1_put_inline64(const unsigned long long * endpoints, int peer, unsigned long long dst, int dst_key, unsigned long long value, unsigned long long *ab_status) {
    using namespace aboleth;
    const long long pid = blockIdx.x;
    (void)pid;
    constexpr long long RANK = 0;
    (void)RANK;
    constexpr long long WORLD = 2;
    (void)WORLD;
    const unsigned long long v_e1 = endpoints[peer] & ~7ull;
    (void)v_e1;
    const unsigned long long v_r2 = (unsigned long long)(dst);
    const unsigned v_r2_key = dst_key;
    (void)v_r2_key;
    // post_inline %t3: carried out at its submission
    // submit %b0: 1 command(s); peer memory has no queue, nothing to reserve or ring
    if (threadIdx.x == 0) {
        t2::store_inline<std::uint64_t>(v_r2 + 0, (unsigned long long)(value));
    }
    // completion of %b0: program order (vacuous on peer memory)
}
