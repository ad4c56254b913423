// Emitted by the aboleth_b200 Tier-2 specializer.  Program 'tier1_put_inline64', transport proxy.
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
    // post_inline %t3: written into its batch at the submission
    std::uint64_t seq_v_b0 = 0;
    if (threadIdx.x == 0) {
        // one reservation, 1 command(s), one release store of ready_sequence
        abi::ProxyCommand cmds[1];
        cmds[0] = abi::ProxyCommand{(unsigned long long)(value), v_r2, 8, 0, v_r2_key, abi::kProxyCommandWeakSignal};
        t2::record(ab_status, proxy::submit(v_e1, cmds, 1, &seq_v_b0), 24577);
    }
    if (threadIdx.x == 0) t2::record(ab_status, proxy::poll(v_e1, seq_v_b0), 24833);
}
