// Emitted by the aboleth_b200 Tier-2 specializer.  Program 'pingpong_follower', transport rdma (served by the host-proxy ring).
#include "aboleth/tier2.cuh"

extern "C" __global__ void pingpong_follower(unsigned long long payload, const unsigned long long * endpoints, const unsigned long long * remote_table, unsigned long long my_flag, long long rounds, long long epoch0, unsigned long long *ab_status) {
    using namespace aboleth;
    const long long pid = blockIdx.x;
    (void)pid;
    constexpr long long RANK = 0;
    (void)RANK;
    constexpr long long WORLD = 2;
    (void)WORLD;
    const unsigned long long v_e1 = endpoints[1] & ~7ull;
    (void)v_e1;
    for (long long round = 0; round < rounds; ++round) {
        t2::wait_signal_cta((unsigned long long)(my_flag), (std::uint64_t)((epoch0 + round + 1)), ab_status, 20480);
        const unsigned long long v_r2 = remote_table[2 * (1)] + (0);
        const unsigned v_r2_key = (unsigned)remote_table[2 * (1) + 1];
        (void)v_r2_key;
        const unsigned long long v_l3 = (unsigned long long)((payload + 0)) + (0);
        const unsigned v_l3_key = 0;
        (void)v_l3_key;
        // post_put %t4: written into its batch at the submission
        const unsigned long long v_r5 = remote_table[2 * (1)] + (4096);
        const unsigned v_r5_key = (unsigned)remote_table[2 * (1) + 1];
        (void)v_r5_key;
        // post_signal %s6: written into its batch at the submission
        std::uint64_t seq_v_b0 = 0;
        if (threadIdx.x == 0) {
            // one reservation, 2 command(s), one release store of ready_sequence
            abi::ProxyCommand cmds[2];
            cmds[0] = abi::ProxyCommand{v_l3, v_r2, (std::uint32_t)(4096), v_l3_key, v_r2_key, abi::kProxyCommandWrite};
            cmds[1] = abi::ProxyCommand{(unsigned long long)((epoch0 + round + 1)), v_r5, 8, 0, v_r5_key, abi::kProxyCommandStrongSignal};
            t2::record(ab_status, proxy::submit(v_e1, cmds, 2, &seq_v_b0), 24577);
        }
        if (threadIdx.x == 0) t2::record(ab_status, proxy::poll(v_e1, seq_v_b0), 24833);
    }
}
