// Emitted by the aboleth_b200 Tier-2 specializer.  Program 'stream_fused', transport rdma (served by the host-proxy ring).
#include "aboleth/tier2.cuh"

extern "C" __global__ void stream_fused(unsigned long long payload, const unsigned long long * endpoints, const unsigned long long * remote_table, long long rounds, unsigned long long *ab_status) {
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
        const unsigned long long v_l2 = (unsigned long long)((payload + 0)) + (0);
        const unsigned v_l2_key = 0;
        (void)v_l2_key;
        const unsigned long long v_r3 = remote_table[2 * (1)] + (0);
        const unsigned v_r3_key = (unsigned)remote_table[2 * (1) + 1];
        (void)v_r3_key;
        // post_put %t4: written into its batch at the submission
        const unsigned long long v_l5 = (unsigned long long)((payload + 1024)) + (0);
        const unsigned v_l5_key = 0;
        (void)v_l5_key;
        const unsigned long long v_r6 = remote_table[2 * (1)] + (1024);
        const unsigned v_r6_key = (unsigned)remote_table[2 * (1) + 1];
        (void)v_r6_key;
        // post_put %t7: written into its batch at the submission
        const unsigned long long v_l8 = (unsigned long long)((payload + 2048)) + (0);
        const unsigned v_l8_key = 0;
        (void)v_l8_key;
        const unsigned long long v_r9 = remote_table[2 * (1)] + (2048);
        const unsigned v_r9_key = (unsigned)remote_table[2 * (1) + 1];
        (void)v_r9_key;
        // post_put %t10: written into its batch at the submission
        const unsigned long long v_l11 = (unsigned long long)((payload + 3072)) + (0);
        const unsigned v_l11_key = 0;
        (void)v_l11_key;
        const unsigned long long v_r12 = remote_table[2 * (1)] + (3072);
        const unsigned v_r12_key = (unsigned)remote_table[2 * (1) + 1];
        (void)v_r12_key;
        // post_put %t13: written into its batch at the submission
        const unsigned long long v_l14 = (unsigned long long)((payload + 4096)) + (0);
        const unsigned v_l14_key = 0;
        (void)v_l14_key;
        const unsigned long long v_r15 = remote_table[2 * (1)] + (4096);
        const unsigned v_r15_key = (unsigned)remote_table[2 * (1) + 1];
        (void)v_r15_key;
        // post_put %t16: written into its batch at the submission
        const unsigned long long v_l17 = (unsigned long long)((payload + 5120)) + (0);
        const unsigned v_l17_key = 0;
        (void)v_l17_key;
        const unsigned long long v_r18 = remote_table[2 * (1)] + (5120);
        const unsigned v_r18_key = (unsigned)remote_table[2 * (1) + 1];
        (void)v_r18_key;
        // post_put %t19: written into its batch at the submission
        const unsigned long long v_l20 = (unsigned long long)((payload + 6144)) + (0);
        const unsigned v_l20_key = 0;
        (void)v_l20_key;
        const unsigned long long v_r21 = remote_table[2 * (1)] + (6144);
        const unsigned v_r21_key = (unsigned)remote_table[2 * (1) + 1];
        (void)v_r21_key;
        // post_put %t22: written into its batch at the submission
        const unsigned long long v_l23 = (unsigned long long)((payload + 7168)) + (0);
        const unsigned v_l23_key = 0;
        (void)v_l23_key;
        const unsigned long long v_r24 = remote_table[2 * (1)] + (7168);
        const unsigned v_r24_key = (unsigned)remote_table[2 * (1) + 1];
        (void)v_r24_key;
        // post_put %t25: written into its batch at the submission
        const unsigned long long v_r26 = remote_table[2 * (1)] + (8192);
        const unsigned v_r26_key = (unsigned)remote_table[2 * (1) + 1];
        (void)v_r26_key;
        // post_signal %s27: written into its batch at the submission
        std::uint64_t seq_v_b0 = 0;
        if (threadIdx.x == 0) {
            // one reservation, 9 command(s), one release store of ready_sequence
            abi::ProxyCommand cmds[9];
            cmds[0] = abi::ProxyCommand{v_l2, v_r3, (std::uint32_t)(1024), v_l2_key, v_r3_key, abi::kProxyCommandWrite};
            cmds[1] = abi::ProxyCommand{v_l5, v_r6, (std::uint32_t)(1024), v_l5_key, v_r6_key, abi::kProxyCommandWrite};
            cmds[2] = abi::ProxyCommand{v_l8, v_r9, (std::uint32_t)(1024), v_l8_key, v_r9_key, abi::kProxyCommandWrite};
            cmds[3] = abi::ProxyCommand{v_l11, v_r12, (std::uint32_t)(1024), v_l11_key, v_r12_key, abi::kProxyCommandWrite};
            cmds[4] = abi::ProxyCommand{v_l14, v_r15, (std::uint32_t)(1024), v_l14_key, v_r15_key, abi::kProxyCommandWrite};
            cmds[5] = abi::ProxyCommand{v_l17, v_r18, (std::uint32_t)(1024), v_l17_key, v_r18_key, abi::kProxyCommandWrite};
            cmds[6] = abi::ProxyCommand{v_l20, v_r21, (std::uint32_t)(1024), v_l20_key, v_r21_key, abi::kProxyCommandWrite};
            cmds[7] = abi::ProxyCommand{v_l23, v_r24, (std::uint32_t)(1024), v_l23_key, v_r24_key, abi::kProxyCommandWrite};
            cmds[8] = abi::ProxyCommand{(unsigned long long)((round + 1)), v_r26, 8, 0, v_r26_key, abi::kProxyCommandStrongSignal};
            t2::record(ab_status, proxy::submit(v_e1, cmds, 9, &seq_v_b0), 24577);
        }
        if (threadIdx.x == 0) t2::record(ab_status, proxy::poll(v_e1, seq_v_b0), 24833);
    }
}
