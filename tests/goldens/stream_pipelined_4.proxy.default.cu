// Emitted by the aboleth_b200 Tier-2 specializer.  Program 'stream_pipelined', transport proxy.
#include "aboleth/tier2.cuh"

extern "C" __global__ void stream_pipelined(unsigned long long payload, const unsigned long long * endpoints, const unsigned long long * remote_table, long long rounds, unsigned long long *ab_status) {
    using namespace aboleth;
    const long long pid = blockIdx.x;
    (void)pid;
    constexpr long long RANK = 0;
    (void)RANK;
    constexpr long long WORLD = 2;
    (void)WORLD;
    const unsigned long long v_e1 = endpoints[1] & ~7ull;
    (void)v_e1;
    long long ab_published_0 = (((0) + 1)) - 1; (void)ab_published_0;
    long long ab_published_1 = (((0) + 1)) - 1; (void)ab_published_1;
    long long ab_published_2 = (((0) + 1)) - 1; (void)ab_published_2;
    long long ab_published_3 = (((0) + 1)) - 1; (void)ab_published_3;
    for (long long round = 0; round < rounds; ++round) {
        const unsigned long long v_l2 = (unsigned long long)((payload + 0)) + (0);
        const unsigned v_l2_key = 0;
        (void)v_l2_key;
        const unsigned long long v_r3 = remote_table[2 * (1)] + (0);
        const unsigned v_r3_key = (unsigned)remote_table[2 * (1) + 1];
        (void)v_r3_key;
        // post_put %t4: written into its batch at the submission
        const unsigned long long v_r5 = remote_table[2 * (1)] + (1024);
        const unsigned v_r5_key = (unsigned)remote_table[2 * (1) + 1];
        (void)v_r5_key;
        // post_signal %s6: written into its batch at the submission
        const unsigned long long v_l7 = (unsigned long long)((payload + 256)) + (0);
        const unsigned v_l7_key = 0;
        (void)v_l7_key;
        const unsigned long long v_r8 = remote_table[2 * (1)] + (256);
        const unsigned v_r8_key = (unsigned)remote_table[2 * (1) + 1];
        (void)v_r8_key;
        // post_put %t9: written into its batch at the submission
        const unsigned long long v_r10 = remote_table[2 * (1)] + (1032);
        const unsigned v_r10_key = (unsigned)remote_table[2 * (1) + 1];
        (void)v_r10_key;
        // post_signal %s11: written into its batch at the submission
        const unsigned long long v_l12 = (unsigned long long)((payload + 512)) + (0);
        const unsigned v_l12_key = 0;
        (void)v_l12_key;
        const unsigned long long v_r13 = remote_table[2 * (1)] + (512);
        const unsigned v_r13_key = (unsigned)remote_table[2 * (1) + 1];
        (void)v_r13_key;
        // post_put %t14: written into its batch at the submission
        const unsigned long long v_r15 = remote_table[2 * (1)] + (1040);
        const unsigned v_r15_key = (unsigned)remote_table[2 * (1) + 1];
        (void)v_r15_key;
        // post_signal %s16: written into its batch at the submission
        const unsigned long long v_l17 = (unsigned long long)((payload + 768)) + (0);
        const unsigned v_l17_key = 0;
        (void)v_l17_key;
        const unsigned long long v_r18 = remote_table[2 * (1)] + (768);
        const unsigned v_r18_key = (unsigned)remote_table[2 * (1) + 1];
        (void)v_r18_key;
        // post_put %t19: written into its batch at the submission
        const unsigned long long v_r20 = remote_table[2 * (1)] + (1048);
        const unsigned v_r20_key = (unsigned)remote_table[2 * (1) + 1];
        (void)v_r20_key;
        // post_signal %s21: written into its batch at the submission
        std::uint64_t seq_v_b3 = 0;
        if (threadIdx.x == 0) {
            // one reservation, 8 command(s), one release store of ready_sequence
            abi::ProxyCommand cmds[8];
            cmds[0] = abi::ProxyCommand{v_l2, v_r3, (std::uint32_t)(256), v_l2_key, v_r3_key, abi::kProxyCommandWrite};
            cmds[1] = abi::ProxyCommand{v_l7, v_r8, (std::uint32_t)(256), v_l7_key, v_r8_key, abi::kProxyCommandWrite};
            cmds[2] = abi::ProxyCommand{v_l12, v_r13, (std::uint32_t)(256), v_l12_key, v_r13_key, abi::kProxyCommandWrite};
            cmds[3] = abi::ProxyCommand{v_l17, v_r18, (std::uint32_t)(256), v_l17_key, v_r18_key, abi::kProxyCommandWrite};
            cmds[4] = ((((((round) & 3) == 3) || ((round == rounds - 1))) || ((round) == (rounds) - 1))) ? abi::ProxyCommand{(unsigned long long)((round + 1)), v_r5, 8, 0, v_r5_key, abi::kProxyCommandStrongSignal} : abi::ProxyCommand{0, 0, 0, 0, 0, abi::kProxyCommandNop};
            cmds[5] = ((((((round) & 3) == 3) || ((round == rounds - 1))) || ((round) == (rounds) - 1))) ? abi::ProxyCommand{(unsigned long long)((round + 1)), v_r10, 8, 0, v_r10_key, abi::kProxyCommandStrongSignal} : abi::ProxyCommand{0, 0, 0, 0, 0, abi::kProxyCommandNop};
            cmds[6] = ((((((round) & 3) == 3) || ((round == rounds - 1))) || ((round) == (rounds) - 1))) ? abi::ProxyCommand{(unsigned long long)((round + 1)), v_r15, 8, 0, v_r15_key, abi::kProxyCommandStrongSignal} : abi::ProxyCommand{0, 0, 0, 0, 0, abi::kProxyCommandNop};
            cmds[7] = ((((((round) & 3) == 3) || ((round == rounds - 1))) || ((round) == (rounds) - 1))) ? abi::ProxyCommand{(unsigned long long)((round + 1)), v_r20, 8, 0, v_r20_key, abi::kProxyCommandStrongSignal} : abi::ProxyCommand{0, 0, 0, 0, 0, abi::kProxyCommandNop};
            t2::record(ab_status, proxy::submit(v_e1, cmds, 8, &seq_v_b3), 24577);
        }
        if (((((round) & 3) == 3) || ((round == rounds - 1))) || ((round) == (rounds) - 1)) ab_published_3 = ((round + 1));
        if (((((round) & 3) == 3) || ((round == rounds - 1))) || ((round) == (rounds) - 1)) ab_published_2 = ((round + 1));
        if (((((round) & 3) == 3) || ((round == rounds - 1))) || ((round) == (rounds) - 1)) ab_published_1 = ((round + 1));
        if (((((round) & 3) == 3) || ((round == rounds - 1))) || ((round) == (rounds) - 1)) ab_published_0 = ((round + 1));
        if (threadIdx.x == 0 && (((((round) & 3) == 3) || ((round == rounds - 1))))) t2::record(ab_status, proxy::poll(v_e1, seq_v_b3), 24833);
    }
    if (threadIdx.x == 0) t2::record(ab_status, proxy::drain(v_e1), 25090);
}
