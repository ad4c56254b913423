// Emitted by the aboleth_b200 Tier-2 specializer.  Program 'windowed', transport efa (served by the host-proxy ring).
#include "aboleth/tier2.cuh"

extern "C" __global__ void windowed(unsigned long long payload, const unsigned long long * endpoints, const unsigned long long * remote_table, long long rounds, unsigned long long *ab_status) {
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
        const unsigned long long v_r2 = remote_table[2 * (1)] + ((pid*524288 + 0));
        const unsigned v_r2_key = (unsigned)remote_table[2 * (1) + 1];
        (void)v_r2_key;
        const unsigned long long v_l3 = (unsigned long long)((payload + pid*524288 + 0)) + (0);
        const unsigned v_l3_key = 0;
        (void)v_l3_key;
        // post_put %t4: written into its batch at the submission
        const unsigned long long v_r5 = remote_table[2 * (1)] + ((pid*524288 + 65536));
        const unsigned v_r5_key = (unsigned)remote_table[2 * (1) + 1];
        (void)v_r5_key;
        const unsigned long long v_l6 = (unsigned long long)((payload + pid*524288 + 65536)) + (0);
        const unsigned v_l6_key = 0;
        (void)v_l6_key;
        // post_put %t7: written into its batch at the submission
        const unsigned long long v_r8 = remote_table[2 * (1)] + ((pid*524288 + 131072));
        const unsigned v_r8_key = (unsigned)remote_table[2 * (1) + 1];
        (void)v_r8_key;
        const unsigned long long v_l9 = (unsigned long long)((payload + pid*524288 + 131072)) + (0);
        const unsigned v_l9_key = 0;
        (void)v_l9_key;
        // post_put %t10: written into its batch at the submission
        const unsigned long long v_r11 = remote_table[2 * (1)] + ((pid*524288 + 196608));
        const unsigned v_r11_key = (unsigned)remote_table[2 * (1) + 1];
        (void)v_r11_key;
        const unsigned long long v_l12 = (unsigned long long)((payload + pid*524288 + 196608)) + (0);
        const unsigned v_l12_key = 0;
        (void)v_l12_key;
        // post_put %t13: written into its batch at the submission
        const unsigned long long v_r14 = remote_table[2 * (1)] + ((pid*524288 + 262144));
        const unsigned v_r14_key = (unsigned)remote_table[2 * (1) + 1];
        (void)v_r14_key;
        const unsigned long long v_l15 = (unsigned long long)((payload + pid*524288 + 262144)) + (0);
        const unsigned v_l15_key = 0;
        (void)v_l15_key;
        // post_put %t16: written into its batch at the submission
        const unsigned long long v_r17 = remote_table[2 * (1)] + ((pid*524288 + 327680));
        const unsigned v_r17_key = (unsigned)remote_table[2 * (1) + 1];
        (void)v_r17_key;
        const unsigned long long v_l18 = (unsigned long long)((payload + pid*524288 + 327680)) + (0);
        const unsigned v_l18_key = 0;
        (void)v_l18_key;
        // post_put %t19: written into its batch at the submission
        const unsigned long long v_r20 = remote_table[2 * (1)] + ((pid*524288 + 393216));
        const unsigned v_r20_key = (unsigned)remote_table[2 * (1) + 1];
        (void)v_r20_key;
        const unsigned long long v_l21 = (unsigned long long)((payload + pid*524288 + 393216)) + (0);
        const unsigned v_l21_key = 0;
        (void)v_l21_key;
        // post_put %t22: written into its batch at the submission
        const unsigned long long v_r23 = remote_table[2 * (1)] + ((pid*524288 + 458752));
        const unsigned v_r23_key = (unsigned)remote_table[2 * (1) + 1];
        (void)v_r23_key;
        const unsigned long long v_l24 = (unsigned long long)((payload + pid*524288 + 458752)) + (0);
        const unsigned v_l24_key = 0;
        (void)v_l24_key;
        // post_put %t25: written into its batch at the submission
        std::uint64_t seq_v_b0 = 0;
        if (threadIdx.x == 0) {
            // one reservation, 8 command(s), one release store of ready_sequence
            abi::ProxyCommand cmds[8];
            cmds[0] = abi::ProxyCommand{v_l3, v_r2, (std::uint32_t)(65536), v_l3_key, v_r2_key, abi::kProxyCommandWrite};
            cmds[1] = abi::ProxyCommand{v_l6, v_r5, (std::uint32_t)(65536), v_l6_key, v_r5_key, abi::kProxyCommandWrite};
            cmds[2] = abi::ProxyCommand{v_l9, v_r8, (std::uint32_t)(65536), v_l9_key, v_r8_key, abi::kProxyCommandWrite};
            cmds[3] = abi::ProxyCommand{v_l12, v_r11, (std::uint32_t)(65536), v_l12_key, v_r11_key, abi::kProxyCommandWrite};
            cmds[4] = abi::ProxyCommand{v_l15, v_r14, (std::uint32_t)(65536), v_l15_key, v_r14_key, abi::kProxyCommandWrite};
            cmds[5] = abi::ProxyCommand{v_l18, v_r17, (std::uint32_t)(65536), v_l18_key, v_r17_key, abi::kProxyCommandWrite};
            cmds[6] = abi::ProxyCommand{v_l21, v_r20, (std::uint32_t)(65536), v_l21_key, v_r20_key, abi::kProxyCommandWrite};
            cmds[7] = abi::ProxyCommand{v_l24, v_r23, (std::uint32_t)(65536), v_l24_key, v_r23_key, abi::kProxyCommandWrite};
            t2::record(ab_status, proxy::submit(v_e1, cmds, 8, &seq_v_b0), 24577);
        }
        if (threadIdx.x == 0) t2::record(ab_status, proxy::poll(v_e1, seq_v_b0), 24833);
    }
    if (threadIdx.x == 0) t2::record(ab_status, proxy::drain(v_e1), 25090);
}
