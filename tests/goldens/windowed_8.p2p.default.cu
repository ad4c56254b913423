// Emitted by the aboleth_b200 Tier-2 specializer.  Program 'windowed', transport p2p.
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
        // post_put %t4: carried out at its submission
        const unsigned long long v_r5 = remote_table[2 * (1)] + ((pid*524288 + 65536));
        const unsigned v_r5_key = (unsigned)remote_table[2 * (1) + 1];
        (void)v_r5_key;
        const unsigned long long v_l6 = (unsigned long long)((payload + pid*524288 + 65536)) + (0);
        const unsigned v_l6_key = 0;
        (void)v_l6_key;
        // post_put %t7: carried out at its submission
        const unsigned long long v_r8 = remote_table[2 * (1)] + ((pid*524288 + 131072));
        const unsigned v_r8_key = (unsigned)remote_table[2 * (1) + 1];
        (void)v_r8_key;
        const unsigned long long v_l9 = (unsigned long long)((payload + pid*524288 + 131072)) + (0);
        const unsigned v_l9_key = 0;
        (void)v_l9_key;
        // post_put %t10: carried out at its submission
        const unsigned long long v_r11 = remote_table[2 * (1)] + ((pid*524288 + 196608));
        const unsigned v_r11_key = (unsigned)remote_table[2 * (1) + 1];
        (void)v_r11_key;
        const unsigned long long v_l12 = (unsigned long long)((payload + pid*524288 + 196608)) + (0);
        const unsigned v_l12_key = 0;
        (void)v_l12_key;
        // post_put %t13: carried out at its submission
        const unsigned long long v_r14 = remote_table[2 * (1)] + ((pid*524288 + 262144));
        const unsigned v_r14_key = (unsigned)remote_table[2 * (1) + 1];
        (void)v_r14_key;
        const unsigned long long v_l15 = (unsigned long long)((payload + pid*524288 + 262144)) + (0);
        const unsigned v_l15_key = 0;
        (void)v_l15_key;
        // post_put %t16: carried out at its submission
        const unsigned long long v_r17 = remote_table[2 * (1)] + ((pid*524288 + 327680));
        const unsigned v_r17_key = (unsigned)remote_table[2 * (1) + 1];
        (void)v_r17_key;
        const unsigned long long v_l18 = (unsigned long long)((payload + pid*524288 + 327680)) + (0);
        const unsigned v_l18_key = 0;
        (void)v_l18_key;
        // post_put %t19: carried out at its submission
        const unsigned long long v_r20 = remote_table[2 * (1)] + ((pid*524288 + 393216));
        const unsigned v_r20_key = (unsigned)remote_table[2 * (1) + 1];
        (void)v_r20_key;
        const unsigned long long v_l21 = (unsigned long long)((payload + pid*524288 + 393216)) + (0);
        const unsigned v_l21_key = 0;
        (void)v_l21_key;
        // post_put %t22: carried out at its submission
        const unsigned long long v_r23 = remote_table[2 * (1)] + ((pid*524288 + 458752));
        const unsigned v_r23_key = (unsigned)remote_table[2 * (1) + 1];
        (void)v_r23_key;
        const unsigned long long v_l24 = (unsigned long long)((payload + pid*524288 + 458752)) + (0);
        const unsigned v_l24_key = 0;
        (void)v_l24_key;
        // post_put %t25: carried out at its submission
        // submit %b0: 8 command(s); peer memory has no queue, nothing to reserve or ring
        t2::put_p2p<2048>(v_r2, v_l3, (std::uint32_t)(65536), 256u, false);
        t2::put_p2p<2048>(v_r5, v_l6, (std::uint32_t)(65536), 256u, false);
        t2::put_p2p<2048>(v_r8, v_l9, (std::uint32_t)(65536), 256u, false);
        t2::put_p2p<2048>(v_r11, v_l12, (std::uint32_t)(65536), 256u, false);
        t2::put_p2p<2048>(v_r14, v_l15, (std::uint32_t)(65536), 256u, false);
        t2::put_p2p<2048>(v_r17, v_l18, (std::uint32_t)(65536), 256u, false);
        t2::put_p2p<2048>(v_r20, v_l21, (std::uint32_t)(65536), 256u, false);
        t2::put_p2p<2048>(v_r23, v_l24, (std::uint32_t)(65536), 256u, false);
        __syncthreads();
        if (threadIdx.x == 0) detail::fence_acq_rel_sys();  // no signal follows: membar.sys
        // completion of %b0: program order (vacuous on peer memory)
    }
    // drain: nothing on peer memory
}
