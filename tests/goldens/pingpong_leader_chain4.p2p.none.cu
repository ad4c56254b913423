// Emitted by the aboleth_b200 Tier-2 specializer.  Program 'pingpong_leader', transport p2p.
#include "aboleth/tier2.cuh"

extern "C" __global__ void pingpong_leader(unsigned long long payload, const unsigned long long * endpoints, const unsigned long long * remote_table, unsigned long long my_flag, long long rounds, long long epoch0, unsigned long long *ab_status) {
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
        const unsigned long long v_r2 = remote_table[2 * (1)] + (0);
        const unsigned v_r2_key = (unsigned)remote_table[2 * (1) + 1];
        (void)v_r2_key;
        const unsigned long long v_l3 = (unsigned long long)((payload + 0)) + (0);
        const unsigned v_l3_key = 0;
        (void)v_l3_key;
        // post_put %t4: carried out at its submission
        const unsigned long long v_r5 = remote_table[2 * (1)] + (1024);
        const unsigned v_r5_key = (unsigned)remote_table[2 * (1) + 1];
        (void)v_r5_key;
        const unsigned long long v_l6 = (unsigned long long)((payload + 1024)) + (0);
        const unsigned v_l6_key = 0;
        (void)v_l6_key;
        // post_put %t7: carried out at its submission
        const unsigned long long v_r8 = remote_table[2 * (1)] + (2048);
        const unsigned v_r8_key = (unsigned)remote_table[2 * (1) + 1];
        (void)v_r8_key;
        const unsigned long long v_l9 = (unsigned long long)((payload + 2048)) + (0);
        const unsigned v_l9_key = 0;
        (void)v_l9_key;
        // post_put %t10: carried out at its submission
        const unsigned long long v_r11 = remote_table[2 * (1)] + (3072);
        const unsigned v_r11_key = (unsigned)remote_table[2 * (1) + 1];
        (void)v_r11_key;
        const unsigned long long v_l12 = (unsigned long long)((payload + 3072)) + (0);
        const unsigned v_l12_key = 0;
        (void)v_l12_key;
        // post_put %t13: carried out at its submission
        const unsigned long long v_r14 = remote_table[2 * (1)] + (4096);
        const unsigned v_r14_key = (unsigned)remote_table[2 * (1) + 1];
        (void)v_r14_key;
        // post_signal %s15: carried out at its submission
        // submit %b0: 5 command(s); peer memory has no queue, nothing to reserve or ring
        t2::put_p2p<128>(v_r2, v_l3, (std::uint32_t)(1024), 256u, false);
        t2::put_p2p<128>(v_r5, v_l6, (std::uint32_t)(1024), 256u, false);
        t2::put_p2p<128>(v_r8, v_l9, (std::uint32_t)(1024), 256u, false);
        t2::put_p2p<128>(v_r11, v_l12, (std::uint32_t)(1024), 256u, false);
        __syncthreads();  // every thread's copy precedes the release; no membar.sys
        if (threadIdx.x == 0) detail::st_release_sys((std::uint64_t *)v_r14, (std::uint64_t)((epoch0 + round + 1)));
        // completion of %b0: program order (vacuous on peer memory)
        t2::wait_signal_cta((unsigned long long)(my_flag), (std::uint64_t)((epoch0 + round + 1)), ab_status, 20480);
    }
}
