// Emitted by the aboleth_b200 Tier-2 specializer.  Program 'stream_pipelined', transport p2p.
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
    for (long long round = 0; round < rounds; ++round) {
        const unsigned long long v_l2 = (unsigned long long)((payload + 0)) + (0);
        const unsigned v_l2_key = 0;
        (void)v_l2_key;
        const unsigned long long v_r3 = remote_table[2 * (1)] + (0);
        const unsigned v_r3_key = (unsigned)remote_table[2 * (1) + 1];
        (void)v_r3_key;
        // post_put %t4: carried out at its submission
        const unsigned long long v_r5 = remote_table[2 * (1)] + (1024);
        const unsigned v_r5_key = (unsigned)remote_table[2 * (1) + 1];
        (void)v_r5_key;
        // post_signal %s6: carried out at its submission
        // submit %b0: 2 command(s); peer memory has no queue, nothing to reserve or ring
        t2::put_p2p<32>(v_r3, v_l2, (std::uint32_t)(256), 256u, false);
        __syncthreads();  // every thread's copy precedes the release; no membar.sys
        if (threadIdx.x == 0) detail::st_release_sys((std::uint64_t *)v_r5, (std::uint64_t)((round + 1)));
        const unsigned long long v_l7 = (unsigned long long)((payload + 256)) + (0);
        const unsigned v_l7_key = 0;
        (void)v_l7_key;
        const unsigned long long v_r8 = remote_table[2 * (1)] + (256);
        const unsigned v_r8_key = (unsigned)remote_table[2 * (1) + 1];
        (void)v_r8_key;
        // post_put %t9: carried out at its submission
        const unsigned long long v_r10 = remote_table[2 * (1)] + (1032);
        const unsigned v_r10_key = (unsigned)remote_table[2 * (1) + 1];
        (void)v_r10_key;
        // post_signal %s11: carried out at its submission
        // submit %b1: 2 command(s); peer memory has no queue, nothing to reserve or ring
        t2::put_p2p<32>(v_r8, v_l7, (std::uint32_t)(256), 256u, false);
        __syncthreads();  // every thread's copy precedes the release; no membar.sys
        if (threadIdx.x == 0) detail::st_release_sys((std::uint64_t *)v_r10, (std::uint64_t)((round + 1)));
        const unsigned long long v_l12 = (unsigned long long)((payload + 512)) + (0);
        const unsigned v_l12_key = 0;
        (void)v_l12_key;
        const unsigned long long v_r13 = remote_table[2 * (1)] + (512);
        const unsigned v_r13_key = (unsigned)remote_table[2 * (1) + 1];
        (void)v_r13_key;
        // post_put %t14: carried out at its submission
        const unsigned long long v_r15 = remote_table[2 * (1)] + (1040);
        const unsigned v_r15_key = (unsigned)remote_table[2 * (1) + 1];
        (void)v_r15_key;
        // post_signal %s16: carried out at its submission
        // submit %b2: 2 command(s); peer memory has no queue, nothing to reserve or ring
        t2::put_p2p<32>(v_r13, v_l12, (std::uint32_t)(256), 256u, false);
        __syncthreads();  // every thread's copy precedes the release; no membar.sys
        if (threadIdx.x == 0) detail::st_release_sys((std::uint64_t *)v_r15, (std::uint64_t)((round + 1)));
        const unsigned long long v_l17 = (unsigned long long)((payload + 768)) + (0);
        const unsigned v_l17_key = 0;
        (void)v_l17_key;
        const unsigned long long v_r18 = remote_table[2 * (1)] + (768);
        const unsigned v_r18_key = (unsigned)remote_table[2 * (1) + 1];
        (void)v_r18_key;
        // post_put %t19: carried out at its submission
        const unsigned long long v_r20 = remote_table[2 * (1)] + (1048);
        const unsigned v_r20_key = (unsigned)remote_table[2 * (1) + 1];
        (void)v_r20_key;
        // post_signal %s21: carried out at its submission
        // submit %b3: 2 command(s); peer memory has no queue, nothing to reserve or ring
        t2::put_p2p<32>(v_r18, v_l17, (std::uint32_t)(256), 256u, false);
        __syncthreads();  // every thread's copy precedes the release; no membar.sys
        if (threadIdx.x == 0) detail::st_release_sys((std::uint64_t *)v_r20, (std::uint64_t)((round + 1)));
        // completion of %b0: program order (vacuous on peer memory)
        // completion of %b1: program order (vacuous on peer memory)
        // completion of %b2: program order (vacuous on peer memory)
        // completion of %b3: program order (vacuous on peer memory)
    }
    // drain: nothing on peer memory
}
