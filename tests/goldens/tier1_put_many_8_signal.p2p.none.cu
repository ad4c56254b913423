// Emitted by the aboleth_b200 Tier-2 specializer.  Program 'tier1_put_many_8_signal', transport p2p.
#include "aboleth/tier2.cuh"

extern "C" __global__ void tier1_put_many_8_signal(const unsigned long long * endpoints, int peer, unsigned long long dst, int dst_key, unsigned long long src, int src_key, int bytes, int stride, unsigned long long flag, int flag_key, unsigned long long value, unsigned long long *ab_status) {
    using namespace aboleth;
    const long long pid = blockIdx.x;
    (void)pid;
    constexpr long long RANK = 0;
    (void)RANK;
    constexpr long long WORLD = 2;
    (void)WORLD;
    const unsigned long long v_e1 = endpoints[peer] & ~7ull;
    (void)v_e1;
    const unsigned long long v_r2 = (unsigned long long)((dst + 0 * stride));
    const unsigned v_r2_key = dst_key;
    (void)v_r2_key;
    const unsigned long long v_l3 = (unsigned long long)((src + 0 * stride)) + (0);
    const unsigned v_l3_key = src_key;
    (void)v_l3_key;
    // post_put %t4: carried out at its submission
    const unsigned long long v_r5 = (unsigned long long)((dst + 1 * stride));
    const unsigned v_r5_key = dst_key;
    (void)v_r5_key;
    const unsigned long long v_l6 = (unsigned long long)((src + 1 * stride)) + (0);
    const unsigned v_l6_key = src_key;
    (void)v_l6_key;
    // post_put %t7: carried out at its submission
    const unsigned long long v_r8 = (unsigned long long)((dst + 2 * stride));
    const unsigned v_r8_key = dst_key;
    (void)v_r8_key;
    const unsigned long long v_l9 = (unsigned long long)((src + 2 * stride)) + (0);
    const unsigned v_l9_key = src_key;
    (void)v_l9_key;
    // post_put %t10: carried out at its submission
    const unsigned long long v_r11 = (unsigned long long)((dst + 3 * stride));
    const unsigned v_r11_key = dst_key;
    (void)v_r11_key;
    const unsigned long long v_l12 = (unsigned long long)((src + 3 * stride)) + (0);
    const unsigned v_l12_key = src_key;
    (void)v_l12_key;
    // post_put %t13: carried out at its submission
    const unsigned long long v_r14 = (unsigned long long)((dst + 4 * stride));
    const unsigned v_r14_key = dst_key;
    (void)v_r14_key;
    const unsigned long long v_l15 = (unsigned long long)((src + 4 * stride)) + (0);
    const unsigned v_l15_key = src_key;
    (void)v_l15_key;
    // post_put %t16: carried out at its submission
    const unsigned long long v_r17 = (unsigned long long)((dst + 5 * stride));
    const unsigned v_r17_key = dst_key;
    (void)v_r17_key;
    const unsigned long long v_l18 = (unsigned long long)((src + 5 * stride)) + (0);
    const unsigned v_l18_key = src_key;
    (void)v_l18_key;
    // post_put %t19: carried out at its submission
    const unsigned long long v_r20 = (unsigned long long)((dst + 6 * stride));
    const unsigned v_r20_key = dst_key;
    (void)v_r20_key;
    const unsigned long long v_l21 = (unsigned long long)((src + 6 * stride)) + (0);
    const unsigned v_l21_key = src_key;
    (void)v_l21_key;
    // post_put %t22: carried out at its submission
    const unsigned long long v_r23 = (unsigned long long)((dst + 7 * stride));
    const unsigned v_r23_key = dst_key;
    (void)v_r23_key;
    const unsigned long long v_l24 = (unsigned long long)((src + 7 * stride)) + (0);
    const unsigned v_l24_key = src_key;
    (void)v_l24_key;
    // post_put %t25: carried out at its submission
    const unsigned long long v_r26 = (unsigned long long)(flag);
    const unsigned v_r26_key = flag_key;
    (void)v_r26_key;
    // post_signal %s27: carried out at its submission
    // submit %b0: 9 command(s); peer memory has no queue, nothing to reserve or ring
    t2::put_p2p<2048>(v_r2, v_l3, (std::uint32_t)(bytes), 256u, false);
    t2::put_p2p<2048>(v_r5, v_l6, (std::uint32_t)(bytes), 256u, false);
    t2::put_p2p<2048>(v_r8, v_l9, (std::uint32_t)(bytes), 256u, false);
    t2::put_p2p<2048>(v_r11, v_l12, (std::uint32_t)(bytes), 256u, false);
    t2::put_p2p<2048>(v_r14, v_l15, (std::uint32_t)(bytes), 256u, false);
    t2::put_p2p<2048>(v_r17, v_l18, (std::uint32_t)(bytes), 256u, false);
    t2::put_p2p<2048>(v_r20, v_l21, (std::uint32_t)(bytes), 256u, false);
    t2::put_p2p<2048>(v_r23, v_l24, (std::uint32_t)(bytes), 256u, false);
    __syncthreads();  // every thread's copy precedes the release; no membar.sys
    if (threadIdx.x == 0) detail::st_release_sys((std::uint64_t *)v_r26, (std::uint64_t)(value));
    // completion of %b0: program order (vacuous on peer memory)
}
