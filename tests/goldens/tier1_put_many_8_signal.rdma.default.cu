// Emitted by the aboleth_b200 Tier-2 specializer.  Program 'tier1_put_many_8_signal', transport rdma (served by the host-proxy ring).
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
    // post_put %t4: written into its batch at the submission
    const unsigned long long v_r5 = (unsigned long long)((dst + 1 * stride));
    const unsigned v_r5_key = dst_key;
    (void)v_r5_key;
    const unsigned long long v_l6 = (unsigned long long)((src + 1 * stride)) + (0);
    const unsigned v_l6_key = src_key;
    (void)v_l6_key;
    // post_put %t7: written into its batch at the submission
    const unsigned long long v_r8 = (unsigned long long)((dst + 2 * stride));
    const unsigned v_r8_key = dst_key;
    (void)v_r8_key;
    const unsigned long long v_l9 = (unsigned long long)((src + 2 * stride)) + (0);
    const unsigned v_l9_key = src_key;
    (void)v_l9_key;
    // post_put %t10: written into its batch at the submission
    const unsigned long long v_r11 = (unsigned long long)((dst + 3 * stride));
    const unsigned v_r11_key = dst_key;
    (void)v_r11_key;
    const unsigned long long v_l12 = (unsigned long long)((src + 3 * stride)) + (0);
    const unsigned v_l12_key = src_key;
    (void)v_l12_key;
    // post_put %t13: written into its batch at the submission
    const unsigned long long v_r14 = (unsigned long long)((dst + 4 * stride));
    const unsigned v_r14_key = dst_key;
    (void)v_r14_key;
    const unsigned long long v_l15 = (unsigned long long)((src + 4 * stride)) + (0);
    const unsigned v_l15_key = src_key;
    (void)v_l15_key;
    // post_put %t16: written into its batch at the submission
    const unsigned long long v_r17 = (unsigned long long)((dst + 5 * stride));
    const unsigned v_r17_key = dst_key;
    (void)v_r17_key;
    const unsigned long long v_l18 = (unsigned long long)((src + 5 * stride)) + (0);
    const unsigned v_l18_key = src_key;
    (void)v_l18_key;
    // post_put %t19: written into its batch at the submission
    const unsigned long long v_r20 = (unsigned long long)((dst + 6 * stride));
    const unsigned v_r20_key = dst_key;
    (void)v_r20_key;
    const unsigned long long v_l21 = (unsigned long long)((src + 6 * stride)) + (0);
    const unsigned v_l21_key = src_key;
    (void)v_l21_key;
    // post_put %t22: written into its batch at the submission
    const unsigned long long v_r23 = (unsigned long long)((dst + 7 * stride));
    const unsigned v_r23_key = dst_key;
    (void)v_r23_key;
    const unsigned long long v_l24 = (unsigned long long)((src + 7 * stride)) + (0);
    const unsigned v_l24_key = src_key;
    (void)v_l24_key;
    // post_put %t25: written into its batch at the submission
    const unsigned long long v_r26 = (unsigned long long)(flag);
    const unsigned v_r26_key = flag_key;
    (void)v_r26_key;
    // post_signal %s27: written into its batch at the submission
    std::uint64_t seq_v_b0 = 0;
    if (threadIdx.x == 0) {
        // one reservation, 9 command(s), one release store of ready_sequence
        abi::ProxyCommand cmds[9];
        cmds[0] = abi::ProxyCommand{v_l3, v_r2, (std::uint32_t)(bytes), v_l3_key, v_r2_key, abi::kProxyCommandWrite};
        cmds[1] = abi::ProxyCommand{v_l6, v_r5, (std::uint32_t)(bytes), v_l6_key, v_r5_key, abi::kProxyCommandWrite};
        cmds[2] = abi::ProxyCommand{v_l9, v_r8, (std::uint32_t)(bytes), v_l9_key, v_r8_key, abi::kProxyCommandWrite};
        cmds[3] = abi::ProxyCommand{v_l12, v_r11, (std::uint32_t)(bytes), v_l12_key, v_r11_key, abi::kProxyCommandWrite};
        cmds[4] = abi::ProxyCommand{v_l15, v_r14, (std::uint32_t)(bytes), v_l15_key, v_r14_key, abi::kProxyCommandWrite};
        cmds[5] = abi::ProxyCommand{v_l18, v_r17, (std::uint32_t)(bytes), v_l18_key, v_r17_key, abi::kProxyCommandWrite};
        cmds[6] = abi::ProxyCommand{v_l21, v_r20, (std::uint32_t)(bytes), v_l21_key, v_r20_key, abi::kProxyCommandWrite};
        cmds[7] = abi::ProxyCommand{v_l24, v_r23, (std::uint32_t)(bytes), v_l24_key, v_r23_key, abi::kProxyCommandWrite};
        cmds[8] = abi::ProxyCommand{(unsigned long long)(value), v_r26, 8, 0, v_r26_key, abi::kProxyCommandStrongSignal};
        t2::record(ab_status, proxy::submit(v_e1, cmds, 9, &seq_v_b0), 24577);
    }
    if (threadIdx.x == 0) t2::record(ab_status, proxy::poll(v_e1, seq_v_b0), 24833);
}
