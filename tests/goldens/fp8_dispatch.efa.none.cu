// Emitted by the aboleth_b200 Tier-2 specializer.  Program 'fp8_dispatch', transport efa (served by the host-proxy ring).
#include "aboleth/tier2.cuh"

extern "C" __global__ void fp8_dispatch(unsigned long long tokens, unsigned long long staging, const unsigned long long * endpoints, const unsigned long long * slot_table, const unsigned long long * count_table, const unsigned long long * flag_table, unsigned long long live, long long iteration, unsigned long long *ab_status) {
    using namespace aboleth;
    const long long pid = blockIdx.x;
    (void)pid;
    constexpr long long RANK = 0;
    (void)RANK;
    constexpr long long WORLD = 2;
    (void)WORLD;
    const long long peer = pid;
    const unsigned long long v_e1 = endpoints[peer] & ~7ull;
    (void)v_e1;
    quantize_tile(tokens, staging, peer, 0);
    // tensor_store staging
    const unsigned long long v_r2 = slot_table[2 * (peer)] + (((iteration % 2)*8448 + 0));
    const unsigned v_r2_key = (unsigned)slot_table[2 * (peer) + 1];
    (void)v_r2_key;
    const unsigned long long v_l3 = (unsigned long long)((staging + (peer*4 + 0)*2112)) + (0);
    const unsigned v_l3_key = 0;
    (void)v_l3_key;
    // post_put %t4: written into its batch at the submission
    quantize_tile(tokens, staging, peer, 1);
    // tensor_store staging
    const unsigned long long v_r5 = slot_table[2 * (peer)] + (((iteration % 2)*8448 + 2112));
    const unsigned v_r5_key = (unsigned)slot_table[2 * (peer) + 1];
    (void)v_r5_key;
    const unsigned long long v_l6 = (unsigned long long)((staging + (peer*4 + 1)*2112)) + (0);
    const unsigned v_l6_key = 0;
    (void)v_l6_key;
    // post_put %t7: written into its batch at the submission
    quantize_tile(tokens, staging, peer, 2);
    // tensor_store staging
    const unsigned long long v_r8 = slot_table[2 * (peer)] + (((iteration % 2)*8448 + 4224));
    const unsigned v_r8_key = (unsigned)slot_table[2 * (peer) + 1];
    (void)v_r8_key;
    const unsigned long long v_l9 = (unsigned long long)((staging + (peer*4 + 2)*2112)) + (0);
    const unsigned v_l9_key = 0;
    (void)v_l9_key;
    // post_put %t10: written into its batch at the submission
    quantize_tile(tokens, staging, peer, 3);
    // tensor_store staging
    const unsigned long long v_r11 = slot_table[2 * (peer)] + (((iteration % 2)*8448 + 6336));
    const unsigned v_r11_key = (unsigned)slot_table[2 * (peer) + 1];
    (void)v_r11_key;
    const unsigned long long v_l12 = (unsigned long long)((staging + (peer*4 + 3)*2112)) + (0);
    const unsigned v_l12_key = 0;
    (void)v_l12_key;
    // post_put %t13: written into its batch at the submission
    const unsigned long long v_r14 = count_table[2 * (peer)] + (RANK*8);
    const unsigned v_r14_key = (unsigned)count_table[2 * (peer) + 1];
    (void)v_r14_key;
    // post_inline %t15: written into its batch at the submission
    const unsigned long long v_r16 = flag_table[2 * (peer)] + (RANK*8);
    const unsigned v_r16_key = (unsigned)flag_table[2 * (peer) + 1];
    (void)v_r16_key;
    // post_signal %s17: written into its batch at the submission
    __syncthreads();  // producer barrier
    std::uint64_t seq_v_b0 = 0;
    if (threadIdx.x == 0) {
        // one reservation, 6 command(s), one release store of ready_sequence
        abi::ProxyCommand cmds[6];
        cmds[0] = ((((const int*)live)[peer*4 + 0])) ? abi::ProxyCommand{v_l3, v_r2, (std::uint32_t)(2112), v_l3_key, v_r2_key, abi::kProxyCommandWrite} : abi::ProxyCommand{0, 0, 0, 0, 0, abi::kProxyCommandNop};
        cmds[1] = ((((const int*)live)[peer*4 + 1])) ? abi::ProxyCommand{v_l6, v_r5, (std::uint32_t)(2112), v_l6_key, v_r5_key, abi::kProxyCommandWrite} : abi::ProxyCommand{0, 0, 0, 0, 0, abi::kProxyCommandNop};
        cmds[2] = ((((const int*)live)[peer*4 + 2])) ? abi::ProxyCommand{v_l9, v_r8, (std::uint32_t)(2112), v_l9_key, v_r8_key, abi::kProxyCommandWrite} : abi::ProxyCommand{0, 0, 0, 0, 0, abi::kProxyCommandNop};
        cmds[3] = ((((const int*)live)[peer*4 + 3])) ? abi::ProxyCommand{v_l12, v_r11, (std::uint32_t)(2112), v_l12_key, v_r11_key, abi::kProxyCommandWrite} : abi::ProxyCommand{0, 0, 0, 0, 0, abi::kProxyCommandNop};
        cmds[4] = abi::ProxyCommand{(unsigned long long)((((const int*)live)[peer*4])), v_r14, 8, 0, v_r14_key, abi::kProxyCommandWeakSignal};
        cmds[5] = abi::ProxyCommand{(unsigned long long)((iteration + 1)), v_r16, 8, 0, v_r16_key, abi::kProxyCommandStrongSignal};
        t2::record(ab_status, proxy::submit(v_e1, cmds, 6, &seq_v_b0), 24577);
    }
    if (threadIdx.x == 0) t2::record(ab_status, proxy::poll(v_e1, seq_v_b0), 24833);
}
