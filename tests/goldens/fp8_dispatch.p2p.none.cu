// Emitted by the aboleth_b200 Tier-2 specializer.  Program 'fp8_dispatch', transport p2p.
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
    // post_put %t4: carried out at its submission
    quantize_tile(tokens, staging, peer, 1);
    // tensor_store staging
    const unsigned long long v_r5 = slot_table[2 * (peer)] + (((iteration % 2)*8448 + 2112));
    const unsigned v_r5_key = (unsigned)slot_table[2 * (peer) + 1];
    (void)v_r5_key;
    const unsigned long long v_l6 = (unsigned long long)((staging + (peer*4 + 1)*2112)) + (0);
    const unsigned v_l6_key = 0;
    (void)v_l6_key;
    // post_put %t7: carried out at its submission
    quantize_tile(tokens, staging, peer, 2);
    // tensor_store staging
    const unsigned long long v_r8 = slot_table[2 * (peer)] + (((iteration % 2)*8448 + 4224));
    const unsigned v_r8_key = (unsigned)slot_table[2 * (peer) + 1];
    (void)v_r8_key;
    const unsigned long long v_l9 = (unsigned long long)((staging + (peer*4 + 2)*2112)) + (0);
    const unsigned v_l9_key = 0;
    (void)v_l9_key;
    // post_put %t10: carried out at its submission
    quantize_tile(tokens, staging, peer, 3);
    // tensor_store staging
    const unsigned long long v_r11 = slot_table[2 * (peer)] + (((iteration % 2)*8448 + 6336));
    const unsigned v_r11_key = (unsigned)slot_table[2 * (peer) + 1];
    (void)v_r11_key;
    const unsigned long long v_l12 = (unsigned long long)((staging + (peer*4 + 3)*2112)) + (0);
    const unsigned v_l12_key = 0;
    (void)v_l12_key;
    // post_put %t13: carried out at its submission
    const unsigned long long v_r14 = count_table[2 * (peer)] + (RANK*8);
    const unsigned v_r14_key = (unsigned)count_table[2 * (peer) + 1];
    (void)v_r14_key;
    // post_inline %t15: carried out at its submission
    const unsigned long long v_r16 = flag_table[2 * (peer)] + (RANK*8);
    const unsigned v_r16_key = (unsigned)flag_table[2 * (peer) + 1];
    (void)v_r16_key;
    // post_signal %s17: carried out at its submission
    // submit %b0: 6 command(s); peer memory has no queue, nothing to reserve or ring
    __syncthreads();  // producer barrier: a source was written by other threads
    if ((((const int*)live)[peer*4 + 0])) {
        t2::put_p2p<512>(v_r2, v_l3, (std::uint32_t)(2112), 256u, false);
    }
    if ((((const int*)live)[peer*4 + 1])) {
        t2::put_p2p<512>(v_r5, v_l6, (std::uint32_t)(2112), 256u, false);
    }
    if ((((const int*)live)[peer*4 + 2])) {
        t2::put_p2p<512>(v_r8, v_l9, (std::uint32_t)(2112), 256u, false);
    }
    if ((((const int*)live)[peer*4 + 3])) {
        t2::put_p2p<512>(v_r11, v_l12, (std::uint32_t)(2112), 256u, false);
    }
    if (threadIdx.x == 0) {
        t2::store_inline<std::uint64_t>(v_r14 + 0, (unsigned long long)((((const int*)live)[peer*4])));
    }
    __syncthreads();  // every thread's copy precedes the release; no membar.sys
    if (threadIdx.x == 0) detail::st_release_sys((std::uint64_t *)v_r16, (std::uint64_t)((iteration + 1)));
    // completion of %b0: program order (vacuous on peer memory)
}
