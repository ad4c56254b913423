// Block-scaled e4m3 -> bf16: out[r, c] = q[r, c] * scales[r / row_block, c / col_block].
//
// The two operand layouts of a block-scaled fp8 GEMM are both covered: activations
// carry one fp32 scale per row and 128 columns (row_block 1, col_block 128, what the
// dispatch kernel and ab_quant_fp8 produce), weights one per 128 x 128 block.  With
// power-of-two scales the product is exact in bf16 (e4m3 has four significant bits,
// bf16 eight), so a bf16 tensor-core GEMM over the result reproduces the block-scaled
// GEMM with fp32 accumulation; with arbitrary fp32 scales each element is rounded once
// to bf16.  The reference has no GEMM at all; this is an operation of this build.
//
// Memory-bound: each thread turns one 16-byte vector of e4m3 into two 16-byte vectors
// of bf16; reads use the streaming path, writes are plain (the GEMM reads them next).
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>

#include "common.cuh"

namespace {

constexpr int kThreads = 256;

__device__ __forceinline__ std::uint32_t scaled_pair(std::uint16_t two_fp8, float scale) {
    const __half2_raw h = __nv_cvt_fp8x2_to_halfraw2(static_cast<__nv_fp8x2_storage_t>(two_fp8), __NV_E4M3);
    const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&h));
    const __nv_bfloat162 b = __floats2bfloat162_rn(f.x * scale, f.y * scale);
    return *reinterpret_cast<const std::uint32_t *>(&b);
}

__global__ void __launch_bounds__(kThreads) dequant_block_scaled_kernel(
    const std::uint8_t *q, const float *scales, std::uint8_t *out, int rows, int cols, int row_block,
    int col_block, long long q_stride, long long out_stride, int scale_stride) {
    const int chunks = cols / 16;  // 16 e4m3 values per thread and step
    const long long total = static_cast<long long>(rows) * chunks;
    for (long long i = static_cast<long long>(blockIdx.x) * kThreads + threadIdx.x; i < total;
         i += static_cast<long long>(gridDim.x) * kThreads) {
        const int r = static_cast<int>(i / chunks);
        const int c = static_cast<int>(i % chunks) * 16;
        const float scale = __ldg(scales + static_cast<long long>(r / row_block) * scale_stride + c / col_block);
        const uint4 v = aboleth::detail::ld_stream16(q + r * q_stride + c);
        uint4 lo, hi;
        lo.x = scaled_pair(static_cast<std::uint16_t>(v.x & 0xffff), scale);
        lo.y = scaled_pair(static_cast<std::uint16_t>(v.x >> 16), scale);
        lo.z = scaled_pair(static_cast<std::uint16_t>(v.y & 0xffff), scale);
        lo.w = scaled_pair(static_cast<std::uint16_t>(v.y >> 16), scale);
        hi.x = scaled_pair(static_cast<std::uint16_t>(v.z & 0xffff), scale);
        hi.y = scaled_pair(static_cast<std::uint16_t>(v.z >> 16), scale);
        hi.z = scaled_pair(static_cast<std::uint16_t>(v.w & 0xffff), scale);
        hi.w = scaled_pair(static_cast<std::uint16_t>(v.w >> 16), scale);
        uint4 *dst = reinterpret_cast<uint4 *>(out + (r * out_stride + c) * 2);
        dst[0] = lo;
        dst[1] = hi;
    }
}

}  // namespace

// q: e4m3 [rows, cols] with row stride q_stride (elements); scales: fp32
// [ceil(rows / row_block), cols / col_block] with row stride scale_stride; out: bf16
// [rows, cols] with row stride out_stride (elements).  cols and col_block are multiples
// of 16, strides keep rows 16-byte aligned.  Returns -1 on arguments outside that.
AB_EXPORT int ab_dequant_block_scaled(const void *q, const float *scales, void *out, int rows, int cols,
                                      int row_block, int col_block, long long q_stride,
                                      long long out_stride, int scale_stride, cudaStream_t stream) {
    if (rows < 1 || cols < 16 || cols % 16 || row_block < 1 || col_block < 16 || col_block % 16 ||
        q_stride % 16 || out_stride % 8 || q_stride < cols || out_stride < cols ||
        scale_stride < (cols + col_block - 1) / col_block ||
        reinterpret_cast<std::uintptr_t>(q) % 16 || reinterpret_cast<std::uintptr_t>(out) % 16)
        return -1;
    const long long work = static_cast<long long>(rows) * (cols / 16);
    long long blocks = (work + kThreads - 1) / kThreads;
    if (blocks > 148 * 16)
        blocks = 148 * 16;
    dequant_block_scaled_kernel<<<static_cast<int>(blocks), kThreads, 0, stream>>>(
        static_cast<const std::uint8_t *>(q), scales, static_cast<std::uint8_t *>(out), rows, cols, row_block,
        col_block, q_stride, out_stride, scale_stride);
    return ab::launch_result("dequant_block_scaled");
}
