// Device helpers shared by the MoE kernels: router softmax/top-k in one warp,
// 1 x group block-scaled e4m3 quantisation, and the record geometry.
//
// Record layout (one record per (token, destination rank); reference:
// python/aboleth/moe/compiled_plan.py:101-107, python/aboleth/moe/kernels.py:98-143):
//   payload row  : hidden x {bf16 | e4m3}
//   metadata row : int32 [token, n_selected, expert_id x k, weight_bits x k, scale_bits x cols]
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp8.h>

#include "common.cuh"

namespace ab::moe {

constexpr int kMaxTopK = 16;
constexpr int kMaxWorld = 32;
constexpr int kMaxExpertsPerLane = 16;  // experts <= 512
constexpr float kFp8Max = 448.0f;

__device__ __forceinline__ float bf16_lo(std::uint32_t v) { return __uint_as_float(v << 16); }
__device__ __forceinline__ float bf16_hi(std::uint32_t v) { return __uint_as_float(v & 0xffff0000u); }

__device__ __forceinline__ std::uint32_t pack_bf16x2(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<std::uint32_t *>(&v);
}

// scale = max(amax, floor) / 448, optionally rounded UP to a power of two.
__device__ __forceinline__ float quant_scale(float amax, float floor_, int round_pow2) {
    float scale = fmaxf(amax, floor_) / kFp8Max;
    if (round_pow2) {
        std::uint32_t bits = __float_as_uint(scale);
        if (bits & 0x007fffffu)
            bits = (bits & 0xff800000u) + 0x00800000u;
        scale = __uint_as_float(bits);
    }
    return scale;
}

// x / scale.  The default is the hardware's approximate division (about 2 ulp,
// far below an e4m3 quantum; a value that sits on a rounding tie may land on
// the other neighbour than IEEE division would pick).  Define
// ABOLETH_EXACT_QUANT_DIV for bit-exact IEEE division at several times the cost.
__device__ __forceinline__ float quant_div(float x, float scale) {
#ifdef ABOLETH_EXACT_QUANT_DIV
    return x / scale;
#else
    return __fdividef(x, scale);
#endif
}

// Four values times the reciprocal scale `inv` -> four e4m3 codes.  The conversion saturates at
// +-448 by itself, so no clamp is spent here (a NaN input stays NaN).
__device__ __forceinline__ std::uint32_t fp8x4(float a, float b, float c, float d, float inv) {
#ifdef ABOLETH_EXACT_QUANT_DIV
    const float scale = inv;  // the caller passes the scale itself
    a = quant_div(a, scale); b = quant_div(b, scale); c = quant_div(c, scale); d = quant_div(d, scale);
#else
    a *= inv; b *= inv; c *= inv; d *= inv;
#endif
    const std::uint32_t p0 = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
    const std::uint32_t p1 = __nv_cvt_float2_to_fp8x2(make_float2(c, d), __NV_SATFINITE, __NV_E4M3);
    return p0 | (p1 << 16);
}

// Sixteen bf16 values (two 16-byte vectors) -> absolute maximum.  Signs are masked off two values
// at a time and the packed maximum unit compares them; one conversion at the end.
__device__ __forceinline__ float amax16(const uint4 &a, const uint4 &b) {
    const std::uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
    __nv_bfloat162 m;
    *reinterpret_cast<std::uint32_t *>(&m) = w[0] & 0x7fff7fffu;
#pragma unroll
    for (int i = 1; i < 8; ++i) {
        __nv_bfloat162 v;
        *reinterpret_cast<std::uint32_t *>(&v) = w[i] & 0x7fff7fffu;
        m = __hmax2(m, v);
    }
    const std::uint32_t bits = *reinterpret_cast<std::uint32_t *>(&m);
    return fmaxf(bf16_lo(bits), bf16_hi(bits));
}

// Sixteen bf16 values -> sixteen e4m3 codes at `scale`.  The default multiplies by the correctly
// rounded reciprocal of the scale (exact for power-of-two scales, within 1.5 ulp of the division
// otherwise: far below an e4m3 quantum, so only a value that sits on a rounding tie can land on the
// other neighbouring code).  ABOLETH_EXACT_QUANT_DIV divides instead.
__device__ __forceinline__ uint4 quant16(const uint4 &a, const uint4 &b, float scale) {
#ifdef ABOLETH_EXACT_QUANT_DIV
    const float inv = scale;
#else
    const float inv = __frcp_rn(scale);
#endif
    uint4 q;
    q.x = fp8x4(bf16_lo(a.x), bf16_hi(a.x), bf16_lo(a.y), bf16_hi(a.y), inv);
    q.y = fp8x4(bf16_lo(a.z), bf16_hi(a.z), bf16_lo(a.w), bf16_hi(a.w), inv);
    q.z = fp8x4(bf16_lo(b.x), bf16_hi(b.x), bf16_lo(b.y), bf16_hi(b.y), inv);
    q.w = fp8x4(bf16_lo(b.z), bf16_hi(b.z), bf16_lo(b.w), bf16_hi(b.w), inv);
    return q;
}

// Reduce a maximum over the `width` consecutive lanes (power of two <= 32)
// that share one quantisation group.
__device__ __forceinline__ float group_max(float v, int width) {
    for (int off = width >> 1; off > 0; off >>= 1)
        v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, off));
    return v;
}

// One warp: softmax over `experts` logits and the `top_k` largest, ties to
// the lower index.  Lane l holds experts l, l+32, ...  On return lane j < top_k
// holds (id, weight) of the j-th choice.  `renormalize` divides the selected
// probabilities by their sum.
template <int PER_LANE>
__device__ __forceinline__ void warp_softmax_topk_n(const float *logits, int experts, int top_k,
                                                    int renormalize, int &out_id, float &out_w) {
    constexpr int kMaxExpertsPerLane = PER_LANE;
    const int lane = threadIdx.x & 31;
    float v[kMaxExpertsPerLane];
    float mx = -INFINITY;
#pragma unroll
    for (int i = 0; i < kMaxExpertsPerLane; ++i) {
        const int e = lane + 32 * i;
        v[i] = e < experts ? logits[e] : -INFINITY;
        mx = fmaxf(mx, v[i]);
    }
    for (int off = 16; off > 0; off >>= 1)
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < kMaxExpertsPerLane; ++i)
        sum += (lane + 32 * i) < experts ? __expf(v[i] - mx) : 0.f;
    for (int off = 16; off > 0; off >>= 1)
        sum += __shfl_xor_sync(0xffffffffu, sum, off);

    out_id = -1;
    out_w = 0.f;
    float picked_sum = 0.f;
    for (int j = 0; j < top_k; ++j) {
        float best = -INFINITY;
        int best_e = 0x7fffffff;
#pragma unroll
        for (int i = 0; i < kMaxExpertsPerLane; ++i) {
            const int e = lane + 32 * i;
            if (e < experts && v[i] > best) {
                best = v[i];
                best_e = e;
            }
        }
        // Warp-wide argmax in two reductions: the largest value (as an order-preserving integer),
        // then the lowest expert index among the lanes that hold it.
        const std::uint32_t raw = __float_as_uint(best);
        const std::uint32_t key = raw ^ ((raw >> 31) ? 0xffffffffu : 0x80000000u);
        const std::uint32_t top = __reduce_max_sync(0xffffffffu, key);
        best_e = static_cast<int>(__reduce_min_sync(
            0xffffffffu, key == top ? static_cast<unsigned>(best_e) : 0x7fffffffu));
        const std::uint32_t back = top ^ ((top >> 31) ? 0x80000000u : 0xffffffffu);
        best = __uint_as_float(back);
        const float w = __expf(best - mx) / sum;
        picked_sum += w;
        if (lane == j) {
            out_id = best_e;
            out_w = w;
        }
        if ((best_e & 31) == lane) {
#pragma unroll
            for (int i = 0; i < kMaxExpertsPerLane; ++i)
                if (i == (best_e >> 5))
                    v[i] = -INFINITY;
        }
    }
    if (renormalize && picked_sum > 0.f)
        out_w /= picked_sum;
}

__device__ __forceinline__ void warp_softmax_topk(const float *logits, int experts, int top_k,
                                                  int renormalize, int &out_id, float &out_w) {
    if (experts <= 128)
        warp_softmax_topk_n<4>(logits, experts, top_k, renormalize, out_id, out_w);
    else if (experts <= 256)
        warp_softmax_topk_n<8>(logits, experts, top_k, renormalize, out_id, out_w);
    else
        warp_softmax_topk_n<kMaxExpertsPerLane>(logits, experts, top_k, renormalize, out_id, out_w);
}

}  // namespace ab::moe
