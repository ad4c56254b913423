#!/usr/bin/env python
"""Block-scaled e4m3 GEMM on the fp8 tensor path, three ways.

    python examples/block_scaled_gemm.py [--m 4096 --n 4096 --k 4096]

Activations carry one power-of-two scale per row and 128 columns (``quant_fp8(round_scale=True)``),
weights one per 128 x 128 block.  (1) ``gemm_e4m3_block_scaled`` packs the scales and multiplies with
``tcgen05.mma.kind::mxf8f6f4.block_scale``; (2) the same with the weight's scales packed once, as a
layer would keep them; (3) ``path="expand"``: dequantise to bf16, bf16 GEMM.  All three are compared
with an fp32 product of the dequantised operands.
"""
import argparse
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--m", type=int, default=2048)
    ap.add_argument("--n", type=int, default=2048)
    ap.add_argument("--k", type=int, default=2048)
    args = ap.parse_args()

    import torch

    from aboleth_b200.ops import (check_gemm_status, gemm_e4m3_block_scaled, gemm_e4m3_mx, pack_scales_mx,
                                  quant_fp8)

    torch.cuda.set_device(0)
    m, n, k = args.m, args.n, args.k
    g = torch.Generator(device="cuda").manual_seed(0)
    x = torch.randn(m, k, generator=g, device="cuda").to(torch.bfloat16)
    w = torch.randn(n, k, generator=g, device="cuda") * 0.05
    x_q, x_s = quant_fp8(x, round_scale=True)                       # [m, k] e4m3, [m, k / 128] fp32
    blocks = w.view(n // 128, 128, k // 128, 128)
    w_s = torch.exp2(torch.ceil(torch.log2(blocks.abs().amax(dim=(1, 3)).clamp_min(1e-10) / 448.0)))
    w_q = (blocks / w_s[:, None, :, None]).reshape(n, k).to(torch.float8_e4m3fn)

    want = (x_q.float() * x_s.repeat_interleave(128, 1)) @ \
           (w_q.float() * w_s.repeat_interleave(128, 0).repeat_interleave(128, 1)).t()

    def timed(fn):
        fn()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(10):
            out = fn()
        stop.record()
        torch.cuda.synchronize()
        return out, start.elapsed_time(stop) / 10 * 1e3

    w_packed = pack_scales_mx(w_s, n, k, weight=True)               # kept with the weight
    results = {
        "block-scaled MMA, scales packed per call": timed(lambda: gemm_e4m3_block_scaled(x_q, x_s, w_q, w_s)),
        "block-scaled MMA, weight scales packed once": timed(
            lambda: gemm_e4m3_mx(x_q, pack_scales_mx(x_s, m, k, weight=False), w_q, w_packed)),
        "expanded to bf16, bf16 GEMM": timed(lambda: gemm_e4m3_block_scaled(x_q, x_s, w_q, w_s, path="expand")),
    }
    check_gemm_status("cuda")
    ok = True
    for name, (out, us) in results.items():
        err = ((out.float() - want).norm() / want.norm()).item()
        ok = ok and err < 5e-3
        print(f"{name:46s} {us:8.1f} us  {2.0 * m * n * k / us / 1e6:7.0f} TFLOP/s  relative error {err:.2e}")
    return 0 if ok else 1


if __name__ == "__main__":
    raise SystemExit(main())
