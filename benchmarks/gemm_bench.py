#!/usr/bin/env python
"""bf16 GEMM on one GPU: the tcgen05 kernels of this package against cuBLAS (torch.matmul).

    python benchmarks/gemm_bench.py                      # dense C = A @ B^T over the TP / FFN shapes
    python benchmarks/gemm_bench.py --shape 4096 4096 4096 --steps 3 --no-library   # small case for a profiler
    python benchmarks/gemm_bench.py --grouped            # grouped (per-expert) GEMM, Mixtral expert shapes
    python benchmarks/gemm_bench.py --fp8                # e4m3 operands, against torch._scaled_mm (cuBLASLt)
    python benchmarks/gemm_bench.py --block-scaled       # e4m3 with 1x128 / 128x128 scales (expansion + bf16 GEMM)

Each timed launch is preceded by an L2 flush; times are medians of CUDA-event brackets.
Fractions are of the measured cuBLAS bf16 burst throughput recorded for this pool.
"""
import argparse

from common import emit, load_measured_peaks, start_clock_sampler

import torch

from aboleth_b200.bench_support import L2Flusher
from aboleth_b200.ops import check_gemm_status, gemm_bf16, grouped_gemm_bf16

DENSE = [(8192, 3584, 8192), (8192, 8192, 3584), (8192, 28672, 8192), (8192, 8192, 8192), (4096, 4096, 4096)]


def timed(fn, flush, steps):
    ts = []
    for i in range(steps + 3):
        flush()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda._sleep(200000)  # the host gets ahead, so launch latency stays outside the bracket
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        if i >= 3:
            ts.append(a.elapsed_time(b))
    ts.sort()
    return ts[len(ts) // 2]


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--shape", type=int, nargs=3, metavar=("M", "N", "K"), default=None)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--grouped", action="store_true")
    ap.add_argument("--fp8", action="store_true", help="e4m3 operands (per-tensor scale), against torch._scaled_mm")
    ap.add_argument("--block-scaled", action="store_true",
                    help="e4m3 operands with 1x128 / 128x128 fp32 scales: the bf16 expansion (against the "
                         "measured copy bandwidth) and the whole block-scaled GEMM")
    ap.add_argument("--no-library", action="store_true", help="skip the cuBLAS arm (profiler runs)")
    ap.add_argument("--out", default=None)
    args = ap.parse_args()
    torch.cuda.set_device(0)
    start_clock_sampler(0)
    flush = L2Flusher("cuda")
    peak = load_measured_peaks().get("bf16_tflops", 1590.0)
    rows = []
    if args.grouped:
        experts, n, k = 8, 28672, 4096
        for per_expert in (512, 2048, 8192):
            total = experts * per_expert
            x = torch.randn(total, k, device="cuda").to(torch.bfloat16)
            w = (torch.randn(experts, n, k, device="cuda") * 0.02).to(torch.bfloat16)
            counts = torch.full((experts,), per_expert, dtype=torch.int32, device="cuda")
            offsets = (torch.arange(experts, device="cuda", dtype=torch.int32) * per_expert).contiguous()
            y = torch.empty(total, n, dtype=torch.bfloat16, device="cuda")
            ms = timed(lambda: grouped_gemm_bf16(x, w, counts, offsets, y), flush, args.steps)
            check_gemm_status("cuda")
            flops = 2.0 * total * n * k
            row = {"experts": experts, "rows_per_expert": per_expert, "n": n, "k": k, "ours_us": ms * 1e3,
                   "ours_tflops": flops / ms / 1e9, "ours_frac_of_measured": flops / ms / 1e9 / peak}
            if not args.no_library:
                def library():
                    for e in range(experts):
                        torch.matmul(x[e * per_expert:(e + 1) * per_expert], w[e].t(),
                                     out=y[e * per_expert:(e + 1) * per_expert])
                ms2 = timed(library, flush, args.steps)
                row.update(cublas_loop_us=ms2 * 1e3, cublas_loop_tflops=flops / ms2 / 1e9)
            rows.append(row)
            del x, w, y
    elif args.block_scaled:
        from aboleth_b200.ops import (dequant_block_scaled, gemm_e4m3_block_scaled, gemm_e4m3_mx, pack_scales_mx,
                                      quant_fp8)

        for m, n, k in ([tuple(args.shape)] if args.shape else DENSE):
            x = torch.randn(m, k, device="cuda").to(torch.bfloat16)
            a_q, a_s = quant_fp8(x, round_scale=True)
            b_q = (torch.randn(n, k, device="cuda")).to(torch.float8_e4m3fn)
            b_s = torch.full((-(-n // 128), k // 128), 2.0 ** -6, device="cuda")
            c = torch.empty(m, n, dtype=torch.bfloat16, device="cuda")
            b_packed = pack_scales_mx(b_s, n, k, weight=True)      # a weight's scales are packed once
            a_packed = pack_scales_mx(a_s, m, k, weight=False)
            # the MMA alone, and with the per-call packing of the activation scales
            mma_ms = timed(lambda: gemm_e4m3_mx(a_q, a_packed, b_q, b_packed, c), flush, args.steps)
            whole_ms = timed(lambda: gemm_e4m3_block_scaled(a_q, a_s, b_q, b_s, out=c, b_packed=b_packed),
                             flush, args.steps)
            # the same product by expansion to bf16 (weight expanded once) and the plain bf16 kernel
            w_bf = dequant_block_scaled(b_q, b_s, block=(128, 128))
            a_bf = torch.empty(m, k, dtype=torch.bfloat16, device="cuda")
            expand_ms = timed(lambda: gemm_bf16(dequant_block_scaled(a_q, a_s, out=a_bf), w_bf, c), flush, args.steps)
            bf16_ms = timed(lambda: gemm_bf16(x, w_bf, c), flush, args.steps)
            check_gemm_status("cuda")
            flops = 2.0 * m * n * k
            row = {"m": m, "n": n, "k": k, "dtype": "e4m3 block-scaled (1x128 / 128x128, ue8m0 in tensor memory)",
                   "mx_mma_us": mma_ms * 1e3, "mx_mma_tflops": flops / mma_ms / 1e9,
                   "mx_with_scale_packing_us": whole_ms * 1e3, "mx_with_packing_tflops": flops / whole_ms / 1e9,
                   "expanded_to_bf16_us": expand_ms * 1e3, "expanded_tflops": flops / expand_ms / 1e9,
                   "bf16_kernel_us": bf16_ms * 1e3, "bf16_kernel_tflops": flops / bf16_ms / 1e9,
                   "mx_over_bf16_kernel": bf16_ms / mma_ms, "mx_over_expansion": expand_ms / whole_ms,
                   "mx_frac_of_measured_bf16_peak": flops / mma_ms / 1e9 / peak}
            if not args.no_library:
                # the library's fp8 GEMM (per-tensor scales: the closest form torch exposes here)
                one = torch.ones((), device="cuda")
                lib_ms = timed(lambda: torch._scaled_mm(a_q, b_q.t(), scale_a=one, scale_b=one,
                                                        out_dtype=torch.bfloat16), flush, args.steps)
                row.update({"cublaslt_fp8_per_tensor_us": lib_ms * 1e3,
                            "cublaslt_fp8_per_tensor_tflops": flops / lib_ms / 1e9,
                            "mx_vs_cublaslt_fp8": lib_ms / mma_ms})
            rows.append(row)
            del x, a_q, a_s, b_q, b_s, a_bf, w_bf, c, a_packed, b_packed
    elif args.fp8:
        from aboleth_b200.ops import gemm_e4m3

        one = torch.ones((), device="cuda")
        for m, n, k in ([tuple(args.shape)] if args.shape else DENSE):
            a = torch.randn(m, k, device="cuda").to(torch.float8_e4m3fn)
            b = (torch.randn(n, k, device="cuda")).to(torch.float8_e4m3fn)
            c = torch.empty(m, n, dtype=torch.bfloat16, device="cuda")
            ms = timed(lambda: gemm_e4m3(a, b, c), flush, args.steps)
            check_gemm_status("cuda:0")
            flops = 2.0 * m * n * k
            row = {"m": m, "n": n, "k": k, "dtype": "e4m3", "ours_us": ms * 1e3, "ours_tflops": flops / ms / 1e9}
            if not args.no_library:
                ref = torch._scaled_mm(a, b.t(), scale_a=one, scale_b=one, out_dtype=torch.bfloat16)
                row["rel_err_vs_cublaslt"] = ((c.float() - ref.float()).norm() / ref.float().norm()).item()
                ms2 = timed(lambda: torch._scaled_mm(a, b.t(), scale_a=one, scale_b=one,
                                                     out_dtype=torch.bfloat16), flush, args.steps)
                row.update(cublaslt_us=ms2 * 1e3, cublaslt_tflops=flops / ms2 / 1e9)
            rows.append(row)
            del a, b, c
    else:
        for m, n, k in ([tuple(args.shape)] if args.shape else DENSE):
            a = torch.randn(m, k, device="cuda").to(torch.bfloat16)
            b = (torch.randn(n, k, device="cuda") * 0.02).to(torch.bfloat16)
            c = torch.empty(m, n, dtype=torch.bfloat16, device="cuda")
            ms = timed(lambda: gemm_bf16(a, b, c), flush, args.steps)
            check_gemm_status("cuda")
            flops = 2.0 * m * n * k
            row = {"m": m, "n": n, "k": k, "ours_us": ms * 1e3, "ours_tflops": flops / ms / 1e9,
                   "ours_frac_of_measured": flops / ms / 1e9 / peak}
            if not args.no_library:
                ref = torch.matmul(a, b.t())
                row["rel_err_vs_cublas"] = ((c.float() - ref.float()).norm() / ref.float().norm()).item()
                ms2 = timed(lambda: torch.matmul(a, b.t(), out=c), flush, args.steps)
                row.update(cublas_us=ms2 * 1e3, cublas_tflops=flops / ms2 / 1e9)
            rows.append(row)
            del a, b, c
    emit({"bench": ("grouped gemm bf16" if args.grouped else "gemm e4m3 block-scaled" if args.block_scaled
                    else "gemm e4m3" if args.fp8 else "gemm bf16"), "n_gpus": 1,
          "dtype": "e4m3" if args.fp8 or args.block_scaled else "bf16",
          "l2": "flushed before every timed launch", "peak_bf16_tflops_measured": peak, "rows": rows},
         args.out)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
