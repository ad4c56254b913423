#!/usr/bin/env python
"""Fused tensor-parallel GEMM collectives at the Llama-3-70B MLP shapes, against
NCCL all-gather / reduce-scatter around torch.matmul (cuBLAS).

    torchrun --nproc-per-node 8 benchmarks/tp_bench.py --out out.json

all-gather -> GEMM : M = 8192 tokens (M / world per rank), K = 8192, N = 28672 / world
GEMM -> reduce-scatter : M = 8192, K = 28672 / world, N = 8192
Weights N(0, 0.02), activations N(0, 1), bf16.  Roofline per kernel = the slower of
FLOPs / measured cuBLAS peak and NVLink bytes / 770 GB/s.

``--fp8`` adds the block-scaled e4m3 forms (1 x 128 activation scales, 128 x 128 weight scales,
both operands e4m3 end to end) against NCCL moving the e4m3 bytes around the library's fp8 GEMM
(torch._scaled_mm with per-tensor scales, the closest form torch exposes).
"""
import argparse

from common import emit, load_measured_peaks, setup, teardown

import torch
import torch.distributed as dist

from aboleth_b200.bench_support import NVLINK_GBS, L2Flusher, device_max, sync_ranks
from aboleth_b200.ops import gemm_bf16
from aboleth_b200.parallel import AllGatherGemm, GemmReduceScatter


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=8192)
    ap.add_argument("--hidden", type=int, default=8192)
    ap.add_argument("--ffn", type=int, default=28672)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--push-parts", type=int, default=0, help="CTAs per (peer, chunk) of the push; 0 = auto")
    ap.add_argument("--fp8", action="store_true", help="also time the block-scaled e4m3 forms")
    ap.add_argument("--multicast", action="store_true",
                    help="also time the all-gather -> GEMM with its push through an NVLink multicast mapping")
    ap.add_argument("--out", default=None)
    args = ap.parse_args()
    ab, world, distributed = setup()
    w, rank, dev = world.world_size, world.rank, world.torch_device
    m_local = args.tokens // w
    g = torch.Generator(device=dev).manual_seed(rank)
    flush = L2Flusher(dev)
    peaks = load_measured_peaks()
    rows = []

    def timed(fn):
        times = []
        for it in range(args.steps + 3):
            flush()
            sync_ranks(distributed)
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda._sleep(200_000)
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            if it >= 3:
                times.append(device_max(a.elapsed_time(b), distributed))
        times.sort()
        spread.append({"min_us": times[0] * 1e3, "max_us": times[-1] * 1e3, "steps": len(times)})
        return times[len(times) // 2] * 1e3  # median, us

    spread: list[dict] = []   # one entry per timed() call, in call order

    def roof(flops, nvlink_bytes):
        t_flop = flops / (peaks["bf16_tflops"] * 1e12) * 1e6
        t_link = nvlink_bytes / (NVLINK_GBS * 1e9) * 1e6
        return max(t_flop, t_link), t_flop, t_link

    # ---- plain GEMM for context ----
    a_full = torch.randn(args.tokens, args.hidden, generator=g, device=dev).to(torch.bfloat16)
    b_col = (torch.randn(args.ffn // w, args.hidden, generator=g, device=dev) * 0.02).to(torch.bfloat16)
    out = torch.empty(args.tokens, args.ffn // w, dtype=torch.bfloat16, device=dev)
    flops = 2.0 * args.tokens * args.hidden * (args.ffn // w)
    t_ours = timed(lambda: gemm_bf16(a_full, b_col, out))
    t_lib = timed(lambda: torch.matmul(a_full, b_col.t(), out=out))
    rows.append({"op": "gemm (no collective)", "ours_us": t_ours, "cublas_us": t_lib,
                 "ours_spread": spread[-2], "cublas_spread": spread[-1],
                 "ours_tflops": flops / t_ours / 1e6, "cublas_tflops": flops / t_lib / 1e6,
                 "frac_of_measured_peak": flops / t_ours / 1e6 / peaks["bf16_tflops"]})

    # ---- all-gather -> GEMM ----
    a_local = a_full[rank * m_local:(rank + 1) * m_local].contiguous()
    fused = AllGatherGemm.create(world, m_local, args.hidden, push_parts=args.push_parts)
    t_fused = timed(lambda: fused(a_local, b_col, out))
    fused.check()
    gathered = torch.empty_like(a_full)

    def baseline_ag():
        if distributed:
            dist.all_gather_into_tensor(gathered, a_local)
        else:
            gathered.copy_(a_full)
        torch.matmul(gathered, b_col.t(), out=out)
    t_base = timed(baseline_ag)
    link = (w - 1) * m_local * args.hidden * 2
    bound, t_flop, t_link = roof(flops, link)
    rows.append({"op": "all-gather -> GEMM", "m": args.tokens, "k": args.hidden, "n": args.ffn // w,
                 "fused_us": t_fused, "nccl_plus_cublas_us": t_base, "speedup": t_base / t_fused,
                 "fused_spread": spread[-2], "baseline_spread": spread[-1],
                 "roof_us": bound, "roof_flops_us": t_flop, "roof_nvlink_us": t_link,
                 "frac_of_roof": bound / t_fused})

    fused_mc = None
    if args.multicast and distributed:
        fused_mc = AllGatherGemm.create_multicast(world, m_local, args.hidden, push_parts=args.push_parts)
        t_mc = timed(lambda: fused_mc(a_local, b_col, out))
        fused_mc.check()
        rows.append({"op": "all-gather -> GEMM, multimem push", "multicast_mapping": bool(fused_mc.multicast[0]),
                     "fused_us": t_mc, "fused_spread": spread[-1], "over_peer_store_push": t_fused / t_mc,
                     "speedup_vs_nccl_plus_cublas": t_base / t_mc, "frac_of_roof": bound / t_mc})

    # ---- GEMM -> reduce-scatter ----
    k_local = args.ffn // w
    a_row = torch.randn(args.tokens, k_local, generator=g, device=dev).to(torch.bfloat16)
    b_row = (torch.randn(args.hidden, k_local, generator=g, device=dev) * 0.02).to(torch.bfloat16)
    rs = GemmReduceScatter.create(world, m_local, args.hidden)
    out_rs = torch.empty(m_local, args.hidden, dtype=torch.bfloat16, device=dev)
    t_fused = timed(lambda: rs(a_row, b_row, out_rs))
    rs.check()
    partial = torch.empty(args.tokens, args.hidden, dtype=torch.bfloat16, device=dev)

    def baseline_rs():
        torch.matmul(a_row, b_row.t(), out=partial)
        if distributed:
            dist.reduce_scatter_tensor(out_rs, partial)
        else:
            out_rs.copy_(partial[:m_local])
    t_base = timed(baseline_rs)
    flops = 2.0 * args.tokens * k_local * args.hidden
    link = (w - 1) * m_local * args.hidden * 2
    bound, t_flop, t_link = roof(flops, link)
    rows.append({"op": "GEMM -> reduce-scatter", "m": args.tokens, "k": k_local, "n": args.hidden,
                 "fused_us": t_fused, "nccl_plus_cublas_us": t_base, "speedup": t_base / t_fused,
                 "fused_spread": spread[-2], "baseline_spread": spread[-1],
                 "roof_us": bound, "roof_flops_us": t_flop, "roof_nvlink_us": t_link,
                 "frac_of_roof": bound / t_fused})
    if args.fp8:
        from aboleth_b200.ops import pack_scales_mx
        from aboleth_b200.ops.moe_ops import quant_fp8

        fp8 = torch.float8_e4m3fn
        one = torch.ones((), device=dev)

        def weight_fp8(weight):  # 128 x 128 power-of-two block scales
            n, k = weight.shape
            blocks = weight.float().view(n // 128, 128, k // 128, 128).abs().amax(dim=(1, 3)).clamp_min(1e-10)
            scales = torch.exp2(torch.ceil(torch.log2(blocks / 448.0)))
            full = scales.repeat_interleave(128, dim=0).repeat_interleave(128, dim=1)
            return (weight.float() / full).to(fp8), pack_scales_mx(scales, n, k, weight=True)

        # all-gather -> GEMM, e4m3 shard + scale-factor atoms over NVLink
        a_q, a_s = quant_fp8(a_local, round_scale=True)
        a_packed = pack_scales_mx(a_s, m_local, args.hidden, weight=False)
        b_q, b_packed = weight_fp8(b_col)
        t_mx = timed(lambda: fused.mx(a_q, a_packed, b_q, b_packed, out))
        fused.check()
        gathered_q = torch.empty(args.tokens, args.hidden, dtype=fp8, device=dev)

        def baseline_ag_fp8():
            if distributed:
                dist.all_gather_into_tensor(gathered_q.view(torch.uint8), a_q.view(torch.uint8))
            else:
                gathered_q.view(torch.uint8)[:m_local].copy_(a_q.view(torch.uint8))
            torch._scaled_mm(gathered_q, b_q.t(), scale_a=one, scale_b=one, out_dtype=torch.bfloat16, out=out)
        t_base = timed(baseline_ag_fp8)
        flops = 2.0 * args.tokens * args.hidden * (args.ffn // w)
        link = (w - 1) * m_local * args.hidden * (1 + 1 / 32)
        rows.append({"op": "all-gather -> GEMM, e4m3 block-scaled", "m": args.tokens, "k": args.hidden,
                     "n": args.ffn // w, "fused_us": t_mx, "nccl_plus_cublaslt_fp8_us": t_base,
                     "speedup": t_base / t_mx, "fused_spread": spread[-2], "baseline_spread": spread[-1],
                     "fused_tflops": flops / t_mx / 1e6, "nvlink_bytes": link,
                     "roof_nvlink_us": link / (NVLINK_GBS * 1e9) * 1e6,
                     "over_bf16_fused": rows[1]["fused_us"] / t_mx})

        if fused_mc is not None:
            t_mc = timed(lambda: fused_mc.mx(a_q, a_packed, b_q, b_packed, out))
            fused_mc.check()
            rows.append({"op": "all-gather -> GEMM, e4m3 block-scaled, multimem push",
                         "multicast_mapping": bool(fused_mc.multicast[0]), "fused_us": t_mc,
                         "fused_spread": spread[-1], "over_peer_store_push": t_mx / t_mc,
                         "fused_tflops": flops / t_mc / 1e6})

        # GEMM -> reduce-scatter on e4m3 operands (the partials still travel as bf16)
        ar_q, ar_s = quant_fp8(a_row, round_scale=True)
        ar_packed = pack_scales_mx(ar_s, args.tokens, k_local, weight=False)
        br_q, br_packed = weight_fp8(b_row)
        t_mx = timed(lambda: rs.mx(ar_q, ar_packed, br_q, br_packed, out_rs))
        rs.check()

        def baseline_rs_fp8():
            torch._scaled_mm(ar_q, br_q.t(), scale_a=one, scale_b=one, out_dtype=torch.bfloat16, out=partial)
            if distributed:
                dist.reduce_scatter_tensor(out_rs, partial)
            else:
                out_rs.copy_(partial[:m_local])
        t_base = timed(baseline_rs_fp8)
        flops = 2.0 * args.tokens * k_local * args.hidden
        rows.append({"op": "GEMM -> reduce-scatter, e4m3 block-scaled", "m": args.tokens, "k": k_local,
                     "n": args.hidden, "fused_us": t_mx, "nccl_plus_cublaslt_fp8_us": t_base,
                     "speedup": t_base / t_mx, "fused_spread": spread[-2], "baseline_spread": spread[-1],
                     "fused_tflops": flops / t_mx / 1e6, "over_bf16_fused": rows[2]["fused_us"] / t_mx})
    emit({"bench": "tp fused collectives", "n_gpus": w, "dtype": "bf16", "peaks": peaks, "rows": rows,
          "methodology": "L2 flushed before every timed launch; CUDA events after a busy-wait kernel; "
                         "median of steps; max over ranks"}, args.out)
    if fused_mc is not None:
        fused_mc._arena.close()
    teardown(world, distributed)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
