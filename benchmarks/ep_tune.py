#!/usr/bin/env python
"""Phase times of the fused EP layer over a few launch configurations, at any number of GPUs.

    torchrun --nproc-per-node 8 benchmarks/ep_tune.py --out ep_tune8.json

For prefill (4096 tokens per rank) and decode (128): sender warps per CTA of the fused combine,
records per readiness block, and both combine forms (gates applied by the kernel or by the
experts).  Same timing rules as bench.py; each row carries the kernels' own phase stamps.
"""
import argparse

from common import emit, load_measured_peaks, setup, teardown

from aboleth_b200.bench_support import EpLayerBench


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--tokens", default="4096,128")
    ap.add_argument("--send-warps", default="6,7,4")
    ap.add_argument("--blocks", default="64,128,32")
    ap.add_argument("--out", default=None)
    args = ap.parse_args()
    ab, world, distributed = setup()
    load_measured_peaks()
    rows = []
    for tokens in [int(t) for t in args.tokens.split(",")]:
        layer = EpLayerBench(world, tokens=tokens, hidden=7168, experts=256, top_k=8, group=128,
                             seed=77 + world.rank, tag=f"tune{tokens}")
        for _ in range(3):
            layer.step()
        layer.check()
        slot = layer.layer.slot
        configs = [(int(w), int(args.blocks.split(",")[0])) for w in args.send_warps.split(",")]
        configs += [(int(args.send_warps.split(",")[0]), int(b)) for b in args.blocks.split(",")[1:]]
        for send_warps, block in configs:
            slot.send_warps, slot.return_block = send_warps, block
            layer.step()          # every rank switches at the same step
            for weighted in (True, False):
                out = layer.phase_times(steps=args.steps, distributed=distributed, flush=tokens <= 512,
                                        weighted=weighted)
                rows.append({"tokens_per_rank": tokens, "send_warps": send_warps, "return_block": block,
                             "combine": out["combine"], "dispatch_us": out["dispatch_us"],
                             "combine_us": out["combine_us"], "dispatch_us_min": out["dispatch_us_min"],
                             "combine_us_min": out["combine_us_min"],
                             "dispatch_frac": out["roofline"].get("dispatch_frac"),
                             "combine_frac": out["roofline"].get("combine_frac"),
                             "kernel_trace_us": out["kernel_trace_us"]})
        rows[-1]["verify_errors"] = layer.verify()
    emit({"bench": "EP layer launch configurations", "n_gpus": world.world_size, "rows": rows}, args.out)
    teardown(world, distributed)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
