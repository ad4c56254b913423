#!/usr/bin/env python
"""Peer-copy bandwidth between two GPUs of one node: the denominator of every NVLink roofline
fraction in this repository (``bench_support.NVLINK_GBS``).

    python benchmarks/peer_copy_bench.py --bytes 1073741824 --out peer_copy.json

One process, two devices.  A device-to-device ``copy_`` between buffers of GPU 0 and GPU 1 (the
copy engines over NVLink) is timed with CUDA events on the source device's stream: one direction
alone, and both directions at once (two streams).  Best and median of ``--iters`` after warm-up;
GB = 1e9 bytes.  The nominal figure is 900 GB/s per direction per GPU.
"""
import argparse
import json
import statistics
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent))


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--bytes", type=int, default=1 << 30)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--out", default=None)
    args = ap.parse_args()

    import torch

    from common import emit, start_clock_sampler

    if torch.cuda.device_count() < 2:
        print(json.dumps({"skipped": "needs two GPUs"}))
        return 77
    start_clock_sampler(0)
    a0 = torch.empty(args.bytes, dtype=torch.uint8, device="cuda:0").fill_(1)
    b1 = torch.empty(args.bytes, dtype=torch.uint8, device="cuda:1").fill_(2)
    a1 = torch.empty(args.bytes, dtype=torch.uint8, device="cuda:1")
    b0 = torch.empty(args.bytes, dtype=torch.uint8, device="cuda:0")
    s0, s1 = torch.cuda.Stream(device="cuda:0"), torch.cuda.Stream(device="cuda:1")

    def sync():
        torch.cuda.synchronize(0)
        torch.cuda.synchronize(1)

    def one_way():
        with torch.cuda.device(0), torch.cuda.stream(s0):
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            a1.copy_(a0, non_blocking=True)
            stop.record()
        sync()
        return start.elapsed_time(stop)

    def both_ways():
        with torch.cuda.device(0), torch.cuda.stream(s0):
            start0, stop0 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start0.record()
            a1.copy_(a0, non_blocking=True)
            stop0.record()
        with torch.cuda.device(1), torch.cuda.stream(s1):
            start1, stop1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start1.record()
            b0.copy_(b1, non_blocking=True)
            stop1.record()
        sync()
        return max(start0.elapsed_time(stop0), start1.elapsed_time(stop1))

    rows = []
    for name, fn in (("one direction", one_way), ("both directions at once", both_ways)):
        for _ in range(3):
            fn()
        ms = [fn() for _ in range(args.iters)]
        gbs = [args.bytes / (t * 1e-3) / 1e9 for t in ms]
        rows.append({"case": name, "bytes": args.bytes, "best_gbs_per_direction": max(gbs),
                     "median_gbs_per_direction": statistics.median(gbs), "iters": args.iters})
    ok = bool(torch.equal(a1[:4096].cpu(), a0[:4096].cpu()))
    emit({"bench": "peer copy (copy engines over NVLink)", "rows": rows, "copied_correctly": ok,
          "nominal_gbs_per_direction": 900.0}, args.out)
    return 0


if __name__ == "__main__":
    sys.exit(main())
