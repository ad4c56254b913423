#!/usr/bin/env python
"""Run the fused EP dispatch -> stand-in experts -> combine layer on ONE GPU.

    python benchmarks/ep_layer.py --tokens 4096 --steps 4 --warmup 2

Small and self-contained so that it can be profiled (one rank, DeepSeek-V3
shape by default).  Prints per-phase device times in microseconds.
"""
import argparse
import json
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=4096)
    ap.add_argument("--hidden", type=int, default=7168)
    ap.add_argument("--experts", type=int, default=256)
    ap.add_argument("--top-k", type=int, default=8)
    ap.add_argument("--steps", type=int, default=4)
    ap.add_argument("--warmup", type=int, default=2)
    ap.add_argument("--flush", action="store_true")
    ap.add_argument("--out", default=None)
    args = ap.parse_args()

    import torch

    import aboleth_b200 as ab
    from aboleth_b200.bench_support import EpLayerBench

    torch.cuda.set_device(0)
    with ab.World(0, 1, device=0) as world:
        world.connect_all("p2p")
        layer = EpLayerBench(world, tokens=args.tokens, hidden=args.hidden, experts=args.experts,
                             top_k=args.top_k, group=128, seed=7)
        for _ in range(args.warmup):
            layer.step()
        layer.check()
        out = layer.phase_times(steps=args.steps, distributed=False, flush=args.flush)
        line = json.dumps({k: out[k] for k in ("dispatch_us", "combine_us", "tokens_per_rank")})
        print(line)
        if args.out:
            Path(args.out).parent.mkdir(parents=True, exist_ok=True)
            Path(args.out).write_text(line + "\n")
    return 0


if __name__ == "__main__":
    sys.exit(main())
