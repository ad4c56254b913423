#!/usr/bin/env python
"""End-to-end expert-parallel MoE serving through the all2all backend entry point.

    torchrun --nproc-per-node 8 benchmarks/serve_bench.py --out out.json

Mixtral-style model (32 layers, hidden 4096, 8 experts top-2, FFN 14336, 32 heads / 8 KV
heads, bf16, random-init), synthetic prompts of uniform-random token ids (vocab 32000),
1024 input / 256 output tokens, global batch 64 split evenly over the ranks.  Reports
request latency (prefill + decode), time to first token and generated tokens/s.
"""
import argparse

from common import emit, setup, teardown

import torch

from aboleth_b200.bench_support import device_max, sync_ranks
from aboleth_b200.models import MixtralConfig, MixtralEP


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=32)
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--prompt", type=int, default=1024)
    ap.add_argument("--generate", type=int, default=256)
    ap.add_argument("--graph", action="store_true", help="replay the decode step as a CUDA graph")
    ap.add_argument("--out", default=None)
    args = ap.parse_args()
    ab, world, distributed = setup()
    w = world.world_size
    local_batch = args.batch // w
    cfg = MixtralConfig(layers=args.layers, max_seq=args.prompt + args.generate)
    cpu_group = None
    if distributed:
        import torch.distributed as dist
        cpu_group = dist.new_group(backend="gloo")
    model = MixtralEP(cfg, world, max_batch=local_batch, max_prompt=args.prompt, seed=0,
                      cpu_group=cpu_group)
    g = torch.Generator(device=world.torch_device).manual_seed(100 + world.rank)
    prompts = torch.randint(0, cfg.vocab, (local_batch, args.prompt), generator=g,
                            device=world.torch_device)
    with torch.no_grad():
        if args.graph:
            model.enable_decode_graph()
        # Warm-up at the timed shapes: library kernel selection for a new shape costs far more than a step.
        nxt = model.forward(prompts, 0).argmax(-1)
        for i in range(3):
            nxt = model.decode(nxt[:, None], args.prompt + i).argmax(-1)
        torch.cuda.synchronize()
        model.check()
        sync_ranks(distributed)
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
        ev[0].record()
        nxt = model.forward(prompts, 0).argmax(-1)
        ev[1].record()
        for i in range(args.generate - 1):
            nxt = model.decode(nxt[:, None], args.prompt + i).argmax(-1)
        ev[2].record()
        torch.cuda.synchronize()
    model.check()
    ttft = device_max(ev[0].elapsed_time(ev[1]), distributed)
    decode = device_max(ev[1].elapsed_time(ev[2]), distributed)
    total = ttft + decode
    emit({"bench": "mixtral-style EP serving", "n_gpus": w, "dtype": "bf16",
          "config": {"layers": args.layers, "hidden": cfg.hidden, "experts": cfg.experts, "top_k": cfg.top_k,
                     "ffn": cfg.ffn, "heads": cfg.heads, "kv_heads": cfg.kv_heads, "batch": args.batch,
                     "prompt": args.prompt, "generate": args.generate, "parallelism": f"ep{w} dp{w} tp1",
                     "decode": "cuda graph" if args.graph else "eager"},
          "request_latency_ms": total, "time_to_first_token_ms": ttft,
          "decode_ms_per_token": decode / max(args.generate - 1, 1),
          "generated_tokens_per_s": args.batch * args.generate / (total * 1e-3),
          "prefill_tokens_per_s": args.batch * args.prompt / (ttft * 1e-3),
          "data": "synthetic uniform-random token ids, random-init weights"}, args.out)
    teardown(world, distributed)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
