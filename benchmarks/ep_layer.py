#!/usr/bin/env python
"""Run the fused EP dispatch -> stand-in experts -> combine layer on ONE GPU.

    python benchmarks/ep_layer.py --tokens 4096 --steps 4 --warmup 2
    python benchmarks/ep_layer.py --tokens 4096 --emulate-ranks 2 --steps 2

Small and self-contained so that it can be profiled (DeepSeek-V3 shape by default).  With one
rank it prints per-phase device times and the kernels' own phase stamps.  ``--emulate-ranks R``
runs R ranks of the layer on the one device (every rank's send half before any rank's receive
half, so no launch waits on another): each rank then moves the record traffic of an R-GPU job
through local memory, which is what the profiler captures for the multi-rank case.
"""
import argparse
import json
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))


def emulate(args) -> int:
    import torch

    from aboleth_b200.moe import LocalMoEGroup, MoESpec
    from aboleth_b200.moe.reference import standin_layer_reference
    from aboleth_b200.ops import expert_offsets, standin_expert

    torch.cuda.set_device(0)
    r = args.emulate_ranks
    spec = MoESpec(capacity=args.tokens, hidden=args.hidden, top_k=args.top_k, experts=args.experts,
                   ranks=r, value_type="f8E4M3FN", scale_group=128)
    group = LocalMoEGroup(spec)
    g = torch.Generator(device="cuda").manual_seed(7)
    xs = [torch.randn(args.tokens, args.hidden, generator=g, device="cuda").to(torch.bfloat16) for _ in range(r)]
    logits = [torch.randn(args.tokens, args.experts, generator=g, device="cuda") for _ in range(r)]
    pairs = r * args.tokens * min(args.top_k, spec.experts_per_rank)
    grouped = [torch.empty(pairs, args.hidden, dtype=torch.bfloat16, device="cuda") for _ in range(r)]
    bad = 0
    for _ in range(args.warmup + args.steps):
        results = group.dispatch(xs, logits=logits)
        offsets = []
        for k, res in enumerate(results):
            off, _ = expert_offsets(res.expert_counts_by_source)
            standin_expert(res.expert_input, res.expert_scales, grouped[k], res.expert_ids,
                           res.expert_weights, res.expert_pos, res.recv_counts, world=r,
                           capacity=spec.capacity, group=spec.scale_group, offsets=off)
            offsets.append(off)
        outs = group.combine(grouped, expert_offsets=offsets)
        torch.cuda.synchronize()
        group.check()
    for k in range(r):
        slot = group.slots[k]
        expected, tol = standin_layer_reference(xs[k], slot.topk_ids[: args.tokens].long(),
                                                slot.topk_weights[: args.tokens], fp8=True)
        err = (outs[k].float() - expected).abs().amax(dim=-1)
        bad += int((~(err <= tol)).sum().item())
    print(json.dumps({"emulated_ranks": r, "tokens_per_rank": args.tokens, "verify_errors": bad}))
    return 0 if bad == 0 else 1


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=4096)
    ap.add_argument("--hidden", type=int, default=7168)
    ap.add_argument("--experts", type=int, default=256)
    ap.add_argument("--top-k", type=int, default=8)
    ap.add_argument("--steps", type=int, default=4)
    ap.add_argument("--warmup", type=int, default=2)
    ap.add_argument("--flush", action="store_true")
    ap.add_argument("--unweighted", action="store_true",
                    help="experts apply the gates, the combine sums partials (the reference's split)")
    ap.add_argument("--emulate-ranks", type=int, default=0)
    ap.add_argument("--out", default=None)
    args = ap.parse_args()
    if args.emulate_ranks > 1:
        return emulate(args)

    import torch

    import aboleth_b200 as ab
    from aboleth_b200.bench_support import EpLayerBench

    torch.cuda.set_device(0)
    with ab.World(0, 1, device=0) as world:
        world.connect_all("p2p")
        layer = EpLayerBench(world, tokens=args.tokens, hidden=args.hidden, experts=args.experts,
                             top_k=args.top_k, group=128, seed=7, weighted=not args.unweighted)
        for _ in range(args.warmup):
            layer.step()
        layer.check()
        out = layer.phase_times(steps=args.steps, distributed=False, flush=args.flush)
        record = {k: out[k] for k in ("dispatch_us", "combine_us", "tokens_per_rank", "combine")}
        record["verify_errors"] = layer.verify()
        # The kernels' own phase stamps (one traced step).
        slot = layer.layer.slot
        slot.enable_trace()
        res = slot.dispatch(layer.x[0], logits=layer.logits[0])
        torch.cuda.synchronize()
        record["dispatch_trace_us"] = slot.trace()
        staged = layer._experts(layer.weighted)(res, slot.expert_output)
        offsets, rows = staged if isinstance(staged, tuple) else (None, slot.expert_output)
        slot.trace_buffer.zero_()
        slot.combine(rows, expert_offsets=offsets)
        torch.cuda.synchronize()
        record["combine_trace_us"] = slot.trace()
        slot.trace_buffer = None
        line = json.dumps(record)
        print(line)
        if args.out:
            Path(args.out).parent.mkdir(parents=True, exist_ok=True)
            Path(args.out).write_text(line + "\n")
    return 0


if __name__ == "__main__":
    sys.exit(main())
