#!/usr/bin/env python
"""Expert-parallel MoE layer: fused dispatch -> experts -> fused combine, checked against fp32.

    python examples/moe_layer.py                      # one GPU: every expert is local
    torchrun --nproc-per-node 8 examples/moe_layer.py # experts split over the ranks, NVLink all-to-all

Dispatch is one launch (router soft-max and top-k, fp8 1x128 quantisation, one record per (token,
destination rank) written straight into the destination's receive segment, counts and flags);
the experts here are the stand-in ``f_e(x) = x * (1 + (e mod 7) / 8)`` the tests use, so that the
result has a closed form;
combine is one launch (expert rows return, gate-weighted sum in fp32).
"""
import argparse

from _world import close_world, open_world


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=512)
    ap.add_argument("--hidden", type=int, default=2048)
    ap.add_argument("--experts", type=int, default=32)
    ap.add_argument("--top-k", type=int, default=4)
    ap.add_argument("--bf16", action="store_true", help="send bf16 rows instead of fp8 + scales")
    args = ap.parse_args()
    world, distributed = open_world()

    import torch

    from aboleth_b200.moe import MoESpec
    from aboleth_b200.moe.reference import standin_layer_reference
    from aboleth_b200.parallel import ExpertParallelLayer

    spec = MoESpec(capacity=args.tokens, hidden=args.hidden, top_k=args.top_k, experts=args.experts,
                   ranks=world.world_size, value_type="bf16" if args.bf16 else "f8E4M3FN", scale_group=128)
    layer = ExpertParallelLayer(world, spec, tag="example")
    g = torch.Generator(device="cuda").manual_seed(1234 + world.rank)
    x = torch.randn(args.tokens, args.hidden, generator=g, device="cuda").to(torch.bfloat16)
    logits = torch.randn(args.tokens, args.experts, generator=g, device="cuda")
    for step in range(3):
        out = layer.forward(x, logits).float()
        torch.cuda.synchronize()
        layer.check()  # raises if a bounded wait gave up or a segment overflowed
    ids, weights = layer.slot.topk_ids[: args.tokens].long(), layer.slot.topk_weights[: args.tokens]
    expected, tolerance = standin_layer_reference(x, ids, weights, fp8=not args.bf16, group=spec.scale_group,
                                                  amax_floor=spec.quant_amax_floor)
    error = (out - expected).abs().amax(dim=-1)
    bad = int((~(error <= tolerance)).sum())
    print(f"rank {world.rank}/{world.world_size}: {args.tokens} tokens x top-{args.top_k} of {args.experts} experts, "
          f"max |error| {error.max().item():.4f}, rows outside tolerance {bad}")
    close_world(world, distributed)
    return 1 if bad else 0


if __name__ == "__main__":
    raise SystemExit(main())
