#!/usr/bin/env python
"""A Mixtral-style MoE layer whose experts run on e4m3 end to end (DeepSeek-V3's recipe).

    python examples/fp8_experts.py                      # one GPU
    torchrun --nproc-per-node 2 examples/fp8_experts.py # experts split over the ranks

``MixtralEP(..., fp8_experts=True)``: the fused dispatch quantises the tokens to e4m3 with
power-of-two 1 x 128 scales and sends them; ``permute`` groups the received rows per expert (every
group on a 128-row boundary) together with their scales; both expert GEMMs run on the block-scaled
tensor-core path against e4m3 weights with 128 x 128 scales; the fused combine applies the gates and
returns the rows.  The result is compared with an fp32 evaluation of the dequantised weights on the
unquantised activations.
"""
import argparse

from _world import close_world, open_world


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=200)
    args = ap.parse_args()
    world, distributed = open_world()

    import torch

    from aboleth_b200.models import MixtralConfig, MixtralEP
    from aboleth_b200.ops import check_gemm_status

    cfg = MixtralConfig(layers=1, hidden=1024, experts=8, top_k=2, ffn=2048, heads=8, kv_heads=2, vocab=256,
                        max_seq=64)
    model = MixtralEP(cfg, world, max_batch=8, max_prompt=32, seed=5, fp8_experts=True)
    g = torch.Generator(device="cuda").manual_seed(100 + world.rank)
    x = torch.randn(args.tokens, cfg.hidden, generator=g, device="cuda").to(torch.bfloat16)
    layer = model.layers[0]
    got = model.moe_layer(x, layer).float()
    torch.cuda.synchronize()
    model.check()
    check_gemm_status("cuda")

    # Every rank holds other experts: gather the dequantised weights for the oracle.
    w13, w2 = model.dequantised_experts(layer)
    if distributed:
        import torch.distributed as dist
        parts13 = [torch.empty_like(w13) for _ in range(world.world_size)]
        parts2 = [torch.empty_like(w2) for _ in range(world.world_size)]
        dist.all_gather(parts13, w13)
        dist.all_gather(parts2, w2)
        w13, w2 = torch.cat(parts13), torch.cat(parts2)
    want = model.reference_moe_layer(x, layer, w13, w2)
    error = ((got - want).norm() / want.norm()).item()
    print(f"rank {world.rank}: {args.tokens} tokens through {cfg.experts} e4m3 experts "
          f"({model.local_experts} on this rank), relative error {error:.3e}")
    close_world(world, distributed)
    return 0 if error < 6e-2 else 1


if __name__ == "__main__":
    raise SystemExit(main())
