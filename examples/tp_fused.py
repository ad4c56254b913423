#!/usr/bin/env python
"""Tensor-parallel linear layers fused with their collective, one launch each.

    torchrun --nproc-per-node N examples/tp_fused.py     # N >= 1

Column-parallel: ``C = all_gather(A) @ B_local^T`` - the tcgen05 main loop starts on the rank's own
rows while its epilogue warps push the shard to the peers.  Row-parallel: ``out = reduce_scatter(A @
B_local^T)`` - the epilogue sends each partial tile to its owner, which sums in fp32.
Both are compared with NCCL + torch.matmul in fp32.
"""
import argparse

from _world import close_world, open_world


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--rows-per-rank", type=int, default=512)
    ap.add_argument("--hidden", type=int, default=2048)
    ap.add_argument("--ffn-per-rank", type=int, default=1024)
    args = ap.parse_args()
    world, distributed = open_world()

    import torch
    import torch.distributed as dist

    from aboleth_b200.parallel import AllGatherGemm, GemmReduceScatter

    n, m_local = world.world_size, args.rows_per_rank
    g = torch.Generator(device="cuda").manual_seed(7 + world.rank)
    a_local = torch.randn(m_local, args.hidden, generator=g, device="cuda").to(torch.bfloat16)
    w_up = torch.randn(args.ffn_per_rank, args.hidden, generator=g, device="cuda").to(torch.bfloat16) * 0.05
    w_down = torch.randn(args.hidden, args.ffn_per_rank, generator=g, device="cuda").to(torch.bfloat16) * 0.05

    ag = AllGatherGemm.create(world, m_local, args.hidden)
    rs = GemmReduceScatter.create(world, m_local, args.hidden)
    h = ag(a_local, w_up)                      # [n * m_local, ffn_per_rank]
    out = rs(h, w_down)                        # [m_local, hidden]
    torch.cuda.synchronize()
    ag.check()
    rs.check()

    a_full = a_local
    if distributed:
        a_full = torch.empty(n * m_local, args.hidden, dtype=torch.bfloat16, device="cuda")
        dist.all_gather_into_tensor(a_full, a_local)
    h_ref = a_full.float() @ w_up.float().t()
    partial = h.float() @ w_down.float().t()   # from the fused h, so that only this step is compared
    if distributed:
        dist.all_reduce(partial)
    out_ref = partial[world.rank * m_local:(world.rank + 1) * m_local]
    rel = lambda got, want: ((got.float() - want).norm() / want.norm()).item()  # noqa: E731
    e1, e2 = rel(h, h_ref), rel(out, out_ref)
    print(f"rank {world.rank}/{n}: all-gather->GEMM rel. error {e1:.2e}, GEMM->reduce-scatter {e2:.2e}")
    close_world(world, distributed)
    return 0 if e1 < 5e-3 and e2 < 8e-3 else 1


if __name__ == "__main__":
    raise SystemExit(main())
