#!/usr/bin/env python
"""All-to-all and put/signal-chain microbenchmarks over NVLink peer memory, with an
NCCL baseline (grouped send/recv through ``all_to_all_single``).

    torchrun --nproc-per-node N benchmarks/comm_bench.py --min-bytes 1024 --max-bytes 268435456 --out out.json

Per-peer message sizes are powers of two; the payload is seeded uniform-random
bytes that the receiver regenerates and checks on the device.  Bus bandwidth is
``(n-1) * S / t`` with ``t`` the mean round time of the slowest rank, GB = 1e9
bytes (the reference's definition, experiments/bench/README.md:111-131).
Chain lengths split each message into that many puts per signal; ``unbatched``
publishes every put separately for comparison.
"""
import argparse

from common import emit, setup, teardown

import torch
import torch.distributed as dist

from aboleth_b200.bench_support import NVLINK_GBS, device_max, sync_ranks
from aboleth_b200.ops import alltoall, check_payload, fill_payload


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--min-bytes", dest="min", type=int, default=1024)
    ap.add_argument("--max-bytes", dest="max", type=int, default=1 << 26)
    ap.add_argument("--rounds", type=int, default=20)
    ap.add_argument("--chains", default="1,8,64")
    ap.add_argument("--max-lanes", type=int, default=64,
                    help="lanes (CTAs) per peer for messages of 64 MiB and more; smaller ones use at most 32")
    ap.add_argument("--graph-max", type=int, default=1 << 20,
                    help="largest message for which the NCCL rounds are also timed as one captured CUDA graph")
    ap.add_argument("--out", default=None)
    args = ap.parse_args()
    ab, world, distributed = setup()
    n, rank, dev = world.world_size, world.rank, world.torch_device
    sizes = [s for s in (1 << e for e in range(10, 31)) if args.min <= s <= args.max]
    top, lanes_cap = max(sizes), args.max_lanes
    arena = world.runtime.allocate(2 * n * top + n * lanes_cap * 8)
    reg = world.register(arena, network=False)
    table = world.exchange_regions([
        world.region("recv", reg, offset=n * top, length=n * top),
        world.region("flags", reg, offset=2 * n * top, length=n * lanes_cap * 8)], tag="comm")
    send, flags = arena[: n * top], arena[2 * n * top:].view(torch.int64)
    status = torch.zeros(2, dtype=torch.int64, device=dev)
    errors = torch.zeros(1, dtype=torch.int64, device=dev)
    nccl_in = torch.empty(n * top, dtype=torch.uint8, device=dev) if distributed else None
    nccl_out = torch.empty_like(nccl_in) if distributed else None
    rows = []

    def timed(fn, rounds):
        sync_ranks(distributed)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        return device_max(a.elapsed_time(b), distributed) / rounds * 1e-3

    for size in sizes:
        for p in range(n):
            fill_payload(send[p * top:], size, 4242, rank, p)
        rounds = max(3, min(args.rounds, (1 << 31) // max(size * max(n - 1, 1), 1)))
        for chain in [int(c) for c in args.chains.split(",")]:
            for mode, batched in (("vector", True), ("bulk", True), ("vector", False)):
                if chain == 1 and not batched:
                    continue
                if chain > 1 and mode == "bulk":
                    continue
                wide = size >= (64 << 20) and mode == "bulk"   # more lanes only help the bulk-copy mode
                lanes = max(1, min(lanes_cap if wide else min(lanes_cap, 32), size // 16384))
                if size // lanes // chain < 16:
                    continue
                flags.zero_()
                sync_ranks(distributed)
                kw = dict(stride=top, nbytes=size, rank=rank, world=n, lanes=lanes, chain=chain,
                          batched=batched, mode=mode, include_self=(n == 1))
                tabs = (table.addresses("recv"), table.addresses("flags"))
                alltoall(send, *tabs, flags, status, epoch0=0, rounds=3, **kw)
                t = timed(lambda: alltoall(send, *tabs, flags, status, epoch0=3, rounds=rounds, **kw), rounds)
                errors.zero_()
                for s in range(n):
                    if s != rank or n == 1:
                        check_payload(arena[n * top + s * top:], size, 4242, s, rank, errors)
                sync_ranks(distributed)
                peers = max(n - 1, 1)
                bus = peers * size / t / 1e9
                rows.append({"impl": "aboleth_b200", "bytes_per_peer": size, "mode": mode, "chain": chain,
                             "batched": batched, "lanes": lanes, "round_us": t * 1e6, "busbw_gbs": bus,
                             "frac_of_770": bus / NVLINK_GBS, "wrong_words": int(errors.item()),
                             "status": status.tolist()})
        if distributed:
            view_in, view_out = nccl_in[: n * size], nccl_out[: n * size]
            for _ in range(3):
                dist.all_to_all_single(view_out, view_in)

            def nccl_rounds():
                for _ in range(rounds):
                    dist.all_to_all_single(view_out, view_in)
            t = timed(nccl_rounds, rounds)
            bus = (n - 1) * size / t / 1e9
            rows.append({"impl": "nccl all_to_all_single", "bytes_per_peer": size, "round_us": t * 1e6,
                         "busbw_gbs": bus, "frac_of_770": bus / NVLINK_GBS})
            if size <= args.graph_max:
                # The same rounds captured once in a CUDA graph: no per-round host launch cost, which is
                # what the rounds-in-one-launch kernel above does not pay either.
                try:
                    graph = torch.cuda.CUDAGraph()
                    side = torch.cuda.Stream()
                    side.wait_stream(torch.cuda.current_stream())
                    with torch.cuda.stream(side):
                        with torch.cuda.graph(graph, stream=side):
                            for _ in range(rounds):
                                dist.all_to_all_single(view_out, view_in)
                    torch.cuda.current_stream().wait_stream(side)
                    graph.replay()
                    torch.cuda.synchronize()
                    t = timed(graph.replay, rounds)
                    bus = (n - 1) * size / t / 1e9
                    rows.append({"impl": "nccl all_to_all_single, graph-captured", "bytes_per_peer": size,
                                 "rounds_per_graph": rounds, "round_us": t * 1e6, "busbw_gbs": bus,
                                 "frac_of_770": bus / NVLINK_GBS})
                    del graph
                except RuntimeError as exc:   # a capture the library refuses is recorded, not fatal
                    rows.append({"impl": "nccl all_to_all_single, graph-captured", "bytes_per_peer": size,
                                 "error": str(exc)[:300]})
    emit({"bench": "alltoall+chains", "n_gpus": n, "rows": rows,
          "methodology": "rounds inside one launch; CUDA events; max over ranks; payload checked on device; "
                         "messages >= 128 MiB in total exceed L2, smaller ones are L2-resident by nature"},
         args.out)
    teardown(world, distributed)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
