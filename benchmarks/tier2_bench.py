#!/usr/bin/env python
"""Latency and bandwidth ladders with kernels EMITTED by the Tier-2 specializer.

    python benchmarks/tier2_bench.py                              # one GPU, endpoint loops back to itself
    torchrun --nproc-per-node 2 benchmarks/tier2_bench.py         # rank 0 leads, rank 1 echoes

``pingpong``: per round ``chain`` puts closed by one signal, then a bounded wait for the echo
(the own signal on a loopback endpoint).  ``windowed``: ``window`` puts per round and CTA, one
completion per round, a drain at the end; bandwidth = bytes moved / CUDA-event time of the
launch.  Programs: aboleth_b200/compiler/programs.py; the reference drives the same two ladders
with its generated kernels (experiments/bench/tier2.py:32-127, ladder.py).
"""
import argparse
import statistics

from common import emit, setup, teardown

import torch

from aboleth_b200.bench_support import device_max, sync_ranks
from aboleth_b200.compiler import LoadedKernel, build_artifact, compilation, compile_program
from aboleth_b200.compiler.programs import pingpong, windowed


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--rounds", type=int, default=200)
    ap.add_argument("--out", default=None)
    args = ap.parse_args()
    ab, world, distributed = setup()
    n, rank, dev = world.world_size, world.rank, world.torch_device
    if n > 2:
        raise SystemExit("tier2_bench runs on one GPU (loopback) or two")
    peer = 1 - rank if n == 2 else 0
    top = 64 << 20
    arena = world.runtime.allocate(2 * top + 64)
    reg = world.register(arena, network=False)
    table = world.exchange_regions([world.region("t2_recv", reg, offset=top, length=top + 64)], tag="tier2")
    recv = int(table.addresses("t2_recv")[peer])
    remote = torch.tensor([0, 0, recv, 0], dtype=torch.int64, device=dev)       # (address, key) pairs, entry 1
    endpoints = torch.tensor([0, world.endpoints[peer].handle if n == 2 else
                              world.runtime.create_local_endpoint(ab.Transport.P2P).handle],
                             dtype=torch.int64, device=dev)
    status = torch.zeros(2, dtype=torch.int64, device=dev)
    stream = lambda: torch.cuda.current_stream().cuda_stream  # noqa: E731
    rows, epoch = [], 0

    def timed(launch, repeats=5):
        times = []
        for i in range(repeats + 1):
            sync_ranks(distributed)
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            launch()
            b.record()
            torch.cuda.synchronize()
            if status.tolist() != [0, 0]:
                raise RuntimeError(f"transport status {status.tolist()}")
            if i:
                times.append(device_max(a.elapsed_time(b), distributed))
        return statistics.median(times)

    # ---- latency: put(s) + signal + wait for the echo ----
    for nbytes in (8, 256, 4096, 65536):
        for chain in (1, 8):
            if nbytes // chain < 8:
                continue
            piece = max(nbytes // chain, 8)
            flag = arena[top + chain * piece: top + chain * piece + 8].view(torch.int64)
            with compilation("p2p", rank=rank, world_size=max(n, 2)):
                kernel = LoadedKernel(build_artifact(compile_program(
                    pingpong(nbytes, chain=chain, leader=(rank == 0)))))

            def launch():
                nonlocal epoch
                kernel.launch(1, 32, [arena.data_ptr(), endpoints.data_ptr(), remote.data_ptr(), flag.data_ptr(),
                                      args.rounds, epoch, status.data_ptr()], stream=stream())
                epoch += args.rounds
            ms = timed(launch)
            rows.append({"ladder": "pingpong", "bytes": nbytes, "chain": chain,
                         "round_us": ms * 1e3 / args.rounds, "loopback": n == 1})
    # ---- bandwidth: windows of puts, one completion per round ----
    for nbytes in (4096, 65536, 1 << 20):
        for ctas in (1, 8, 32):
            window = 8
            if ctas * window * nbytes > top:
                continue
            with compilation("p2p", rank=rank, world_size=max(n, 2)):
                kernel = LoadedKernel(build_artifact(compile_program(windowed(nbytes, window=window, threads=256))))
            rounds = max(4, min(args.rounds, (256 << 20) // (ctas * window * nbytes)))
            ms = timed(lambda: kernel.launch(ctas, 256, [arena.data_ptr(), endpoints.data_ptr(), remote.data_ptr(),
                                                         rounds, status.data_ptr()], stream=stream()))
            moved = ctas * window * nbytes * rounds
            rows.append({"ladder": "windowed", "bytes": nbytes, "ctas": ctas, "window": window,
                         "gbs": moved / (ms * 1e-3) / 1e9, "loopback": n == 1})
    emit({"bench": "tier-2 emitted kernels: latency and bandwidth ladders", "n_gpus": n, "rows": rows,
          "methodology": "kernels emitted by the specializer and compiled by nvcc for sm_100a; rounds inside "
                         "one launch; CUDA events; median of 5 launches after a warm-up; max over ranks"},
         args.out)
    table.close()
    teardown(world, distributed)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
