#!/usr/bin/env python
"""Tier 2 in one page: write a transport program, see what the passes do to it, run it.

The program sends ``--bytes`` in ``--chain`` puts to a peer, publishes them with one signal and
waits for the peer's signal (here the peer is the rank itself, through a loopback endpoint).
Puts chained by ``after=`` are one submission closed by one release.  The same puts written
without ``after=`` are one submission each; the passes merge them on a queue transport and let
them share the signal's barrier and release on peer memory - the table this script prints shows
both forms with the passes off and on.  ``--compile-only`` stops before the launch and needs no GPU.
"""
import argparse
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))

from aboleth_b200.compiler import ProgramBuilder, build_artifact, compilation, compile_program  # noqa: E402


def program(nbytes: int, chain: int, chained: bool = True) -> ProgramBuilder:
    b = ProgramBuilder("chain", threads=128, args=[
        ("src", "ptr"), ("endpoints", "table"), ("dst_table", "table"), ("flag_table", "table"),
        ("my_flag", "ptr"), ("epoch", "u64")])
    endpoint = b.endpoint("endpoints", 0)
    piece = nbytes // chain
    token = None
    for c in range(chain):
        token = b.put(endpoint, b.remote("dst_table", 0, offset=c * piece), b.local(f"src + {c * piece}"),
                      bytes=piece, after=token if chained else None)
    published = b.signal(endpoint, b.remote("flag_table", 0), epoch="epoch", after=token)
    b.wait_signal("my_flag", "epoch")   # the peer's signal (our own, on a loopback endpoint)
    b.wait(published)                   # local completion of the chain
    return b


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--transport", default="p2p", choices=["p2p", "proxy", "rdma"])
    ap.add_argument("--bytes", type=int, default=1 << 16)
    ap.add_argument("--chain", type=int, default=8)
    ap.add_argument("--compile-only", action="store_true")
    ap.add_argument("--show", action="store_true", help="print the scheduled IR and the emitted CUDA")
    args = ap.parse_args()

    results = {}
    for chained in (True, False):
        for passes in ("none", "default"):
            with compilation(args.transport, rank=0, world_size=1, passes=passes):
                results[chained, passes] = compile_program(program(args.bytes, args.chain, chained))
    for (chained, passes), compiled in results.items():
        facts = compiled.facts
        print(f"{'chained' if chained else 'unchained':9s} passes={passes:8s} submissions={facts['batches']} "
              f"commands={facts['commands']} barriers={facts['barriers']} system_fences={facts['system_fences']} "
              f"ready_stores={facts['ready_stores']} rewrites={ {k: v for k, v in compiled.passes.items() if v} }")
    compiled = results[True, "default"]
    if args.show:
        print(compiled.ir)
        print(compiled.cuda)
    artifact = build_artifact(compiled)
    print(f"cubin {artifact.cubin_bytes} bytes, {artifact.registers} registers, {artifact.spill_bytes} spill bytes")
    if args.compile_only:
        return 0

    import torch

    import aboleth_b200 as ab
    from aboleth_b200.compiler import LoadedKernel

    torch.cuda.set_device(0)
    runtime = ab.Runtime(0)
    try:
        endpoint = runtime.create_local_endpoint(ab.Transport(args.transport))
        src = torch.arange(args.bytes // 4, dtype=torch.int32, device="cuda").view(torch.uint8)
        dst = torch.zeros(args.bytes, dtype=torch.uint8, device="cuda")
        flag = torch.zeros(1, dtype=torch.int64, device="cuda")
        status = torch.zeros(2, dtype=torch.int64, device="cuda")
        endpoints = torch.tensor([endpoint.handle], dtype=torch.int64, device="cuda")
        dst_table = torch.tensor([dst.data_ptr(), 0], dtype=torch.int64, device="cuda")
        flag_table = torch.tensor([flag.data_ptr(), 0], dtype=torch.int64, device="cuda")
        kernel = LoadedKernel(artifact)
        for epoch in (1, 2, 3):
            dst.zero_()
            torch.cuda.synchronize()
            kernel.launch(1, 128, [src.data_ptr(), endpoints.data_ptr(), dst_table.data_ptr(),
                                   flag_table.data_ptr(), flag.data_ptr(), epoch, status.data_ptr()],
                          stream=torch.cuda.current_stream().cuda_stream)
            torch.cuda.synchronize()
            ok = status.tolist() == [0, 0] and torch.equal(dst, src) and flag.item() == epoch
            print(f"epoch {epoch}: status {status.tolist()} bytes {'match' if torch.equal(dst, src) else 'DIFFER'} "
                  f"flag {flag.item()}")
            if not ok:
                return 1
    finally:
        runtime.close()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
