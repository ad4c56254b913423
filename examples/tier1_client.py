#!/usr/bin/env python
"""Tier 1: compile a user kernel against the packaged device library and run it.

``device_library()`` publishes the header, a manifest and the nvcc flags; the kernel in
``tier1_client.cu`` is compiled with exactly those flags to a cubin and launched through the CUDA
driver on a loopback endpoint (the rank is its own peer).  ``--compile-only`` needs no GPU.
"""
import argparse
import subprocess
import sys
import tempfile
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))

import aboleth_b200 as ab  # noqa: E402

SOURCE = Path(__file__).resolve().parent / "tier1_client.cu"


def compile_client(out_dir: Path) -> Path:
    lib = ab.device_library(transports=["p2p", "proxy"])
    cubin = out_dir / "tier1_client.cubin"
    subprocess.run(["nvcc", *lib.nvcc_flags(), "-cubin", str(SOURCE), "-o", str(cubin)], check=True)
    print(f"device library {lib.digest[:16]}: {lib.header}")
    print(f"compiled {SOURCE.name} -> {cubin.stat().st_size} bytes")
    return cubin


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--compile-only", action="store_true")
    ap.add_argument("--ctas", type=int, default=8)
    ap.add_argument("--slice-bytes", type=int, default=1 << 16)
    args = ap.parse_args()
    with tempfile.TemporaryDirectory() as tmp:
        cubin = compile_client(Path(tmp))
        if args.compile_only:
            return 0
        import torch

        from aboleth_b200.compiler import Artifact, LoadedKernel

        torch.cuda.set_device(0)
        runtime = ab.Runtime(0)
        try:
            endpoint = runtime.create_local_endpoint(ab.Transport.P2P)
            kernel = LoadedKernel(Artifact("exchange_slices", "example", cubin, SOURCE, None, None, None,
                                           cubin.stat().st_size, ""))
            total = args.ctas * args.slice_bytes
            send = torch.randint(0, 255, (total,), dtype=torch.uint8, device="cuda")
            recv = torch.zeros(total, dtype=torch.uint8, device="cuda")
            flags = torch.zeros(2 * args.ctas, dtype=torch.int64, device="cuda")
            status = torch.zeros(1, dtype=torch.int64, device="cuda")
            endpoints = torch.tensor([endpoint.handle], dtype=torch.int64, device="cuda")
            for epoch in (1, 2):
                kernel.launch(args.ctas, 256, [endpoints.data_ptr(), status.data_ptr(), recv.data_ptr(),
                                               flags.data_ptr(), send.data_ptr(), flags.data_ptr(),
                                               args.slice_bytes, epoch],
                              stream=torch.cuda.current_stream().cuda_stream)
                torch.cuda.synchronize()
                words = flags[args.ctas:].tolist()
                ok = (status.item() == 0 and torch.equal(recv, send)
                      and flags[: args.ctas].tolist() == [epoch] * args.ctas
                      and words == [epoch * 1000 + c for c in range(args.ctas)])
                print(f"epoch {epoch}: status {status.item()}, payload {'matches' if torch.equal(recv, send) else 'DIFFERS'}, "
                      f"control words {words[:3]}...")
                if not ok:
                    return 1
        finally:
            runtime.close()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
