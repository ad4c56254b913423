#!/usr/bin/env python
"""Build and run the reference project's own baseline arms, unmodified, on this machine.

The reference's transports need its compiler plug-in, which cannot be built offline; two of its
C++ benchmark arms need only CUDA plus a library that ships with this image:

``nccl_host``  experiments/bench/bench_tier1_nccl_host.cu: the all-to-all through NCCL's host API
               (grouped ncclSend / ncclRecv per peer; ``--graph-rounds K`` captures K rounds in a
               CUDA graph).  Built against the NCCL of the PyTorch wheels.
``nvshmem``    experiments/bench/bench_tier1_nvshmem.cu: the same benchmark kernels over NVSHMEM
               (put + signal per peer, or ``--collective on`` for NVSHMEM's own all-to-all).  Built
               against the ``nvidia-nvshmem`` wheel.  Two settings of the LIBRARY (not of the
               benchmark) are added to the ranks' environment unless already set: the unique-id
               bootstrap is pointed at the loopback interface, and the symmetric heap is taken
               from cudaMalloc + CUDA IPC instead of the virtual-memory API - with the latter the
               ranks of this container do not return from ``nvshmemx_init_attr``.

The sources are copied as they are from the reference checkout into ``baseline/_ref/bench`` (or
used from there when the checkout is not present) and compiled by nvcc for sm_100a; nothing of
this repository is on their path.  One process per GPU, ranks rendezvous over 127.0.0.1.

    python baseline/run_reference_arms.py --arm nccl_host --gpus 8 --out nccl_host_8.json
    python baseline/run_reference_arms.py --arm nccl_host --gpus 8 --graph-rounds 16
    python baseline/run_reference_arms.py --arm nvshmem --gpus 2 -- --collective on
"""
from __future__ import annotations

import argparse
import json
import os
import shutil
import site
import subprocess
import sys
import time
from pathlib import Path

HERE = Path(__file__).resolve().parent
BENCH = HERE / "_ref" / "bench"
# The reference checkout: ABOLETH_REFERENCE, or a directory named `reference` next to this repository.
REFERENCE = Path(os.environ.get("ABOLETH_REFERENCE", HERE.parent.parent / "reference")) / "experiments" / "bench"
SOURCES = ["bench_tier1_nccl_host.cu", "bench_tier1_nvshmem.cu", "bench_tier1_arms.cuh", "bench_common.h",
           "kernels/bench_kernels.cuh", "kernels/comm_nvshmem.cuh"]
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]


def _wheel(name: str) -> Path:
    for root in site.getsitepackages():
        path = Path(root) / "nvidia" / name
        if path.exists():
            return path
    raise RuntimeError(f"the nvidia-{name} wheel is not installed")


def stage_sources() -> None:
    """Copy the reference's files, byte for byte, next to where they are built."""
    for name in SOURCES:
        dst = BENCH / name
        if dst.exists():
            continue
        src = REFERENCE / name
        if not src.exists():
            raise RuntimeError(f"{src} is missing and {dst} was not staged earlier")
        dst.parent.mkdir(parents=True, exist_ok=True)
        shutil.copyfile(src, dst)


def build(arm: str, force: bool = False) -> Path:
    stage_sources()
    out = BENCH / f"bench_tier1_{arm}"
    if out.exists() and not force:
        return out
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    common = [nvcc, *ARCH, "-O3", "-std=c++17", f"-I{BENCH}", f"-I{BENCH / 'kernels'}"]
    if arm == "nccl_host":
        nccl = _wheel("nccl")
        cmd = [*common, f"-I{nccl / 'include'}", str(BENCH / "bench_tier1_nccl_host.cu"), "-o", str(out),
               f"-L{nccl / 'lib'}", "-l:libnccl.so.2", "-Xlinker", f"-rpath={nccl / 'lib'}"]
    else:
        shmem = _wheel("nvshmem")
        cmd = [*common, "-rdc=true", f"-I{shmem / 'include'}", str(BENCH / "bench_tier1_nvshmem.cu"), "-o",
               str(out), f"-L{shmem / 'lib'}", "-l:libnvshmem_host.so.3", "-lnvshmem_device", "-lcuda",
               "-Xlinker", f"-rpath={shmem / 'lib'}"]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError("the reference arm does not build:\n" + " ".join(cmd) + "\n" + proc.stderr[-4000:])
    return out


def run(arm: str, gpus: int, extra: list[str], *, port: int, timeout: float) -> dict:
    binary = build(arm)
    transport = "host" if arm == "nccl_host" else "ibrc"
    args = [str(binary), "--bench", "alltoall", "--transport", transport, *extra]
    procs = []
    library_env = {}
    if arm == "nvshmem":
        library_env = {"NVSHMEM_BOOTSTRAP_UID_SOCK_IFNAME": "lo", "NVSHMEM_DISABLE_CUDA_VMM": "1"}
        library_env = {k: v for k, v in library_env.items() if k not in os.environ}
    for rank in range(gpus):
        env = dict(os.environ, RANK=str(rank), WORLD_SIZE=str(gpus), LOCAL_RANK=str(rank),
                   MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), **library_env)
        procs.append(subprocess.Popen(args, env=env, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True))
    deadline = time.time() + timeout
    outputs = []
    for proc in procs:
        try:
            out, err = proc.communicate(timeout=max(1.0, deadline - time.time()))
        except subprocess.TimeoutExpired:
            for p in procs:      # only the processes started here
                p.kill()
            out, err = proc.communicate()
            err += "\n[killed: timeout]"
        outputs.append((proc.returncode, out, err))
    code, out, err = outputs[0]
    record: dict = {"arm": arm, "gpus": gpus, "command": " ".join(args[1:]), "returncodes": [o[0] for o in outputs],
                    "library_env_added": library_env}
    lines = out.splitlines()
    record["table"] = [line for line in lines if line and not line.startswith("{")]
    try:
        parsed = json.loads([line for line in lines if line.startswith("{")][-1])
        for row in parsed.get("rows", []):   # thousands of raw samples per row: keep the statistics
            row.pop("samples_ns", None)
        record["record"] = parsed
    except (IndexError, json.JSONDecodeError):
        record["stdout_tail"] = out[-3000:]
    if any(o[0] != 0 for o in outputs):
        record["stderr_tail"] = [o[2][-1500:] for o in outputs if o[0] != 0][:2]
    return record


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--arm", choices=["nccl_host", "nvshmem"], required=True)
    ap.add_argument("--gpus", type=int, default=2)
    ap.add_argument("--minbytes", type=int, default=1024)
    ap.add_argument("--maxbytes", type=int, default=1 << 28)
    ap.add_argument("--iters", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--graph-rounds", type=int, default=0)
    ap.add_argument("--port", type=int, default=29611)
    ap.add_argument("--timeout", type=float, default=600.0)
    ap.add_argument("--build-only", action="store_true")
    ap.add_argument("--out", default=None)
    ap.add_argument("extra", nargs="*", help="further flags of the reference's option parser, after --")
    args = ap.parse_args()
    if args.build_only:
        print(build(args.arm, force=True))
        return 0
    extra = ["-b", str(args.minbytes), "-e", str(args.maxbytes), "-f", "2", "-n", str(args.iters),
             "-w", str(args.warmup), *args.extra]
    if args.graph_rounds:
        extra += ["--graph-rounds", str(args.graph_rounds)]
    record = run(args.arm, args.gpus, extra, port=args.port, timeout=args.timeout)
    line = json.dumps(record)
    print(line)
    if args.out:
        Path(args.out).parent.mkdir(parents=True, exist_ok=True)
        Path(args.out).write_text(line + "\n")
    return 0 if all(c == 0 for c in record["returncodes"]) else 1


if __name__ == "__main__":
    sys.exit(main())
