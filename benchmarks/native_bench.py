"""Build and run the standalone C++ arm of the Tier-1 ladder (``benchmarks/native/bench_tier1.cu``).

    python benchmarks/native_bench.py [--gpus N] [--bench pingpong|window|alltoall|all] [--bytes B ...]
                                      [--sweep] [--out results.json]

The program is one process for all ranks (rank r on GPU r, peers through CUDA peer access) and is
written against ``aboleth/device.cuh`` alone; this driver only compiles it with nvcc for sm_100a,
forwards the options and collects the JSON lines it prints.  ``--sweep`` repeats the ladder over
8 B-equivalent (16 B), 4 KiB, 64 KiB and 1 MiB payloads.  Exit code 77 means "no GPU here".

``--arm nccl_host`` builds and runs ``benchmarks/native/bench_nccl_host.cu`` instead: the NCCL
host-API baseline (one grouped ncclSend / ncclRecv exchange per round, same bus-bandwidth formula),
linked against the NCCL of the ``nvidia.nccl`` package; it needs at least two GPUs.
"""
from __future__ import annotations

import argparse
import json
import shutil
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent
SOURCE = ROOT / "native" / "bench_tier1.cu"
BINARY = ROOT / "native" / "build" / "bench_tier1"
INCLUDE = ROOT.parent / "aboleth_b200" / "include"


def build(force: bool = False) -> Path:
    """Compile the program if the binary is older than its source or the Tier-1 header."""
    newest = max(SOURCE.stat().st_mtime, (INCLUDE / "aboleth" / "device.cuh").stat().st_mtime)
    if not force and BINARY.exists() and BINARY.stat().st_mtime >= newest:
        return BINARY
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    BINARY.parent.mkdir(parents=True, exist_ok=True)
    cmd = [nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo",
           f"-I{INCLUDE}", str(SOURCE), "-o", str(BINARY)]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError("native bench build failed:\n" + " ".join(cmd) + "\n" + proc.stdout + proc.stderr)
    return BINARY


NCCL_SOURCE = ROOT / "native" / "bench_nccl_host.cu"
NCCL_BINARY = ROOT / "native" / "build" / "bench_nccl_host"


def _nccl_paths() -> tuple[Path, Path]:
    """Header and library of the NCCL that ships with PyTorch's wheels (``nvidia.nccl``)."""
    import importlib.util

    spec = importlib.util.find_spec("nvidia.nccl")
    if spec is None or not spec.submodule_search_locations:
        raise RuntimeError("the nvidia.nccl package (NCCL headers and library) is not installed")
    base = Path(list(spec.submodule_search_locations)[0])
    libraries = sorted((base / "lib").glob("libnccl.so*"))
    if not (base / "include" / "nccl.h").exists() or not libraries:
        raise RuntimeError(f"no nccl.h / libnccl.so under {base}")
    return base / "include", libraries[0]


def build_nccl(force: bool = False) -> Path:
    """Compile the NCCL host-API baseline arm (grouped ncclSend / ncclRecv all-to-all)."""
    if not force and NCCL_BINARY.exists() and NCCL_BINARY.stat().st_mtime >= NCCL_SOURCE.stat().st_mtime:
        return NCCL_BINARY
    include, library = _nccl_paths()
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    NCCL_BINARY.parent.mkdir(parents=True, exist_ok=True)
    cmd = [nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", f"-I{include}",
           str(NCCL_SOURCE), f"-L{library.parent}", f"-l:{library.name}", "-Xlinker", f"-rpath={library.parent}",
           "-o", str(NCCL_BINARY)]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError("NCCL arm build failed:\n" + " ".join(cmd) + "\n" + proc.stdout + proc.stderr)
    return NCCL_BINARY


def run_nccl(args: list[str], timeout: float = 300.0) -> tuple[int, list[dict]]:
    proc = subprocess.run([str(build_nccl()), *args], capture_output=True, text=True, timeout=timeout)
    rows = [json.loads(line) for line in proc.stdout.splitlines() if line.startswith("{")]
    if proc.returncode not in (0, 77):
        sys.stderr.write(proc.stderr)
    return proc.returncode, rows


def run(args: list[str], timeout: float = 300.0) -> tuple[int, list[dict]]:
    proc = subprocess.run([str(build()), *args], capture_output=True, text=True, timeout=timeout)
    rows = [json.loads(line) for line in proc.stdout.splitlines() if line.startswith("{")]
    if proc.returncode not in (0, 77):
        sys.stderr.write(proc.stderr)
    return proc.returncode, rows


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--sweep", action="store_true")
    ap.add_argument("--out", default=None)
    ap.add_argument("--build-only", action="store_true")
    ap.add_argument("--arm", choices=["tier1", "nccl_host"], default="tier1",
                    help="tier1: the Tier-1 ladder; nccl_host: the grouped ncclSend/ncclRecv all-to-all baseline")
    known, rest = ap.parse_known_args()
    if known.build_only:
        print(build(force=True) if known.arm == "tier1" else build_nccl(force=True))
        return 0
    sys.path.insert(0, str(ROOT.parent))
    from aboleth_b200.utils.clocks import ClockSampler

    sampler = ClockSampler(0)   # the C++ arms run as child processes; GPU 0 is sampled around them
    sampler.start()
    if known.arm == "nccl_host":
        rows, code = [], 0
        for size in (["1024", "16384", "262144", "4194304", "67108864"] if known.sweep else [None]):
            rc, out = run_nccl(rest if size is None else [*rest, "--bytes", size])
            rows += out
            code = code or rc
            if rc == 77:
                break
        for row in rows:
            print(json.dumps(row))
        if known.out:
            sys.path.insert(0, str(ROOT))
            from common import provenance  # benchmarks/common.py
            Path(known.out).write_text(json.dumps({"bench": "nccl host all-to-all", "rows": rows,
                                                   "clocks": sampler.stop(),
                                                   "provenance": provenance()}, indent=1))
        return code
    rows: list[dict] = []
    code = 0
    sizes = ["16", "4096", "65536", "1048576"] if known.sweep else [None]
    for size in sizes:
        extra = rest if size is None else [*rest, "--bytes", size]
        rc, out = run(extra)
        rows += out
        code = code or rc
        if rc == 77:
            break
    for row in rows:
        print(json.dumps(row))
    if known.out:
        sys.path.insert(0, str(ROOT))
        from common import provenance  # benchmarks/common.py
        Path(known.out).write_text(json.dumps({"bench": "native tier-1 ladder", "rows": rows,
                                               "clocks": sampler.stop(),
                                               "provenance": provenance()}, indent=1))
    return code


if __name__ == "__main__":
    sys.exit(main())
