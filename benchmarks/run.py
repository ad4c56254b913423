#!/usr/bin/env python
"""Benchmark presets: one name per experiment, the launcher line built for you.

    python benchmarks/run.py list
    python benchmarks/run.py alltoall --gpus 8 --out results/
    python benchmarks/run.py all --gpus 2 --dry-run

Every preset runs one of the scripts in this directory (one process per GPU through
``torch.distributed.run`` on 127.0.0.1 when ``--gpus`` > 1) and writes its JSON record to
``--out``.  The reference ships the same idea as ``scripts/aboleth-bench``.
"""
import argparse
import os
import shlex
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent

# name -> (script, extra arguments, GPU counts it accepts, what it measures)
PRESETS = {
    "headline": ("../bench.py", ["--steps", "20", "--warmup", "5"], (1, 2, 4, 8),
                 "EP dispatch + combine, DeepSeek-V3 shape, tokens/s (the JSON line of bench.py)"),
    "alltoall": ("comm_bench.py", ["--max-bytes", str(256 << 20)], (2, 4, 8),
                 "all-to-all bus bandwidth and put/signal chains against NCCL"),
    "ladder": ("tier2_bench.py", [], (1, 2), "latency / bandwidth ladders with emitted Tier-2 kernels"),
    "ablation": ("ablation.py", [], (1,), "pass waterfall of the specializer on the stream microbenchmark"),
    "moe": ("ep_layer.py", ["--tokens", "4096", "--steps", "10", "--warmup", "3"], (1,),
            "one-rank dispatch / combine phase times (profiling case)"),
    "moe-decode": ("ep_layer.py", ["--tokens", "128", "--steps", "10", "--warmup", "3", "--flush"], (1,),
                   "decode-size dispatch / combine with a flushed L2"),
    "gemm": ("gemm_bench.py", [], (1,), "bf16 tcgen05 GEMM against cuBLAS"),
    "gemm-fp8": ("gemm_bench.py", ["--fp8"], (1,), "e4m3 GEMM against cuBLASLt"),
    "gemm-fp8-block": ("gemm_bench.py", ["--block-scaled"], (1,),
                       "block-scaled e4m3 GEMM on the fp8 tensor path, against its bf16 expansion, the bf16 kernel and cuBLASLt"),
    "gemm-grouped": ("gemm_bench.py", ["--grouped"], (1,), "grouped expert GEMM against a loop of cuBLAS calls"),
    "tp": ("tp_bench.py", [], (2, 4, 8), "AG->GEMM and GEMM->RS fused kernels against NCCL + cuBLAS"),
    "tp-fp8": ("tp_bench.py", ["--fp8", "--multicast", "--steps", "20"], (2, 4, 8),
               "the same plus the block-scaled e4m3 forms and the all-gather push through NVLink multicast"),
    "peer-copy": ("peer_copy_bench.py", [], (2,), "copy-engine peer copy, one way and both ways: the NVLink denominator"),
    "moe-emulated": ("ep_layer.py", ["--tokens", "2048", "--emulate-ranks", "2", "--steps", "2"], (1,),
                     "two ranks of the EP layer on one GPU (the profiler's multi-rank case)"),
    "tp-emulated": ("tp_local.py", ["--ranks", "2", "--tokens", "4096", "--hidden", "4096", "--ffn", "8192"], (1,),
                    "two ranks of the fused TP kernels on one GPU (the profiler's multi-rank case)"),
    "serve": ("serve_bench.py", ["--graph"], (1, 2, 4, 8), "Mixtral-style EP serving, decode replayed as a CUDA graph"),
    "native": ("native_bench.py", ["--sweep"], (1, 2, 4, 8), "C++ arm of the Tier-1 ladder (one process, rank per GPU)"),
    "nccl-host": ("native_bench.py", ["--arm", "nccl_host", "--sweep"], (2, 4, 8),
                  "C++ NCCL host-API all-to-all baseline (grouped ncclSend / ncclRecv)"),
    "probe": ("-m aboleth_b200.endpoint_probe", [], (1, 2, 4, 8), "endpoint calibration (lanes x warps) and the fitted profile"),
}


def command(name: str, gpus: int, out: Path, port: int) -> list[str]:
    script, extra, allowed, _ = PRESETS[name]
    if gpus not in allowed:
        raise SystemExit(f"preset {name!r} runs on {allowed} GPUs, not {gpus}")
    target = script.split() if script.startswith("-m") else [str((HERE / script).resolve())]
    launcher = [sys.executable]
    one_process = name in ("native", "nccl-host", "peer-copy")  # these programs drive every GPU themselves
    if gpus > 1 and not one_process:
        launcher += ["-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={gpus}",
                     "--master-addr", "127.0.0.1", "--master-port", str(port)]
    args = list(extra)
    if name == "headline":
        args = ["--gpus", str(gpus)] + args
    elif one_process and name != "peer-copy":
        args += ["--gpus", str(gpus)]
    elif name == "probe" and gpus == 1:
        args += ["--loopback"]
    if name != "headline":
        args += ["--out", str(out / f"{name}_{gpus}gpu.json")]
    return launcher + target + args


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("preset", help="a preset name, `all` or `list`")
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--out", type=Path, default=Path("bench_results"))
    ap.add_argument("--port", type=int, default=29600)
    ap.add_argument("--dry-run", action="store_true", help="print the command lines only")
    args = ap.parse_args()
    if args.preset == "list":
        for name, (_, _, allowed, what) in PRESETS.items():
            print(f"{name:14s} gpus {','.join(map(str, allowed)):8s} {what}")
        return 0
    names = [n for n in PRESETS if args.gpus in PRESETS[n][2]] if args.preset == "all" else [args.preset]
    if any(n not in PRESETS for n in names):
        raise SystemExit(f"unknown preset {args.preset!r}; try `list`")
    args.out.mkdir(parents=True, exist_ok=True)
    status = 0
    for offset, name in enumerate(names):
        cmd = command(name, args.gpus, args.out, args.port + offset)
        print("+", " ".join(shlex.quote(c) for c in cmd), flush=True)
        if args.dry_run:
            continue
        env = dict(os.environ, PYTHONPATH=f"{ROOT}{os.pathsep}{os.environ.get('PYTHONPATH', '')}")
        if name == "headline":
            with open(args.out / f"headline_{args.gpus}gpu.json", "w") as sink:
                rc = subprocess.run(cmd, cwd=ROOT, env=env, stdout=sink).returncode
        else:
            rc = subprocess.run(cmd, cwd=ROOT, env=env).returncode
        status = status or rc
    return status


if __name__ == "__main__":
    raise SystemExit(main())
