#!/usr/bin/env python
"""Pass ablation of the Tier-2 specializer on the stream microbenchmark (one GPU, self loop).

    python benchmarks/ablation.py --out out.json

The stream program (K independent put + signal chains per round, planned completion with
reuse 4, final drain; aboleth_b200/compiler/programs.py ``stream("pipelined", ...)``) is
compiled with all optimisations off, then with the passes added one at a time in pipeline
order ("waterfall"), then with the defaults, for the queue transport (``proxy``: the
host-pinned command ring served by a host thread) and for peer memory (``p2p``).  Each
variant runs as ONE launch of ``rounds`` rounds against an endpoint that leads back to the
same GPU; the time per round is the CUDA-event time of the launch divided by ``rounds``
(median of 5 launches after one warm-up).  The reference reports the same experiment on
its NIC transport (experiments/bench/ablation.py; README.md:186).
"""
import argparse
import statistics

from common import emit, start_clock_sampler

import torch

import aboleth_b200 as ab
from aboleth_b200.compiler import LoadedKernel, build_artifact, compilation, compile_program
from aboleth_b200.compiler.options import PIPELINE_ORDER
from aboleth_b200.compiler.programs import stream


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--chains", default="1,4,16")
    ap.add_argument("--bytes", type=int, default=256)
    ap.add_argument("--rounds", type=int, default=2000)
    ap.add_argument("--backends", default="proxy,p2p")
    ap.add_argument("--out", default=None)
    args = ap.parse_args()
    torch.cuda.set_device(0)
    start_clock_sampler(0)
    runtime = ab.Runtime(0)
    rows = []
    try:
        for backend in args.backends.split(","):
            endpoint = runtime.create_local_endpoint(ab.Transport(backend))
            variants = [("none", "none")]
            enabled = []
            for name in PIPELINE_ORDER:
                enabled.append(name)
                variants.append((f"+{name}", "none," + ",".join("+" + n for n in enabled)))
            variants.append(("default", "default"))
            for chains in [int(c) for c in args.chains.split(",")]:
                nbytes = args.bytes
                payload = torch.arange(chains * nbytes, dtype=torch.uint8, device="cuda")
                remote = torch.zeros(chains * nbytes + chains * 8, dtype=torch.uint8, device="cuda")
                status = torch.zeros(2, dtype=torch.int64, device="cuda")
                endpoints = torch.tensor([0, endpoint.handle], dtype=torch.int64, device="cuda")
                table = torch.tensor([0, 0, remote.data_ptr(), 0], dtype=torch.int64, device="cuda")
                for label, passes in variants:
                    queue = {} if backend == "p2p" else {"queue_capacity": endpoint.capacity}
                    with compilation(backend, rank=0, world_size=2, passes=passes, **queue):
                        compiled = compile_program(stream("pipelined", chains, nbytes))
                    kernel = LoadedKernel(build_artifact(compiled))
                    times = []
                    for trial in range(6):
                        remote.zero_()
                        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                        start.record()
                        kernel.launch(1, 32, [payload.data_ptr(), endpoints.data_ptr(), table.data_ptr(),
                                              args.rounds, status.data_ptr()],
                                      stream=torch.cuda.current_stream().cuda_stream)
                        stop.record()
                        torch.cuda.synchronize()
                        if status.tolist() != [0, 0]:
                            raise RuntimeError(f"{backend} {label}: transport status {status.tolist()}")
                        if trial:
                            times.append(start.elapsed_time(stop) * 1e3 / args.rounds)
                    ok = bool(torch.equal(remote[: chains * nbytes], payload)) and \
                        remote[chains * nbytes:].view(torch.int64).tolist() == [args.rounds] * chains
                    if not ok:
                        raise RuntimeError(f"{backend} {label}: payload or epochs wrong after the run")
                    facts = compiled.facts
                    rows.append({"backend": backend, "chains": chains, "bytes": nbytes, "passes": label,
                                 "us_per_round": statistics.median(times),
                                 "batches": facts.get("batches"), "reservations": facts.get("reservations"),
                                 "completion_waits": facts.get("completion_waits"),
                                 "strong_signals": facts.get("strong_signals"),
                                 "elided_signals": facts.get("elided_signals")})
            endpoint.close()
    finally:
        runtime.close()
    base = {(r["backend"], r["chains"]): r["us_per_round"] for r in rows if r["passes"] == "none"}
    for r in rows:
        r["speedup_vs_none"] = base[(r["backend"], r["chains"])] / r["us_per_round"]
    emit({"bench": "tier-2 pass ablation, stream (pipelined chains)", "n_gpus": 1, "rounds": args.rounds,
          "rows": rows,
          "methodology": "one launch of `rounds` rounds per variant against a self-loop endpoint; CUDA events; "
                         "median of 5 launches after a warm-up; payload and epochs checked after every launch"},
         args.out)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
