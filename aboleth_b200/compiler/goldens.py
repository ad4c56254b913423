"""Golden files of the specializer: scheduled IR, emitted CUDA C++ and facts for a
fixed set of (program, transport, switches) cases.

    python -m aboleth_b200.compiler.goldens --check tests/goldens
    python -m aboleth_b200.compiler.goldens --write tests/goldens

The reference pins byte-exact lowered IR per backend x variant x optimisation
prefix but ships no golden files (test/compiler/goldens.py:29-78); these are
committed.
"""
from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

from . import programs
from .driver import compile_program
from .options import PIPELINE_ORDER, compilation

CASES = {
    "alltoall_4096": lambda: programs.alltoall(4096),
    "stream_fused_8": lambda: programs.stream("fused", 8, 1024),
    "stream_chains_4": lambda: programs.stream("chains", 4, 256),
    "stream_pipelined_4": lambda: programs.stream("pipelined", 4, 256, reuse=4),
    "fp8_dispatch": lambda: programs.fp8_dispatch(),
    "pingpong_leader_chain4": lambda: programs.pingpong(4096, chain=4),
    "pingpong_follower": lambda: programs.pingpong(4096, leader=False),
    "windowed_8": lambda: programs.windowed(65536, window=8),
    "tier1_put_many_8_signal": lambda: _tier1("put_many_8_signal"),
    "tier1_put_inline64": lambda: _tier1("put_inline64"),
}


def _tier1(name: str):
    from ..tier1 import tier1_program

    return tier1_program(name)


BACKENDS = ("p2p", "proxy", "rdma", "efa")
VARIANTS = {"default": "default", "none": "none"}


def waterfall() -> dict[str, str]:
    """Switch sets that add the optional passes one at a time, in pipeline order."""
    out, spec = {}, "none"
    for name in PIPELINE_ORDER:
        spec += f",+{name}"
        out[f"upto_{name}"] = spec
    return out


def render(case: str, backend: str, passes: str) -> dict[str, str]:
    with compilation(backend, rank=0, world_size=2, passes=passes):
        compiled = compile_program(CASES[case]())
    return {"ir": compiled.ir, "cu": compiled.cuda,
            "facts.json": json.dumps({"facts": compiled.facts, "passes": compiled.passes},
                                     indent=1, sort_keys=True) + "\n"}


def all_files() -> dict[str, str]:
    files = {}
    for case in CASES:
        for backend in BACKENDS:
            for variant, passes in VARIANTS.items():
                for ext, text in render(case, backend, passes).items():
                    files[f"{case}.{backend}.{variant}.{ext}"] = text
    for variant, passes in waterfall().items():  # the ablation prefixes, facts only
        files[f"stream_pipelined_4.rdma.{variant}.facts.json"] = render(
            "stream_pipelined_4", "rdma", passes)["facts.json"]
    return files


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("directory", type=Path)
    mode = ap.add_mutually_exclusive_group(required=True)
    mode.add_argument("--write", action="store_true")
    mode.add_argument("--check", action="store_true")
    args = ap.parse_args(argv)
    files = all_files()
    if args.write:
        args.directory.mkdir(parents=True, exist_ok=True)
        for name, text in files.items():
            (args.directory / name).write_text(text)
        print(f"wrote {len(files)} golden files")
        return 0
    bad = [name for name, text in files.items()
           if not (args.directory / name).exists() or (args.directory / name).read_text() != text]
    for name in bad:
        print("golden mismatch:", name)
    return 1 if bad else 0


if __name__ == "__main__":
    sys.exit(main())
