"""A kernel whose transport phases are planned outside it and spliced in at compile time.

The kernel only says WHERE a phase runs (``invoke_phase <id> <arguments>``); what the phase
does, how often it has to complete and how deep the peers' queues are come from an external
transport program.  ``compile_program(kernel, plan=...)`` splices the fragment at every
invocation, stamps the planned completion interval on its waits and runs the usual pipeline.
Compile-only: needs no GPU.

    python examples/planned_phase.py [--transport rdma|proxy|p2p]
"""
import argparse
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))

from aboleth_b200.compiler import compilation, compile_program, materialize_phases  # noqa: E402

PLAN = """program dispatch.plan kind=transport_program
phase dispatch program_id=1 interval=8 capacities=64,64
phase dispatch.tail program_id=1 interval=4 capacities=32
fragment send_slot program_id=1 params=table:i64,peer:i64,dst:i64,src:i64,bytes:i64,flag:i64,it:i64 {
  %e = endpoint table peer
  %r = remote_at dst
  %l = local src
  %t = put %e %r %l bytes=bytes
  %f = remote_at flag
  %s = signal %e %f epoch=(it+1) after=%t
  planned_wait %s iteration=it
}
"""

KERNEL = """program dispatch backend={backend}
arg endpoints table
arg slots ptr
arg staging ptr
arg flags ptr
arg rows u64
for it 0 16 {{
  invoke_phase 1 endpoints 1 (slots+(it%4)*65536) (staging+(it%4)*65536) rows*128 (flags+8) it
}}
"""


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--transport", default="rdma", choices=["rdma", "proxy", "p2p"])
    args = ap.parse_args()
    kernel = KERNEL.format(backend=args.transport)
    spliced = materialize_phases(kernel, PLAN)
    wait = next(line.strip() for line in spliced.splitlines() if "planned_wait" in line)
    print("spliced wait:", wait)
    with compilation(args.transport, rank=0, world_size=2):
        compiled = compile_program(kernel, plan=PLAN)
    poll = [line.strip() for line in compiled.ir.splitlines() if line.strip().startswith(("poll", "wait "))]
    print(f"transport={args.transport} submissions={compiled.facts.get('submissions', compiled.facts.get('batches'))} "
          f"completion={poll[0] if poll else 'vacuous'}")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
