"""Per-rank environment from a SLURM step, then exec the program.

    srun --ntasks-per-node=8 python -m aboleth_b200.utils.launch -- python bench.py --gpus 8

``srun`` starts one copy per task; each derives ``RANK``, ``WORLD_SIZE``,
``LOCAL_RANK``, ``MASTER_ADDR`` and ``MASTER_PORT`` from its own SLURM variables and
then replaces itself with the command, which is what
:meth:`aboleth_b200.bootstrap.TcpStoreBootstrap.from_env` and ``torch.distributed``
read.  The reference does the same in a shell script (scripts/multinode-launch.sh:1-75)
and asks ``scontrol`` for the host names; here the node list is expanded in Python so
that a compute node needs nothing but the package.

Rank 0 hosts the store and SLURM places it on the first node of the *step*, which is
not always the first node of the job, so ``SLURM_STEP_NODELIST`` comes before
``SLURM_JOB_NODELIST``.  The port is one per job and below Linux's ephemeral range.
"""
from __future__ import annotations

import os
import sys
from typing import Mapping, Optional, Sequence


def expand_nodelist(nodelist: str) -> list[str]:
    """``"gpu[01-03,07],login1"`` -> ``["gpu01", "gpu02", "gpu03", "gpu07", "login1"]``."""
    hosts: list[str] = []
    depth, start = 0, 0
    parts = []
    for i, ch in enumerate(nodelist):
        if ch == "[":
            depth += 1
        elif ch == "]":
            depth -= 1
            if depth < 0:
                raise ValueError(f"unbalanced ] in node list {nodelist!r}")
        elif ch == "," and depth == 0:
            parts.append(nodelist[start:i])
            start = i + 1
    if depth != 0:
        raise ValueError(f"unbalanced [ in node list {nodelist!r}")
    parts.append(nodelist[start:])
    for part in (p.strip() for p in parts):
        if not part:
            continue
        if "[" not in part:
            hosts.append(part)
            continue
        prefix, rest = part.split("[", 1)
        ranges, suffix = rest.rsplit("]", 1)
        if "[" in suffix:
            raise ValueError(f"node list {nodelist!r} has more than one bracket group per name")
        for item in ranges.split(","):
            low, _, high = item.partition("-")
            if not low.isdigit() or (high and not high.isdigit()):
                raise ValueError(f"cannot read the range {item!r} in node list {nodelist!r}")
            for value in range(int(low), int(high or low) + 1):
                hosts.append(f"{prefix}{value:0{len(low)}d}{suffix}")
    return hosts


def slurm_environment(env: Optional[Mapping[str, str]] = None) -> dict[str, str]:
    """The variables one rank needs, from the SLURM variables of its task."""
    env = os.environ if env is None else env
    nodelist = env.get("SLURM_STEP_NODELIST") or env.get("SLURM_JOB_NODELIST")
    if not nodelist:
        raise RuntimeError("SLURM_JOB_NODELIST is unset: run this through srun")
    if not env.get("SLURM_PROCID") or not env.get("SLURM_NTASKS"):
        raise RuntimeError("SLURM_PROCID/SLURM_NTASKS are unset: run this through srun")
    hosts = expand_nodelist(nodelist)
    if not hosts:
        raise RuntimeError(f"no host name in {nodelist!r}")
    job = int(env.get("SLURM_JOB_ID") or 0)
    return {
        "MASTER_ADDR": hosts[0],
        "MASTER_PORT": env.get("MASTER_PORT") or str(20000 + job % 10000),
        "RANK": env["SLURM_PROCID"],
        "WORLD_SIZE": env["SLURM_NTASKS"],
        "LOCAL_RANK": env.get("SLURM_LOCALID") or "0",
        "PYTHONUNBUFFERED": "1",
    }


def main(argv: Optional[Sequence[str]] = None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    if argv and argv[0] == "--":
        argv = argv[1:]
    if not argv:
        print("usage: python -m aboleth_b200.utils.launch -- <command> [args...]", file=sys.stderr)
        return 2
    try:
        os.environ.update(slurm_environment())
    except (RuntimeError, ValueError) as error:
        print(f"launch: {error}", file=sys.stderr)
        return 1
    os.execvp(argv[0], argv)
    return 0  # not reached


if __name__ == "__main__":
    raise SystemExit(main())
