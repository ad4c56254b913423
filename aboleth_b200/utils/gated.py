"""Run a command only where the machine can run it; otherwise exit 77.

``python -m aboleth_b200.utils.gated --needs gpu --needs gpus=2 [--timeout S] -- <command>...``

CTest (``SKIP_RETURN_CODE 77``) and shell callers read exit code 77 as
"skipped", so a CPU-only box reports GPU tests as skipped rather than failed.
Any other exit code of the command passes through; a command that outlives
``--timeout`` is stopped (its own process group only) and reports 124.

Requirements: ``gpu``, ``multi-gpu``, ``gpus=<n>``, ``b200`` (compute
capability 10.x), ``nvcc``, and the NIC ones of the reference's gate
(``hca``, ``mlx5``, ``efa``), which look under ``/sys/class/infiniband``.
Same contract as the reference's ``scripts/run-gated.sh:1-120``.
"""
from __future__ import annotations

import argparse
import os
import shutil
import signal
import subprocess
import sys
from pathlib import Path
from typing import Callable, Optional, Sequence

SKIP = 77


def gpu_count(run: Callable[..., subprocess.CompletedProcess] = subprocess.run) -> int:
    if shutil.which("nvidia-smi") is None:
        return 0
    try:
        out = run(["nvidia-smi", "--list-gpus"], capture_output=True, text=True, timeout=30)
    except (OSError, subprocess.SubprocessError):
        return 0
    return sum(1 for line in out.stdout.splitlines() if line.strip()) if out.returncode == 0 else 0


def _is_b200(run: Callable[..., subprocess.CompletedProcess] = subprocess.run) -> bool:
    if shutil.which("nvidia-smi") is None:
        return False
    try:
        out = run(["nvidia-smi", "--query-gpu=compute_cap", "--format=csv,noheader"], capture_output=True,
                  text=True, timeout=30)
    except (OSError, subprocess.SubprocessError):
        return False
    caps = [line.strip() for line in out.stdout.splitlines() if line.strip()]
    return out.returncode == 0 and bool(caps) and all(c.startswith("10.") for c in caps)


def _verbs_device(prefix: str, root: Path = Path("/sys/class/infiniband")) -> bool:
    if not root.is_dir():
        return False
    return any(entry.name.startswith(prefix) for entry in root.iterdir())


def missing(need: str, *, gpus: Optional[int] = None, verbs_root: Path = Path("/sys/class/infiniband")) -> Optional[str]:
    """Why requirement ``need`` is not met here, or None when it is."""
    count = gpu_count() if gpus is None else gpus
    if need == "gpu":
        return None if count >= 1 else "no GPU"
    if need == "multi-gpu":
        return None if count >= 2 else f"{count} GPU(s), two needed"
    if need.startswith("gpus="):
        wanted = int(need.split("=", 1)[1])
        return None if count >= wanted else f"{count} GPU(s), {wanted} needed"
    if need == "b200":
        return None if _is_b200() else "no compute-capability 10.x GPU"
    if need == "nvcc":
        return None if shutil.which("nvcc") else "nvcc not on PATH"
    if need == "hca":
        return None if _verbs_device("", verbs_root) else "no verbs device"
    if need == "mlx5":
        return None if _verbs_device("mlx5_", verbs_root) else "no mlx5 device"
    if need == "efa":
        return None if _verbs_device("rdmap", verbs_root) or _verbs_device("efa", verbs_root) else "no EFA device"
    if need == "sudo":
        return None if os.geteuid() == 0 else "not root"
    raise ValueError(f"unknown requirement {need!r}")


def run_gated(needs: Sequence[str], command: Sequence[str], *, timeout: Optional[float] = None,
              gpus: Optional[int] = None) -> int:
    for need in needs:
        why = missing(need, gpus=gpus)
        if why is not None:
            print(f"SKIP: needs {need}: {why}")
            return SKIP
    proc = subprocess.Popen(list(command), start_new_session=True)
    try:
        return proc.wait(timeout=timeout)
    except subprocess.TimeoutExpired:
        # Stop exactly the process group started above.
        os.killpg(proc.pid, signal.SIGTERM)
        try:
            proc.wait(timeout=10)
        except subprocess.TimeoutExpired:
            os.killpg(proc.pid, signal.SIGKILL)
            proc.wait()
        print(f"TIMEOUT after {timeout} s: {' '.join(command)}")
        return 124


def main(argv: Optional[Sequence[str]] = None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    if "--" not in argv:
        print(__doc__)
        return 2
    split = argv.index("--")
    ap = argparse.ArgumentParser(prog="aboleth_b200.utils.gated")
    ap.add_argument("--needs", action="append", default=[])
    ap.add_argument("--timeout", type=float, default=None)
    args = ap.parse_args(argv[:split])
    command = argv[split + 1:]
    if not command:
        print(__doc__)
        return 2
    return run_gated(args.needs, command, timeout=args.timeout)


if __name__ == "__main__":
    sys.exit(main())
