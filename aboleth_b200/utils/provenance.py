"""The provenance block attached to every benchmark record (reference:
experiments/bench/common.py:977-1047): when, where, which revision, which library versions and
which ``ABOLETH_*`` / ``NCCL_*`` environment variables were set."""
from __future__ import annotations

import os
import platform
import subprocess
import time
from pathlib import Path


def provenance() -> dict:
    import torch

    root = Path(__file__).resolve().parent.parent.parent

    def git(*args: str) -> str:
        try:
            return subprocess.run(["git", *args], capture_output=True, text=True, timeout=5,
                                  cwd=root).stdout.strip()
        except Exception:  # noqa: BLE001
            return ""

    record = {"time": time.strftime("%Y-%m-%dT%H:%M:%SZ", time.gmtime()), "host": platform.node(),
              # A copy of the tree without its history names its revision in ABOLETH_GIT_REV.
              "git": git("rev-parse", "--short", "HEAD") or os.environ.get("ABOLETH_GIT_REV", ""),
              "torch": torch.__version__,
              "cuda": torch.version.cuda,
              "env": {k: v for k, v in os.environ.items() if k.startswith(("ABOLETH_", "NCCL_"))}}
    if torch.cuda.is_available():
        record["gpu"] = torch.cuda.get_device_name(0)
        record["nccl"] = ".".join(map(str, torch.cuda.nccl.version()))
    return record
