"""Shared set-up of the multi-rank benchmark scripts (one process per GPU under torchrun)."""
from __future__ import annotations

import json
import os
import platform
import subprocess
import sys
import time
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402


def setup():
    """Returns (ab module, world, distributed flag).  Rank/world from the torchrun environment."""
    import aboleth_b200 as ab

    rank = int(os.environ.get("RANK", "0"))
    size = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    bootstrap = None
    if size > 1:
        dist.init_process_group("cpu:gloo,cuda:nccl", rank=rank, world_size=size,
                                device_id=torch.device("cuda", local))
        bootstrap = ab.TorchDistributedBootstrap(dist.new_group(backend="gloo"))
    world = ab.World(rank, size, device=local, bootstrap=bootstrap)
    world.connect_all("p2p")
    return ab, world, size > 1


def teardown(world, distributed: bool) -> None:
    torch.cuda.synchronize()
    if distributed:
        dist.barrier()
    world.close()
    if distributed:
        dist.destroy_process_group()


def provenance() -> dict:
    def git(*args):
        try:
            return subprocess.run(["git", *args], capture_output=True, text=True, timeout=5,
                                  cwd=Path(__file__).resolve().parent.parent).stdout.strip()
        except Exception:  # noqa: BLE001
            return ""
    return {"time": time.strftime("%Y-%m-%dT%H:%M:%SZ", time.gmtime()), "host": platform.node(),
            "git": git("rev-parse", "--short", "HEAD"), "torch": torch.__version__,
            "cuda": torch.version.cuda, "gpu": torch.cuda.get_device_name(0),
            "nccl": ".".join(map(str, torch.cuda.nccl.version())),
            "env": {k: v for k, v in os.environ.items() if k.startswith(("ABOLETH_", "NCCL_"))}}


def emit(record: dict, out: str | None) -> None:
    """Rank 0 prints one JSON line and optionally writes it to ``out``."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    record = {**record, "provenance": provenance()}
    line = json.dumps(record)
    print(line, flush=True)
    if out:
        Path(out).parent.mkdir(parents=True, exist_ok=True)
        Path(out).write_text(line + "\n")
