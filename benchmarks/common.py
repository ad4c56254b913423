"""Shared set-up of the multi-rank benchmark scripts (one process per GPU under torchrun)."""
from __future__ import annotations

import json
import os
import sys
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
    start_clock_sampler(local)
    return ab, world, size > 1


_SAMPLER = None


def start_clock_sampler(index: int = 0) -> None:
    """Sample the GPU's SM clock and throttle reasons until ``emit`` (read-only NVML queries)."""
    global _SAMPLER
    from aboleth_b200.utils.clocks import ClockSampler

    if _SAMPLER is None:
        _SAMPLER = ClockSampler(index)
        _SAMPLER.start()


def load_measured_peaks() -> dict:
    """The copy bandwidth and cuBLAS rate measured on this machine, when a record of them sits at
    the root of the checkout; the documented fall-back figures otherwise."""
    from aboleth_b200 import bench_support

    path = Path(__file__).resolve().parent.parent / "MEASURED_PEAKS.json"
    if path.exists():
        bench_support.set_peaks({**json.loads(path.read_text()), "source": "measured"})
    return bench_support.measured_peaks()


def teardown(world, distributed: bool) -> None:
    torch.cuda.synchronize()
    if distributed:
        dist.barrier()
    world.close()
    if distributed:
        dist.destroy_process_group()


from aboleth_b200.utils import provenance  # noqa: E402,F401


def emit(record: dict, out: str | None) -> None:
    """Rank 0 prints one JSON line and optionally writes it to ``out``."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    global _SAMPLER
    clocks = _SAMPLER.stop() if _SAMPLER is not None else None
    _SAMPLER = None
    record = {**record, "clocks": clocks, "provenance": provenance()}
    line = json.dumps(record)
    print(line, flush=True)
    if out:
        Path(out).parent.mkdir(parents=True, exist_ok=True)
        Path(out).write_text(line + "\n")
