"""World bring-up shared by the examples: one process per GPU under torchrun, or a single rank."""
import os
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))


def open_world(transport: str = "p2p"):
    """Returns ``(world, distributed)``.  Under torchrun the control plane is a gloo group (metadata
    only); the data plane is CUDA IPC over NVLink set up by ``connect_all``."""
    import torch
    import torch.distributed as dist

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
    world.connect_all(transport)
    return world, size > 1


def close_world(world, distributed: bool) -> None:
    import torch
    import torch.distributed as dist

    torch.cuda.synchronize()
    if distributed:
        dist.barrier()
    world.close()
    if distributed:
        dist.destroy_process_group()
