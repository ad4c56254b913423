"""Symmetric allocations with an NVLink multicast mapping (NVLS).

A buffer every rank allocates with the same size through CUDA's virtual-memory API, mapped into
every peer (unicast addresses, as with CUDA IPC) and, where the fabric supports it, bound to one
NVLink multicast object: a ``multimem.st`` to the multicast address lands at the same offset of
every rank's buffer, replicated by NVSwitch, so a broadcast leaves the sending GPU once.

The allocation, the handle exchange and the multicast binding are PyTorch's
(``torch.distributed._symmetric_memory``, over the process group's store); the kernels that use
the addresses are this package's (``put`` through a peer address, ``st_multicast16`` /
``copy_strided_multicast`` in ``include/aboleth/device.cuh``).  This is the allocation provider the
reference reserves as ``CUDA_VMM`` (python/aboleth/runtime.py:83-86) without an implementation.

A process that dies while its memory is bound to a multicast object can fault its peers' NVLink
ports; release (:meth:`SymmetricArena.close`) between steps and never use this in a test that
makes a rank leave.
"""
from __future__ import annotations

from typing import Optional

import torch


class SymmetricArena:
    """``nbytes`` of zeroed device memory, the same on every rank of ``group``."""

    def __init__(self, nbytes: int, device: torch.device, group=None):
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm_mem

        if not dist.is_initialized():
            raise RuntimeError("a symmetric arena needs an initialised torch.distributed process group")
        self.group = group if group is not None else dist.group.WORLD
        self.tensor = symm_mem.empty(int(nbytes), dtype=torch.uint8, device=device)
        self.handle = symm_mem.rendezvous(self.tensor, self.group)
        self.tensor.zero_()
        torch.cuda.synchronize(device)
        self.handle.barrier()            # every rank's buffer is zero before anyone writes into a peer's
        self.rank, self.world_size = self.handle.rank, self.handle.world_size
        self.peer_addresses = [int(p) for p in self.handle.buffer_ptrs]
        # 0 when the fabric (or the driver) offers no multicast object for these GPUs
        self.multicast_address = int(self.handle.multicast_ptr or 0)

    @property
    def has_multicast(self) -> bool:
        return self.multicast_address != 0

    def addresses(self, offset: int) -> torch.Tensor:
        """int64 device table: the address of byte ``offset`` of every rank's buffer."""
        return torch.tensor([p + offset for p in self.peer_addresses], dtype=torch.int64, device=self.tensor.device)

    def multicast(self, offset: int) -> int:
        return self.multicast_address + offset if self.multicast_address else 0

    def barrier(self) -> None:
        self.handle.barrier()

    def close(self) -> None:
        """Drop the mappings (collective in effect: every rank should do it at the same point)."""
        self.handle = None
        self.tensor = None


def multicast_supported(device: Optional[torch.device] = None) -> bool:
    """Whether this build of PyTorch and this GPU can bind symmetric memory to a multicast object."""
    try:
        from torch._C._distributed_c10d import _SymmetricMemory
    except Exception:  # noqa: BLE001
        return False
    if not torch.cuda.is_available():
        return False
    device = device or torch.device("cuda", torch.cuda.current_device())
    try:
        from torch._C._autograd import DeviceType
        return bool(_SymmetricMemory.has_multicast_support(DeviceType.CUDA, device.index or 0))
    except Exception:  # noqa: BLE001
        return False
