"""KV-cache transfer manager: producer pushes page runs into a consumer's slot storage.

``CompiledKVTransferManager`` keeps, per rank, the registered page pool, the slot storage
peers write into and the readiness cells indexed ``(slot, layer group, source rank)``; it
turns a request's block lists into runs, launches the push, and lets the consumer wait per
layer group (4 layers per readiness event on NVLink profiles, so layer 0 waits for layers
0-3 and compute overlaps the next group).  API shape: reference python/aboleth/kv/manager.py:47-127
(``begin_step / start_transfer / wait_for_layer / poll``); direction: push (producer stores),
as in the reference's generic frontend kernels.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Sequence

import torch

from ..world import World
from . import copy as kvcopy
from .lifecycle import TransferLedger, TransferRecord, TransferState
from .profile import KVTargetProfile, select_kv_target_profile


@dataclass(frozen=True)
class KVPoolLayout:
    layers: int
    blocks: int            # pages in this rank's pool, per layer
    page_bytes: int
    slots: int             # in-flight transfers a consumer accepts
    slot_pages: int        # pages per layer a slot can hold

    @property
    def layer_bytes(self) -> int:
        return self.blocks * self.page_bytes

    @property
    def slot_layer_bytes(self) -> int:
        return self.slot_pages * self.page_bytes


class CompiledKVTransferManager:
    def __init__(self, world: World, layout: KVPoolLayout, *,
                 profile: Optional[KVTargetProfile] = None, tag: str = "kv"):
        self.world, self.layout = world, layout
        name = torch.cuda.get_device_name(world.device) if not world.runtime._cpu else ""
        self.profile = profile or select_kv_target_profile(name)
        l, ranks = layout, world.world_size
        self.groups = -(-l.layers // self.profile.consumers_per_readiness)
        pool_bytes = l.layers * l.layer_bytes
        slot_bytes = l.slots * l.layers * l.slot_layer_bytes
        cells = l.slots * self.groups * ranks
        self.arena = world.runtime.allocate(pool_bytes + slot_bytes + cells * 8)
        self.pool = self.arena[:pool_bytes].view(l.layers, l.blocks, l.page_bytes)
        self.slots = self.arena[pool_bytes:pool_bytes + slot_bytes].view(l.slots, l.layers, l.slot_pages,
                                                                         l.page_bytes)
        self.ready = self.arena[pool_bytes + slot_bytes:].view(torch.int64).view(l.slots, self.groups, ranks)
        reg = world.register(self.arena, network=False)
        self.table = world.exchange_regions([
            world.region("kv_slots", reg, offset=pool_bytes, length=slot_bytes),
            world.region("kv_ready", reg, offset=pool_bytes + slot_bytes, length=cells * 8)], tag=tag)
        self.status = torch.zeros(2, dtype=torch.int64, device=world.torch_device)
        self.ledger = TransferLedger(l.slots)
        self._arrivals = torch.zeros(4096, dtype=torch.int32, device=world.torch_device)
        self.last_transfer_us: Optional[float] = None

    # -- producer side ---------------------------------------------------------------------
    def start_transfer(self, request_id: str, consumer: int, src_blocks: Sequence[int],
                       slot: int, epoch: int, *, dst_pages: Optional[Sequence[int]] = None) -> int:
        """Push ``src_blocks`` (every layer) into ``slot`` of rank ``consumer``; returns the number of
        (run, layer) batches launched.  ``epoch`` is the readiness value the consumer waits for."""
        l, rank = self.layout, self.world.rank
        dst_pages = list(range(len(src_blocks))) if dst_pages is None else list(dst_pages)
        if max(dst_pages, default=0) >= l.slot_pages:
            raise ValueError("the transfer does not fit the consumer's slot")
        runs = kvcopy.canonicalize_block_runs(src_blocks, dst_pages)
        slots_base = self.table.addresses("kv_slots")[consumer].item()
        ready_base = self.table.addresses("kv_ready")[consumer].item()
        ranks = self.world.world_size
        batches = []
        per_group = self.profile.consumers_per_readiness
        for group in range(self.groups):
            layers = range(group * per_group, min((group + 1) * per_group, l.layers))
            cell = ready_base + ((slot * self.groups + group) * ranks + rank) * 8
            for layer in layers:
                for s, d, n in runs:
                    src = self.pool[layer, s].data_ptr()
                    dst = slots_base + ((slot * l.layers + layer) * l.slot_pages + d) * l.page_bytes
                    batches.append((src, dst, n * l.page_bytes, cell))
        # ONE launch for the whole transfer.  The batches of a readiness group name the same cell and
        # share one arrival counter: the cell is published by the last worker of the group's last
        # batch, never by a batch that merely finished first.
        dev = self.world.torch_device
        packed = kvcopy.pack_batches(batches, dev)
        group_of, group_target, groups = kvcopy.pack_groups([b[3] for b in batches],
                                                            self.profile.copy_workers, dev)
        if groups > self._arrivals.numel():
            self._arrivals = torch.zeros(groups, dtype=torch.int32, device=dev)
        kvcopy.push(packed, self._arrivals, len(batches), epoch, workers=self.profile.copy_workers,
                    threads=self.profile.threads, status=self.status, group_of=group_of,
                    group_target=group_target)
        launched = len(batches)
        return launched

    # -- consumer side ----------------------------------------------------------------------
    def begin_step(self, request_id: str, layers: Optional[int] = None) -> Optional[TransferRecord]:
        """Admit a transfer (None when every slot is busy).  The record's slot and epoch are what
        the producer must be told."""
        return self.ledger.admit(request_id, layers or self.layout.layers)

    def wait_for_layer(self, request_id: str, layer: int, source: int) -> None:
        """Enqueue a bounded wait for the readiness group holding ``layer`` from rank ``source``."""
        record = self.ledger.get(request_id)
        if record.state == TransferState.ADMITTED:
            record.move(TransferState.TRANSFERRING)
        group = layer // self.profile.consumers_per_readiness
        cell = self.ready[record.slot, group, source:source + 1]
        kvcopy.wait_ready(cell, record.epoch, self.status)

    def poll(self, request_id: str, source: int) -> TransferState:
        """Host-side check: ready once every group's cell reached the epoch; failed on a status."""
        record = self.ledger.get(request_id)
        if record.terminal:
            return record.state
        status = self.status.tolist()
        if status[0]:
            record.move(TransferState.FAILED, error=f"transport status {status[0]} detail {status[1]:#x}")
            return record.state
        cells = self.ready[record.slot, :, source]
        record.ready_layers = int((cells >= record.epoch).sum().item()) * self.profile.consumers_per_readiness
        if record.ready_layers >= record.layers:
            if record.state == TransferState.ADMITTED:
                record.move(TransferState.TRANSFERRING)
            record.move(TransferState.READY)
        return record.state

    def slot_pages(self, request_id: str, layer: int) -> torch.Tensor:
        record = self.ledger.get(request_id)
        return self.slots[record.slot, layer]

    def release(self, request_id: str) -> None:
        self.ledger.get(request_id).move(TransferState.CONSUMED)

    def abort(self, request_id: str) -> None:
        self.ledger.get(request_id).move(TransferState.ABORTED)
