"""Persistent same-node KV-cache migration runtime for a prefill/decode pair of engines.

``VLLMKVPeerRuntime`` owns one two-rank P2P world and the engine's registered per-layer
KV caches.  The decode rank PULLS: it reads the prefill rank's blocks over NVLink into its
own cache (block ids are remapped) and records one event per layer group, so attention on
layer 0 can start while later layers are still in flight.  Below the plan's copy-engine
threshold the SMs copy (``kv_push_kernel`` with a peer address as its source - 16-byte
vectors, several workers per run); at or above it, and with few enough runs, the copy
engine does (one ``cudaMemcpyAsync`` per run and layer).

API after the reference's python/aboleth/integrations/vllm_kv.py:31-561 (1P1D only,
``register_kv_caches`` / ``pull_blocks`` / ``start_pull_blocks`` /
``start_layered_pull_blocks``); an existing :class:`World` may be passed instead of a
host/port pair.
"""
from __future__ import annotations

import time
from dataclasses import dataclass
from typing import Optional

import torch

from ..bootstrap import TcpStoreBootstrap
from ..kv import copy as kvcopy
from ..kv.profile import KVRuntimeOverrides, KVTargetProfile, select_kv_target_profile
from ..patterns import (CompiledKVCacheMigrationPlan, KVCacheLayoutContract, KVCacheMigrationSpec,
                        compile_kv_cache_migration)
from ..world import World


@dataclass(frozen=True)
class KVCachePullTicket:
    completion: torch.cuda.Event
    layer_events: dict[str, torch.cuda.Event]


class VLLMKVPeerRuntime:
    def __init__(self, *, rank: int, world_size: int, device: int, host: str = "127.0.0.1", port: int = 0,
                 timeout: float = 300.0, target_profile: Optional[KVTargetProfile] = None,
                 overrides: Optional[KVRuntimeOverrides] = None, world: Optional[World] = None):
        if world_size != 2:
            raise NotImplementedError("KV migration between engines supports one prefill and one decode rank")
        self.rank, self.world_size, self.device = rank, world_size, device
        self.target_profile = target_profile or select_kv_target_profile(
            torch.cuda.get_device_name(device), overrides=overrides)
        self.overrides = overrides or KVRuntimeOverrides()
        self._owns_world = world is None
        if world is None:
            self.bootstrap = TcpStoreBootstrap(rank, world_size, host=host, port=port, timeout=timeout)
            world = World(rank, world_size, device=device, bootstrap=self.bootstrap)
            world.connect_all("p2p")
        self.world = world
        self._registrations: list = []
        self._table = None
        self._kv_caches: dict[str, torch.Tensor] = {}
        self._order: tuple[str, ...] = ()
        self._plan: Optional[CompiledKVCacheMigrationPlan] = None
        self._page_bytes = self._max_blocks = 0
        self._status = torch.zeros(2, dtype=torch.int64, device=world.torch_device)
        self._ready = None
        self._arrivals = torch.zeros(4096, dtype=torch.int32, device=world.torch_device)
        self._epoch = 0
        self._last_transfer_us = 0.0
        self._last_physicalization = "none"
        self._last_transfer_bytes = self._last_run_count = 0
        self.profile_transfers = False

    # -- facts --------------------------------------------------------------------------------
    @property
    def plan(self) -> CompiledKVCacheMigrationPlan:
        if self._plan is None:
            raise RuntimeError("KV caches are not registered")
        return self._plan

    last_transfer_us = property(lambda self: self._last_transfer_us)
    last_physicalization = property(lambda self: self._last_physicalization)
    last_transfer_bytes = property(lambda self: self._last_transfer_bytes)
    last_run_count = property(lambda self: self._last_run_count)
    asynchronous_completion = property(lambda self: self.plan.physicalization.asynchronous_completion)
    consumer_layer_pipeline = property(lambda self: self.plan.physicalization.consumer_layer_pipeline)

    # -- registration ----------------------------------------------------------------------------
    def register_kv_caches(self, kv_caches: dict[str, torch.Tensor], *,
                           consumer_order: Optional[tuple[str, ...]] = None) -> None:
        """``kv_caches``: layer name -> contiguous tensor whose first dimension indexes blocks (the
        same geometry on both ranks).  ``consumer_order`` is the order layers are consumed in."""
        if self._kv_caches:
            raise RuntimeError("KV caches are already registered")
        if not kv_caches:
            raise ValueError("no KV cache to register")
        order = tuple(consumer_order or kv_caches)
        if set(order) != set(kv_caches):
            raise ValueError("consumer_order must name every registered layer once")
        first = kv_caches[order[0]]
        blocks = first.shape[0]
        page_bytes = first[0].numel() * first.element_size()
        for name in order:
            cache = kv_caches[name]
            if not cache.is_contiguous() or cache.shape[0] != blocks or \
                    cache[0].numel() * cache.element_size() != page_bytes:
                raise ValueError(f"layer {name!r} does not share the block geometry of {order[0]!r}")
            if cache.data_ptr() % 16 or page_bytes % 16:
                raise ValueError("KV pages must be 16-byte aligned")
        regions = []
        for name in order:
            registration = self.world.register(kv_caches[name], network=False)
            self._registrations.append(registration)
            regions.append(self.world.region(f"kv.{name}", registration, kv_caches[name]))
        self._table = self.world.exchange_regions(regions, tag="vllm_kv")
        self._kv_caches, self._order = dict(kv_caches), order
        self._page_bytes, self._max_blocks = page_bytes, blocks
        per_event = self.target_profile.consumers_per_readiness
        self._groups = [order[i:i + per_event] for i in range(0, len(order), per_event)]
        self._ready = torch.zeros(len(self._groups), dtype=torch.int64, device=self.world.torch_device)
        self._plan = compile_kv_cache_migration(
            KVCacheMigrationSpec(max_pages=blocks, page_bytes=page_bytes, num_ranks=2,
                                 max_consumers=len(order), consumer_asynchronous=True),
            layout_contract=KVCacheLayoutContract(consumer_ordered=consumer_order is not None),
            target_profile=self.target_profile, rank=self.rank)

    # -- transfers -------------------------------------------------------------------------------
    def pull_blocks(self, *, local_block_ids: list[int], remote_block_ids: list[int],
                    remote_rank: int) -> float:
        started = time.perf_counter()
        self.start_pull_blocks(local_block_ids=local_block_ids, remote_block_ids=remote_block_ids,
                               remote_rank=remote_rank).synchronize()
        self._last_transfer_us = (time.perf_counter() - started) * 1e6
        self.check()
        if self.profile_transfers:
            print(f"aboleth_kv_transfer=physicalization={self.last_physicalization} "
                  f"pages={len(local_block_ids)} bytes={self._last_transfer_bytes} "
                  f"us={self._last_transfer_us:.1f}", flush=True)
        return self._last_transfer_us

    def start_pull_blocks(self, *, local_block_ids: list[int], remote_block_ids: list[int],
                          remote_rank: int) -> torch.cuda.Event:
        return self._start(local_block_ids, remote_block_ids, remote_rank, layered=False).completion

    def start_layered_pull_blocks(self, *, local_block_ids: list[int], remote_block_ids: list[int],
                                  remote_rank: int) -> KVCachePullTicket:
        return self._start(local_block_ids, remote_block_ids, remote_rank, layered=True)

    def _start(self, local_ids, remote_ids, remote_rank: int, *, layered: bool) -> KVCachePullTicket:
        plan = self.plan
        if remote_rank == self.rank or not 0 <= remote_rank < self.world_size:
            raise ValueError("remote_rank must be the other rank")
        if len(local_ids) != len(remote_ids):
            raise ValueError("local and remote block lists differ in length")
        if any(not 0 <= b < self._max_blocks for b in list(local_ids) + list(remote_ids)):
            raise ValueError("block id outside the registered cache")
        runs = kvcopy.canonicalize_block_runs(remote_ids, local_ids)   # (remote start, local start, pages)
        total = len(local_ids) * self._page_bytes * len(self._order)
        engine = plan.select_transfer_engine(transfer_bytes=total, run_count=len(runs) * len(self._order))
        self._last_physicalization = f"{plan.physicalization.name}/{engine}"
        self._last_transfer_bytes, self._last_run_count = total, len(runs)
        self._epoch += 1
        events: dict[str, torch.cuda.Event] = {}
        stream = torch.cuda.current_stream()
        for index, group in enumerate(self._groups):
            if engine == "copy_engine":
                for name in group:
                    remote = int(self._table.addresses(f"kv.{name}")[remote_rank])
                    local = self._kv_caches[name].data_ptr()
                    for r, l, n in runs:
                        kvcopy.cuda_memcpy_async(local + l * self._page_bytes, remote + r * self._page_bytes,
                                                 n * self._page_bytes, stream.cuda_stream)
            else:
                cell = self._ready[index:index + 1].data_ptr()
                batches = []
                for name in group:
                    remote = int(self._table.addresses(f"kv.{name}")[remote_rank])
                    local = self._kv_caches[name].data_ptr()
                    batches += [(remote + r * self._page_bytes, local + l * self._page_bytes,
                                 n * self._page_bytes, cell) for r, l, n in runs]
                if len(batches) > self._arrivals.numel():
                    self._arrivals = torch.zeros(len(batches), dtype=torch.int32, device=self.world.torch_device)
                # Every batch of the group publishes the group's cell: one shared arrival counter.
                workers = plan.physicalization.generated_copy_workers
                group_of, group_target, _ = kvcopy.pack_groups([b[3] for b in batches], workers,
                                                               self.world.torch_device)
                kvcopy.push(kvcopy.pack_batches(batches, self.world.torch_device), self._arrivals,
                            len(batches), self._epoch, workers=workers,
                            threads=self.target_profile.threads, status=self._status,
                            group_of=group_of, group_target=group_target)
            if layered:
                event = torch.cuda.Event()
                event.record(stream)
                for name in group:
                    events[name] = event
        completion = torch.cuda.Event()
        completion.record(stream)
        return KVCachePullTicket(completion, events)

    def check(self) -> None:
        status = self._status.tolist()
        if status[0]:
            raise RuntimeError(f"KV migration transport status {status[0]} (detail {status[1]:#x})")

    def close(self) -> None:
        if self._table is not None:
            self._table.close()
            self._table = None
        for registration in reversed(self._registrations):
            registration.close()
        self._registrations.clear()
        self._kv_caches.clear()
        if self._owns_world:
            self.world.close()
