"""Patterns: a communication dataflow plus the client kernels (opaque stages) around it.

A ``Pattern`` is declared once (regions, views, worksets, transfers, copies, reductions,
opaque compute stages); ``compile()`` runs the dataflow simplification and returns a
``CompiledPattern`` whose ``compile_plan(resources)`` runs the storage, endpoint and
transport planners and selects, per phase, how it is realised:

* strategy ``inline_transport`` (payload below 4 KiB: the transfer rides inside the
  producing kernel), ``direct_destination`` (the producer writes the peer's memory directly)
  or ``parallel_copy`` (a copy kernel with lanes moves it);
* publication ``inline`` (the same kernel publishes), ``fused_kernel``, ``separate_kernel``,
  ``coalesced_kernel`` (one kernel publishes several phases), ``consumer_prologue`` or
  ``packed_doorbell`` (queue transports).

Reference: python/aboleth/pattern.py:224-626,628-873,887-1161,1164-1393,1396-2122.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Mapping, Optional, Sequence

from .endpoint_profiles import SEED_PROFILES, EndpointProfile
from .planning import (CommunicationDataflow, CommunicationRegion, RegionEffect,
                       SimplifiedCommunicationDataflow, TransportPhase, plan_endpoint_work, plan_storage,
                       plan_transport, simplify_communication_dataflow)

INLINE_TRANSPORT_BYTES = 4096
STRATEGIES = ("inline_transport", "direct_destination", "parallel_copy")
PUBLICATIONS = ("inline", "separate_kernel", "coalesced_kernel", "consumer_prologue", "packed_doorbell",
                "fused_kernel")


@dataclass(frozen=True)
class CommunicationStage:
    name: str
    reads: tuple[str, ...]
    writes: tuple[str, ...]


@dataclass(frozen=True)
class OpaqueCapabilities:
    accepts_destination_rewrite: bool = False
    grouped_receiver: bool = True
    graph_capturable: bool = True


@dataclass(frozen=True)
class OpaqueStage(CommunicationStage):
    capabilities: OpaqueCapabilities = OpaqueCapabilities()


@dataclass(frozen=True)
class Workset:
    """An unordered domain of records (e.g. rows of a per-peer segment)."""

    name: str
    region: str
    max_items: int
    item_bytes: int

    def field(self, name: str) -> str:
        return f"{self.name}.{name}"


@dataclass(frozen=True)
class KernelBinding:
    operation: str
    kernel: str
    arguments: tuple[str, ...] = ()

    def __post_init__(self):
        if not self.operation or not self.kernel:
            raise ValueError("a kernel binding names an operation and a kernel")


@dataclass(frozen=True)
class P2PRealizationProfile:
    """Client-owned kernels for the realisations the planner may select on peer memory."""

    direct_destination_kernel: str
    direct_publication_kernels: tuple[tuple[str, Optional[str]], ...]
    parallel_copy_kernel: str
    parallel_publication_kernels: tuple[tuple[str, Optional[str]], ...]

    def __post_init__(self):
        if not self.direct_destination_kernel or not self.parallel_copy_kernel:
            raise ValueError("P2P realization kernels cannot be empty")
        for mappings in (self.direct_publication_kernels, self.parallel_publication_kernels):
            names = [s for s, _ in mappings]
            if len(set(names)) != len(names) or any(not s for s in names):
                raise ValueError("P2P publication strategies must be unique and nonempty")

    def direct_publication_kernel(self, strategy: str) -> Optional[str]:
        return dict(self.direct_publication_kernels)[strategy]

    def parallel_publication_kernel(self, strategy: str) -> Optional[str]:
        return dict(self.parallel_publication_kernels)[strategy]


@dataclass(frozen=True)
class PhaseResources:
    """Runtime facts a plan is compiled against."""

    peers: Mapping[int, str]                      # rank -> transport name
    available_lanes: int = 16
    platform: str = "B200"
    profiles: Mapping[str, EndpointProfile] = field(default_factory=lambda: {
        "p2p": SEED_PROFILES["B200_NV18"], "proxy": SEED_PROFILES["B200_HOSTRING"]})
    queue_capacity: int = 0
    buffer_depth: int = 1
    realization: Optional[P2PRealizationProfile] = None
    # What the client's kernels can do; the schedule of every phase is chosen from these
    # (reference: python/aboleth/pattern.py:628-790 ``PhaseResources``, 887-1079 selection).
    direct_destination: bool = True            # an indexed transfer may write the final storage
    fused_publication: bool = True             # the moving kernel can publish (last worker releases)
    packed_doorbell: bool = False              # count and epoch travel in one 8-byte release store
    coalesce_publication_wait: bool = True     # one kernel may publish and wait for several phases
    coalesce_return_with_consumer: bool = False  # the consumer's prologue may publish and wait
    consumer_grid_size: int = 0                # CTAs of that consumer (it needs one per peer)
    iteration_count: int = 1                   # steps the plan is unrolled over (1: not cyclic)
    parallel_threshold_bytes: int = 4096       # at or below this a phase rides in its producer

    def __post_init__(self):
        if self.available_lanes < 1 or self.buffer_depth < 1:
            raise ValueError("lanes and buffer depth must be positive")
        if self.iteration_count < 1 or self.parallel_threshold_bytes < 0 or self.consumer_grid_size < 0:
            raise ValueError("iteration count, threshold and consumer grid cannot be negative or zero-step")


@dataclass(frozen=True)
class PhaseSchedule:
    name: str
    strategy: str
    kernel: str
    publication_kernel: Optional[str]
    publication_strategy: str
    recycled_buffers: tuple[str, ...]
    advanced_values: tuple[str, ...]
    grid_axes: tuple[str, ...]
    payload_bytes: int
    block_elements: int
    num_warps: int
    buffer_depth: int
    rationale: str
    p2p_coop_elements: Optional[int] = None

    def __post_init__(self):
        if self.strategy not in STRATEGIES:
            raise ValueError(f"unknown phase strategy {self.strategy!r}")
        if self.publication_strategy not in PUBLICATIONS:
            raise ValueError(f"unknown publication strategy {self.publication_strategy!r}")
        for names in (self.recycled_buffers, self.advanced_values):
            if len(set(names)) != len(names) or any(not n for n in names):
                raise ValueError("phase buffer and value names must be unique and nonempty")
        if self.payload_bytes < 0 or self.block_elements < 0:
            raise ValueError("phase payload and block size cannot be negative")
        if self.num_warps <= 0 or self.buffer_depth <= 0:
            raise ValueError("phase warp count and buffer depth must be positive")
        if not self.kernel or not self.grid_axes:
            raise ValueError("phase schedule requires a kernel and launch grid")
        e = self.p2p_coop_elements
        if e is not None and (e < 32 or e > 4096 or e & (e - 1)):
            raise ValueError("p2p_coop_elements must be a power of two in [32, 4096]")


@dataclass(frozen=True)
class RegionRequirement:
    name: str
    element_type: str
    shape: tuple[int, ...]
    strides: tuple[int, ...]


def _publication_for(profile_lookup, preferred: tuple[str, ...]) -> tuple[str, Optional[str]]:
    """The first preferred publication strategy the client's kernels realise, with its kernel."""
    for strategy in preferred:
        try:
            return strategy, profile_lookup(strategy)
        except KeyError:
            continue
    raise ValueError(f"the realisation profile offers none of the publication strategies {preferred}")


def _select_schedule(name: str, payload_bytes: int, backend: str, lanes: int, warps: int,
                     resources: PhaseResources, buffers: tuple[str, ...], *, per_item: bool = False,
                     retargeted: bool = False) -> PhaseSchedule:
    """How one phase is carried out.

    ``per_item``: the phase moves indexed items (a workset), not one contiguous span.
    ``retargeted``: the dataflow simplifier proved that the transfer may write the final storage.

    Movement: a payload up to the threshold rides inside the kernel that produced it; an indexed
    transfer with a legal direct destination is written in place by one kernel over the items;
    anything else is a lane-parallel copy.  Publication, in order of preference and subject to
    what the client's kernels offer: the moving kernel publishes itself (``fused_kernel``); count
    and epoch share one release store (``packed_doorbell``); the consumer's prologue publishes and
    waits (``consumer_prologue``: two ranks, a consumer grid that covers the peers); one kernel
    publishes and waits for several phases (``coalesced_kernel``); or a kernel of its own
    (``separate_kernel``).  Queue transports publish with their doorbell.
    """
    peer_memory = backend == "p2p"
    profile = resources.realization
    publication_kernel: Optional[str] = None
    grid_axes: tuple[str, ...] = ("peers", "lanes")
    if payload_bytes <= resources.parallel_threshold_bytes:
        strategy, publication = "inline_transport", "inline"
        kernel = f"{name}.producer"
        grid_axes = ("peers",)
        why = f"{payload_bytes} B <= {resources.parallel_threshold_bytes} B: the producing kernel carries it"
    elif not peer_memory:
        strategy, publication = "parallel_copy", "packed_doorbell"
        kernel = profile.parallel_copy_kernel if profile else f"{name}.copy"
        why = f"{lanes} lanes post {payload_bytes} B to a queue; one doorbell per packed batch"
    elif per_item and retargeted and resources.direct_destination:
        strategy = "direct_destination"
        kernel = profile.direct_destination_kernel if profile else f"{name}.direct"
        grid_axes = ("items",)
        preferred = (("packed_doorbell",) if resources.packed_doorbell else ()) + \
            (("fused_kernel",) if resources.fused_publication else ()) + \
            (("coalesced_kernel", "separate_kernel") if resources.coalesce_publication_wait
             else ("separate_kernel", "coalesced_kernel"))
        if profile:
            publication, publication_kernel = _publication_for(profile.direct_publication_kernel, preferred)
        else:
            publication = preferred[0]
        why = ("indexed items with unique destinations: written into the final storage in place; "
               f"published by {publication.replace('_', ' ')}")
    else:
        strategy = "parallel_copy"
        kernel = profile.parallel_copy_kernel if profile else f"{name}.copy"
        prologue = (not per_item and resources.coalesce_return_with_consumer and len(resources.peers) == 1
                    and resources.consumer_grid_size >= max(len(resources.peers), 1))
        preferred = (("fused_kernel",) if resources.fused_publication else ()) + \
            (("consumer_prologue",) if prologue else ()) + \
            (("coalesced_kernel", "separate_kernel") if resources.coalesce_publication_wait
             else ("separate_kernel", "coalesced_kernel"))
        if profile:
            publication, publication_kernel = _publication_for(profile.parallel_publication_kernel, preferred)
        else:
            publication = preferred[0]
        shape = "indexed items staged through a copy" if per_item else "one contiguous span per peer"
        why = f"{lanes} lanes move {payload_bytes} B ({shape}); published by {publication.replace('_', ' ')}"
    coop = None
    if peer_memory and strategy != "inline_transport":
        per_lane = max(payload_bytes // max(lanes, 1), 256)
        coop = 32
        while coop < 4096 and coop * 8 < per_lane:
            coop *= 2
    depth = resources.buffer_depth
    if strategy == "parallel_copy" and not per_item and resources.iteration_count > 1:
        depth = max(depth, 2)   # a cyclic plan refills one buffer while the other is read
    return PhaseSchedule(name=name, strategy=strategy, kernel=kernel, publication_kernel=publication_kernel,
                         publication_strategy=publication, recycled_buffers=buffers,
                         advanced_values=("epoch",), grid_axes=grid_axes,
                         payload_bytes=payload_bytes, block_elements=coop or 0, num_warps=warps,
                         buffer_depth=depth, rationale=why, p2p_coop_elements=coop)


@dataclass(frozen=True)
class CompiledPatternPlan:
    name: str
    dataflow: SimplifiedCommunicationDataflow
    storage: Mapping[str, dict]
    transport: dict
    launches: Mapping[str, tuple]
    schedules: Mapping[str, PhaseSchedule]
    bindings: tuple[KernelBinding, ...]

    def binding(self, operation: str) -> KernelBinding:
        for b in self.bindings:
            if b.operation == operation:
                return b
        raise KeyError(f"no kernel is bound to {operation!r}")

    def completion_interval_for(self, phase: str) -> int:
        for p in self.transport["phases"]:
            if p["name"] == phase:
                return p["completion_interval"]
        raise KeyError(phase)

    def phase_schedule(self, name: str) -> PhaseSchedule:
        return self.schedules[name]

    def to_dict(self) -> dict:
        return {"name": self.name, "operations": list(self.dataflow.operations),
                "removed": list(self.dataflow.removed), "storage": dict(self.storage),
                "transport": self.transport,
                "schedules": {k: vars(v) for k, v in self.schedules.items()},
                "launches": {k: [vars(l) for l in v] for k, v in self.launches.items()}}


@dataclass
class CompiledPattern:
    name: str
    dataflow: SimplifiedCommunicationDataflow
    regions: tuple[CommunicationRegion, ...]
    effects: tuple[RegionEffect, ...]
    stages: tuple[OpaqueStage, ...]
    worksets: tuple[Workset, ...]
    bindings: tuple[KernelBinding, ...] = ()

    def opaque_stage(self, name: str) -> OpaqueStage:
        for s in self.stages:
            if s.name == name:
                return s
        raise KeyError(f"unknown opaque stage {name!r}")

    def binding(self, operation: str) -> KernelBinding:
        for b in self.bindings:
            if b.operation == operation:
                return b
        raise KeyError(operation)

    def capabilities(self, stage: str) -> OpaqueCapabilities:
        return self.opaque_stage(stage).capabilities

    def transport_operations(self) -> tuple[dict, ...]:
        return tuple(op for op in self.dataflow.operations if op["kind"] == "transfer")

    def compile_plan(self, resources: PhaseResources) -> CompiledPatternPlan:
        storage = plan_storage(self.regions, self.effects)
        by_region = {r.name: r for r in self.regions}
        phases, launches, schedules = [], {}, {}
        backends = sorted(set(resources.peers.values())) or ["p2p"]
        partitions = []
        for backend in backends:
            peers = [p for p, b in sorted(resources.peers.items()) if b == backend]
            partitions.append(dict(backend=backend, peers=peers, platform=resources.platform,
                                   queueMemory="none" if backend == "p2p" else "host",
                                   peerLink="NV18" if backend == "p2p" else "",
                                   availableLanes=resources.available_lanes,
                                   participantLanes=[resources.available_lanes] * (len(resources.peers) + 1),
                                   participantLinks=["NV18" if backend == "p2p" else ""] * len(peers)))
        worksets = {w.region: w for w in self.worksets}
        for op in self.transport_operations():
            src = by_region.get(op["src"])
            rows = storage.get(op["src"], {}).get("physical_rows", src.rows if src else 0)
            payload = rows * (src.row_bytes if src else 0)
            workset = worksets.get(op["src"])
            max_items = workset.max_items if workset else max(rows, 1)
            plans = tuple(plan_endpoint_work(op["name"], payload_bytes=payload, max_items=max_items,
                                             partitions=partitions, profiles=resources.profiles.values()))
            launches[op["name"]] = plans
            lanes = max((l.lanes for l in plans), default=1)
            warps = max((l.sender_warps for l in plans), default=1)
            phases.append(TransportPhase(op["name"].replace(".", "_"), backends[0], commands=1,
                                         reuse=resources.buffer_depth, buffer_slots=resources.buffer_depth,
                                         queue_capacity=resources.queue_capacity, lanes=lanes,
                                         payload_bytes=min(payload, 2 ** 31 - 1)))
            retargeted = any(op["dst"] in str(r.get("why", "")) and "forwarded" in str(r.get("why", ""))
                             for r in self.dataflow.removed)
            schedules[op["name"]] = _select_schedule(op["name"], payload, backends[0], lanes, warps,
                                                     resources, (op["dst"],), per_item=workset is not None,
                                                     retargeted=retargeted)
        transport = plan_transport(dict(resources.peers), phases)
        return CompiledPatternPlan(self.name, self.dataflow, storage, transport, launches, schedules,
                                   self.bindings)


class Pattern(CommunicationDataflow):
    """Builder: declare regions and what moves between them, then ``compile()``."""

    def __init__(self, name: str):
        super().__init__()
        self.name = name
        self._effects: list[RegionEffect] = []
        self._stages: list[OpaqueStage] = []
        self._worksets: list[Workset] = []
        self._bindings: list[KernelBinding] = []

    def workset(self, name: str, region: str, *, max_items: int, item_bytes: int) -> Workset:
        ws = Workset(name, region, max_items, item_bytes)
        self._worksets.append(ws)
        return ws

    def reads(self, region: str, stage: str, rows: tuple[int, int], *, prefix: bool = False,
              through: Optional[int] = None) -> None:
        self._effects.append(RegionEffect(region, "read", stage, rows, prefix, through))

    def writes(self, region: str, stage: str, rows: tuple[int, int]) -> None:
        self._effects.append(RegionEffect(region, "write", stage, rows))

    def transfer_each(self, name: str, workset: Workset, dst: str) -> str:
        """Transfer every record of a workset (unordered, sliceable across lanes)."""
        return self.transfer(name, workset.region, dst)

    def copy_each(self, name: str, workset: Workset, dst: str) -> str:
        return self.copy(name, workset.region, dst)

    def copy_each_from(self, name: str, src: str, dst: str) -> str:
        """Copy every received record of ``src`` into ``dst`` (the materialising copy after a transfer)."""
        return self.copy(name, src, dst)

    def opaque_compute(self, name: str, reads: Sequence[str], writes: str, *,
                       capabilities: OpaqueCapabilities = OpaqueCapabilities(),
                       kernel: Optional[str] = None) -> str:
        self._stages.append(OpaqueStage(name, tuple(reads), (writes,), capabilities))
        if kernel:
            self._bindings.append(KernelBinding(name, kernel))
        return self.opaque_stage(name, reads, writes,
                                 bindable_outputs=capabilities.accepts_destination_rewrite)

    def bind(self, operation: str, kernel: str, *arguments: str) -> None:
        self._bindings.append(KernelBinding(operation, kernel, tuple(arguments)))

    def analyze(self) -> SimplifiedCommunicationDataflow:
        return simplify_communication_dataflow(self)

    def compile(self) -> CompiledPattern:
        return CompiledPattern(self.name, self.analyze(), tuple(self.regions), tuple(self._effects),
                               tuple(self._stages), tuple(self._worksets), tuple(self._bindings))
