"""Requests to the native planning passes and typed views of their answers.

``plan_endpoint_work``       lanes, row slices, grids and readiness stride per backend partition
``plan_storage``             reached rows, physical shapes, prefix bindings
``plan_transport``           launch partitions, completion intervals, publication modes, plan blobs
``simplify_communication_dataflow``  dead communication, forwarded copies, aliases

Reference: python/aboleth/planning.py:13-190,236-420,532-1094,1882-2113 and the C++ passes it drives.
The arithmetic lives in csrc/spec/planning.cpp.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Iterable, Mapping, Optional, Sequence

from .compiler.driver import run_planner
from .compiler.options import current_options
from .endpoint_profiles import EndpointProfile


def _enable() -> str:
    return ",".join(sorted(current_options().passes)) or "none"


@dataclass(frozen=True)
class RegionEffect:
    """One stage's access to a region: rows ``[begin, end)``, read or write."""

    region: str
    kind: str                      # "read" | "write"
    stage: str
    rows: tuple[int, int]
    prefix: bool = False           # reads only the valid prefix
    through: Optional[int] = None  # bounded by an indexed view of this many rows


@dataclass(frozen=True)
class CommunicationRegion:
    name: str
    rows: int
    row_bytes: int
    escapes: bool = False
    immutable: bool = False
    registered: bool = False
    donated: bool = False
    valid_count: Optional[str] = None
    max_inflight: int = 1


@dataclass
class LaunchPlan:
    backend: str
    peers: tuple[int, ...]
    lanes: int
    slices: tuple[tuple[int, int], ...]
    slice_quotient: int
    slice_remainder: int
    count_lane: int
    signal_slots: int
    sender_grid: tuple[int, int]
    receiver_grid: tuple[int, int]
    receiver_lanes_per_program: int
    sender_warps: int
    ready_stride: int
    profile_identity: str


def plan_endpoint_work(name: str, *, payload_bytes: int, max_items: int,
                       partitions: Sequence[Mapping], profiles: Iterable[EndpointProfile],
                       rank_count: Optional[int] = None,
                       grouped_receiver: bool = True) -> list[LaunchPlan]:
    """``partitions``: dicts with backend, peers, platform, queueMemory, peerLink, availableLanes
    (and participantLanes / participantLinks lists when every rank's facts are known)."""
    lines = [f"program plan enable={_enable()}",
             f"endpoint_work name={name} payload_bytes={payload_bytes} max_items={max_items} "
             f"grouped_receiver={int(grouped_receiver)}" +
             (f" rank_count={rank_count}" if rank_count is not None else "") + " {"]
    for part in partitions:
        attrs = " ".join(f"{k}={','.join(map(str, v)) if isinstance(v, (list, tuple)) else v}"
                         for k, v in part.items())
        lines.append(f"  partition {attrs}")
    for profile in profiles:
        lines.append("  profile " + profile.to_request())
    lines.append("}")
    program = run_planner("plan-endpoints", "\n".join(lines) + "\n")["programs"][0]
    return [LaunchPlan(
        backend=l["backend"], peers=tuple(l["peers"]), lanes=l["lanes"],
        slices=tuple(tuple(s) for s in l["slices"]), slice_quotient=l["slice_quotient"],
        slice_remainder=l["slice_remainder"], count_lane=l["count_lane"],
        signal_slots=l["signal_slots"], sender_grid=tuple(l["sender_grid"]),
        receiver_grid=tuple(l["receiver_grid"]),
        receiver_lanes_per_program=l["receiver_lanes_per_program"], sender_warps=l["sender_warps"],
        ready_stride=l["ready_stride"], profile_identity=l["profile_identity"])
        for l in program["launches"]]


def plan_storage(regions: Sequence[CommunicationRegion], effects: Sequence[RegionEffect]) -> dict[str, dict]:
    lines = [f"program plan enable={_enable()}"]
    for region in regions:
        head = (f"region name={region.name} rows={region.rows} row_bytes={region.row_bytes} "
                f"escapes={int(region.escapes)} immutable={int(region.immutable)} "
                f"max_inflight={region.max_inflight}")
        if region.valid_count:
            head += f" valid_count={region.valid_count}"
        lines.append(head + " {")
        for e in effects:
            if e.region != region.name:
                continue
            text = f"  access kind={e.kind} stage={e.stage} rows={e.rows[0]}:{e.rows[1]} prefix={int(e.prefix)}"
            if e.through is not None:
                text += f" through={e.through}"
            lines.append(text)
        lines.append("}")
    return {r["name"]: r for r in run_planner("plan-storage", "\n".join(lines) + "\n")["regions"]}


@dataclass(frozen=True)
class TransportPhase:
    name: str
    backend: str = "p2p"
    commands: int = 1
    reuse: Optional[int] = None
    buffer_slots: int = 1
    queue_capacity: int = 0
    lanes: int = 1
    payload_bytes: int = 0
    completion_before: str = ""
    publication_before: str = ""
    first_overwrite: str = ""
    policy_interval: Optional[int] = None
    strict_registrations: bool = False
    exclusive: bool = False
    # Program-level planning (plan_transport_program): what the phase reads and writes per
    # iteration, and the queues it goes through.
    iterations: int = 1
    peer_transports: tuple[str, ...] = ()
    peer_capacities: tuple[int, ...] = ()
    completion_intervals: tuple[int, ...] = ()
    explicit_interval: Optional[int] = None
    tiny_payload_bytes: int = 4096
    reads: tuple["RegionAccess", ...] = ()
    writes: tuple["RegionAccess", ...] = ()


def plan_transport(peers: Mapping[int, str], phases: Sequence[TransportPhase]) -> dict:
    """``peers``: rank -> transport name.  Returns launch partitions and one plan per phase
    (with the 112-byte ``TransportPhasePlan`` as hex in ``plan_blob``)."""
    lines = [f"program plan enable={_enable()}"]
    for rank, backend in sorted(peers.items()):
        lines.append(f"peer rank={rank} backend={backend}")
    for ph in phases:
        text = (f"phase name={ph.name} backend={ph.backend} commands={ph.commands} "
                f"buffer_slots={ph.buffer_slots} queue_capacity={ph.queue_capacity} lanes={ph.lanes} "
                f"payload_bytes={ph.payload_bytes} strict_registrations={int(ph.strict_registrations)} "
                f"exclusive={int(ph.exclusive)}")
        if ph.reuse is not None:
            text += f" reuse={ph.reuse}"
        if ph.policy_interval is not None:
            text += f" policy_interval={ph.policy_interval}"
        for key in ("completion_before", "publication_before", "first_overwrite"):
            if getattr(ph, key):
                text += f" {key}={getattr(ph, key)}"
        lines.append(text)
    return run_planner("plan-transport", "\n".join(lines) + "\n")


def plan_transport_partitions(peers: Mapping[int, str]) -> list[dict]:
    return plan_transport(peers, [])["launch_partitions"]


@dataclass
class CommunicationDataflow:
    """A graph of regions and the transfers, copies, reductions and uses between them."""

    regions: list[CommunicationRegion] = field(default_factory=list)
    operations: list[dict] = field(default_factory=list)

    def region(self, name: str, rows: int, row_bytes: int, **flags) -> str:
        self.regions.append(CommunicationRegion(name, rows, row_bytes, **flags))
        return name

    def _op(self, kind: str, name: str, **attrs) -> str:
        self.operations.append({"kind": kind, "name": name, **attrs})
        return name

    def transfer(self, name: str, src: str, dst: str) -> str:
        return self._op("transfer", name, src=src, dst=dst)

    def copy(self, name: str, src: str, dst: str) -> str:
        return self._op("copy", name, src=src, dst=dst)

    def reduction(self, name: str, src: Sequence[str], dst: str) -> str:
        return self._op("reduction", name, src=",".join(src), dst=dst)

    def transform(self, name: str, src: str, dst: str) -> str:
        return self._op("transform", name, src=src, dst=dst)

    def opaque_stage(self, name: str, reads: Sequence[str], writes: str, *, bindable_outputs: bool = False) -> str:
        return self._op("opaque_stage", name, reads=",".join(reads), writes=writes,
                        bindable_outputs=int(bindable_outputs))

    def use(self, stage: str, reads: Sequence[str]) -> str:
        return self._op("use", stage, reads=",".join(reads))

    def to_request(self) -> str:
        lines = [f"program dataflow enable={_enable()}"]
        for r in self.regions:
            lines.append(f"region name={r.name} escapes={int(r.escapes)} registered={int(r.registered)} "
                         f"donated={int(r.donated)} immutable={int(r.immutable)}")
        for op in self.operations:
            attrs = " ".join(f"{k}={v}" for k, v in op.items() if k != "kind")
            lines.append(f"{op['kind']} {attrs}")
        return "\n".join(lines) + "\n"


@dataclass(frozen=True)
class SimplifiedCommunicationDataflow:
    operations: tuple[dict, ...]
    removed: tuple[dict, ...]
    aliases: Mapping[str, str]
    unallocated_regions: tuple[str, ...]

    def has(self, name: str) -> bool:
        return any(op.get("name") == name for op in self.operations)


def simplify_communication_dataflow(dataflow: CommunicationDataflow) -> SimplifiedCommunicationDataflow:
    result = run_planner("simplify-dataflow", dataflow.to_request())
    return SimplifiedCommunicationDataflow(tuple(result["operations"]), tuple(result["removed"]),
                                           result["aliases"], tuple(result["unallocated_regions"]))


# ---- program-level transport planning -----------------------------------------------------------

@dataclass(frozen=True)
class RegionAccess:
    """An arithmetic walk over one allocation: iteration ``i`` touches
    ``[offset + (i * stride mod period), + length)``; ``unknown`` overlaps everything."""

    allocation: int
    generation: int = 0
    offset: int = 0
    length: int = 0
    stride: int = 0
    period: int = 0
    count: int = 1
    unknown: bool = False

    def to_request(self, kind: str) -> str:
        return (f"  {kind} allocation={self.allocation} generation={self.generation} offset={self.offset} "
                f"length={self.length} stride={self.stride} period={self.period} count={self.count} "
                f"unknown={int(self.unknown)}")


@dataclass(frozen=True)
class TransportKernel:
    """A compute step between phases.  ``opaque``: the client compiles it, nothing may be placed inside."""

    name: str
    reads: tuple[RegionAccess, ...] = ()
    writes: tuple[RegionAccess, ...] = ()
    asynchronous: bool = False
    max_inflight: int = 1
    event_ordered: bool = False
    opaque: bool = False


@dataclass(frozen=True)
class TransportPlan:
    completion_interval: int
    reuse_distance: int
    completion_before: str
    completion_iteration_delta: int
    publication_before: str
    publication_iteration_delta: int
    requires_final_drain: bool = False


@dataclass(frozen=True)
class OutputLifetimePlan:
    last_consumer: str
    last_consumer_iteration_delta: int
    reuse_before: str
    reuse_iteration_delta: int
    pool_depth: int


def _program_request(operations: Sequence[object], cyclic: bool) -> str:
    lines = [f"program plan cyclic={int(cyclic)} enable={_enable()}"]
    for op in operations:
        if isinstance(op, TransportPhase):
            transports = op.peer_transports or (op.backend,)
            capacities = op.peer_capacities or (op.queue_capacity,) * len(transports)
            head = (f"phase name={op.name} commands={op.commands} iterations={op.iterations} "
                    f"payload_bytes={op.payload_bytes} tiny={op.tiny_payload_bytes} "
                    f"transports={','.join(transports)} capacities={','.join(map(str, capacities))}")
            if op.completion_intervals:
                head += f" intervals={','.join(map(str, op.completion_intervals))}"
            if op.explicit_interval is not None:
                head += f" interval={op.explicit_interval}"
        elif isinstance(op, TransportKernel):
            head = (f"kernel name={op.name} asynchronous={int(op.asynchronous)} max_inflight={op.max_inflight} "
                    f"event_ordered={int(op.event_ordered)} opaque={int(op.opaque)}")
        else:
            raise TypeError("a transport program is made of TransportPhase and TransportKernel")
        lines.append(head + " {")
        lines += [a.to_request("read") for a in op.reads] + [a.to_request("write") for a in op.writes]
        lines.append("}")
    return "\n".join(lines) + "\n"


def plan_transport_facts(operations: Sequence[object], cyclic: bool = False) -> dict:
    """The native planner's facts for one ordered program of phases and kernels (read-only)."""
    return run_planner("plan-transport-program", _program_request(tuple(operations), cyclic))


def plan_transport_program(operations: Sequence[object], cyclic: bool = False) -> dict[str, TransportPlan]:
    facts = plan_transport_facts(operations, cyclic)
    plans = {p["name"]: TransportPlan(p["resolvedCompletionInterval"], p["reuseDistance"],
                                      p["completionBefore"], p["completionIterationDelta"],
                                      p["publicationBefore"], p["publicationIterationDelta"],
                                      p["requiresFinalDrain"]) for p in facts["phases"]}
    expected = {op.name for op in operations if isinstance(op, TransportPhase)}
    if set(plans) != expected:
        raise RuntimeError("transport planner omitted a phase")
    return plans


def plan_output_lifetimes(operations: Sequence[object], cyclic: bool = False) -> dict[str, OutputLifetimePlan]:
    """Kernels whose output buffer may be pooled: last consumer, first overwriter, pool depth."""
    facts = plan_transport_facts(operations, cyclic)
    return {k["name"]: OutputLifetimePlan(k["outputLastConsumer"], k["outputLastConsumerIterationDelta"],
                                          k["outputReuseBefore"], k["outputReuseIterationDelta"],
                                          k["outputPoolDepth"])
            for k in facts["kernels"] if k.get("outputReusable")}


@dataclass(frozen=True)
class CommunicationDataflowOperation:
    """Typed view of one entry of ``CommunicationDataflow.operations``."""

    kind: str
    name: str
    attributes: Mapping[str, object] = field(default_factory=dict)

    @classmethod
    def from_dict(cls, record: Mapping[str, object]) -> "CommunicationDataflowOperation":
        return cls(str(record["kind"]), str(record["name"]),
                   {k: v for k, v in record.items() if k not in ("kind", "name")})
