"""Compile-time plan of one MoE layer's communication: the region graph, what the
planners decide about it, and the facts the executor binds to.

``compile_moe_plan`` builds the dataflow the reference describes
(python/aboleth/moe/compiled_plan.py:124-291: pack -> dispatch.{payload,metadata,count} ->
unpack -> experts (opaque) -> copy -> return.{payload,metadata,count} -> gather), runs the
native planners over it and records the outcome: returned metadata and counts are dead
communication, the expert output is forwarded into the donated return source, the
received payload shrinks to the rows that are reached, and token inputs are borrowed in
place.  The fused kernels implement exactly the surviving graph.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

from ..endpoint_profiles import SEED_PROFILES, EndpointProfile
from ..planning import (CommunicationDataflow, CommunicationRegion, RegionEffect, TransportPhase,
                        plan_endpoint_work, plan_storage, plan_transport,
                        simplify_communication_dataflow)
from .spec import MoESpec


@dataclass(frozen=True)
class CompiledMoEPlan:
    spec: MoESpec
    dataflow: object
    storage: dict
    transport: dict
    dispatch_launches: tuple
    return_launches: tuple
    forwarded_expert_output: bool
    removed_transfers: tuple[str, ...]
    profile_max_lanes: tuple = ()       # (backend, lanes the matched endpoint profile allows), per partition

    def manifest(self) -> dict:
        s = self.spec
        return {"capacity": s.capacity, "metadata_words": s.metadata_words,
                "received_rows": self.storage["received_payload"]["physical_rows"],
                "prefix_bound_inputs": [n for n, r in self.storage.items() if r["prefix_binding"]],
                "removed": list(self.removed_transfers),
                "forwarded_expert_output": self.forwarded_expert_output,
                "dispatch_lanes": [l.lanes for l in self.dispatch_launches],
                "return_lanes": [l.lanes for l in self.return_launches],
                "phases": {p["name"]: {"completion_interval": p["completion_interval"],
                                       "publication_mode": p["publication_mode"]}
                           for p in self.transport["phases"]}}


def build_dataflow(spec: MoESpec) -> CommunicationDataflow:
    s, rb = spec, spec.ranks * spec.capacity
    d = CommunicationDataflow()
    d.region("tokens", s.capacity, s.hidden * 2, immutable=True, valid_count="num_tokens")
    d.region("send_payload", rb, s.row_bytes, registered=True)
    d.region("send_metadata", rb, s.metadata_words * 4, registered=True)
    d.region("send_counts", s.ranks, 8, registered=True)
    d.region("received_payload", rb * s.top_k, s.row_bytes, registered=True)
    d.region("received_metadata", rb, s.metadata_words * 4, registered=True)
    d.region("received_counts", s.ranks, 8, registered=True)
    d.region("expert_output", rb, s.hidden * 2)
    d.region("return_source", rb, s.hidden * 2, registered=True, donated=True)
    d.region("returned_payload", rb, s.hidden * 2, registered=True)
    d.region("returned_metadata", rb, s.metadata_words * 4, registered=True)
    d.region("returned_counts", s.ranks, 8, registered=True)
    d.region("final_output", s.capacity, s.hidden * 2, escapes=True)
    d.opaque_stage("pack", ["tokens"], "send_payload")
    d.transfer("dispatch.payload", "send_payload", "received_payload")
    d.transfer("dispatch.metadata", "send_metadata", "received_metadata")
    d.transfer("dispatch.count", "send_counts", "received_counts")
    d.opaque_stage("experts", ["received_payload", "received_metadata", "received_counts"],
                   "expert_output", bindable_outputs=True)
    d.copy("expert_copy", "expert_output", "return_source")
    d.transfer("return.payload", "return_source", "returned_payload")
    d.transfer("return.metadata", "received_metadata", "returned_metadata")
    d.transfer("return.count", "received_counts", "returned_counts")
    d.transform("gather", "returned_payload", "final_output")
    return d


def compile_moe_plan(spec: MoESpec, world=None, *, profiles: Optional[dict[str, EndpointProfile]] = None,
                     available_lanes: int = 16) -> CompiledMoEPlan:
    dataflow = simplify_communication_dataflow(build_dataflow(spec))
    s, rb = spec, spec.ranks * spec.capacity
    regions = [
        CommunicationRegion("tokens", s.capacity, s.hidden * 2, immutable=True, valid_count="num_tokens"),
        CommunicationRegion("received_payload", rb * s.top_k, s.row_bytes, registered=True),
        CommunicationRegion("returned_payload", rb, s.hidden * 2, registered=True),
        CommunicationRegion("final_output", s.capacity, s.hidden * 2, escapes=True),
    ]
    effects = [
        RegionEffect("tokens", "read", "pack", (0, s.capacity), prefix=True),
        # Records are rank-deduplicated: one row per (token, destination), not per choice.
        RegionEffect("received_payload", "write", "dispatch", (0, rb)),
        RegionEffect("received_payload", "read", "experts", (0, rb * s.top_k), through=rb),
        RegionEffect("returned_payload", "write", "return", (0, rb)),
        RegionEffect("returned_payload", "read", "gather", (0, rb)),
    ]
    storage = plan_storage(regions, effects)
    peers = {r: "p2p" for r in range(s.ranks)}
    if world is not None and world.peer_transports:
        peers = {p: (t.value if t.value in ("p2p", "rdma", "efa", "ionic") else "proxy")
                 for p, t in world.peer_transports.items()}
    transport = plan_transport(peers, [
        TransportPhase("dispatch", next(iter(peers.values()), "p2p"), commands=3, reuse=1,
                       payload_bytes=min(s.capacity * s.row_bytes, 2 ** 31 - 1),
                       completion_before="next_pack", publication_before="experts"),
        TransportPhase("combine", next(iter(peers.values()), "p2p"), commands=1, reuse=1,
                       payload_bytes=min(s.capacity * s.hidden * 2, 2 ** 31 - 1),
                       completion_before="next_pack", publication_before="next_pack"),
    ])
    profiles = profiles or {"p2p": SEED_PROFILES["B200_NV18"], "proxy": SEED_PROFILES["B200_HOSTRING"]}
    partitions = []
    for part in transport["launch_partitions"]:
        backend = part["backend"]
        partitions.append(dict(backend=backend, peers=part["peers"], platform="B200",
                               queueMemory="none" if backend == "p2p" else "host",
                               peerLink="NV18" if backend == "p2p" else "",
                               availableLanes=available_lanes,
                               participantLanes=[available_lanes] * s.ranks,
                               participantLinks=["NV18" if backend == "p2p" else ""] * len(part["peers"])))
    launches = {}
    for phase, row in (("dispatch", s.row_bytes + s.metadata_words * 4), ("return", s.hidden * 2)):
        launches[phase] = tuple(plan_endpoint_work(
            phase, payload_bytes=s.capacity * row, max_items=s.capacity, partitions=partitions,
            profiles=profiles.values(), rank_count=s.ranks)) if partitions else ()
    removed = tuple(r["name"] for r in dataflow.removed)
    limits = tuple((p.backend, min(p.max_lanes, available_lanes)) for p in profiles.values())
    return CompiledMoEPlan(spec, dataflow, storage, transport, launches["dispatch"], launches["return"],
                           forwarded_expert_output="expert_copy" in removed, removed_transfers=removed,
                           profile_max_lanes=limits)
