"""Compile KV-cache page migration: pattern -> plan -> phase(s) + execution contract + physicalisation.

``compile_kv_cache_migration`` decides how many pages ride in one transfer (a power of two,
at most 16, bounded by the pages per consumer and the target batch size), proves that unique
destinations let the transfer write the cache's final storage directly, compiles the phase
(and a one-page fallback phase for batches that are not contiguous runs partitioned by
consumer) and records the choices in a :class:`KVCachePhysicalization`.

Reference: python/aboleth/patterns/kv_cache_transport.py:35-60 (client kernels per
realisation), 62-130 (contracts), 132-260 (plan), 355-545 (compile).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

from ..execution import (CapacityContract, ExecutionContract, ExecutionFallback, PaddingSemantics,
                         RankControl, RuntimeGuard, compile_execution_plan)
from ..kv.profile import GENERIC_KV_TARGET_PROFILE, KVTargetProfile
from ..pattern import P2PRealizationProfile, PhaseResources
from ..phase import CompiledPhase, compile_phase
from .kv_cache import KVCacheMigrationSpec, build_kv_cache_migration_pattern

# The kernels of this library that realise a KV migration on peer memory.  ``kv_push_kernel``
# (csrc/kernels/kv_kernels.cu) both stores page runs into the consumer's final storage and
# publishes the readiness cell from the group's last worker, so "publication in the copy kernel"
# needs no second kernel; a consumer that waits inside its own stream uses ``kv_wait_kernel``; a
# host-driven copy-engine transfer publishes with a packed doorbell (one stream-ordered write).
KV_CACHE_P2P_REALIZATION = P2PRealizationProfile(
    direct_destination_kernel="kv_push_kernel",
    direct_publication_kernels=(("fused_kernel", None),
                                ("consumer_prologue", "kv_wait_kernel"),
                                ("packed_doorbell", None)),
    parallel_copy_kernel="kv_push_kernel",
    parallel_publication_kernels=(("fused_kernel", None),
                                  ("consumer_prologue", "kv_wait_kernel")),
)


@dataclass(frozen=True)
class KVCacheLayoutContract:
    """Promises of the caller about every batch it will submit.  Each one buys something:
    contiguous runs allow several pages per transfer, consumer-partitioned batches allow one
    readiness cell per consumer, consumer-ordered batches allow layer-by-layer readiness, and
    stable addresses allow a fixed-capacity (graph-held) launch."""

    contiguous_page_runs: bool = True
    consumer_partitioned: bool = True
    consumer_ordered: bool = False
    graph_stable_addresses: bool = True


_POSITIVE_FIELDS = ("pages_per_transfer", "slot_count", "generated_copy_workers", "generated_block_elements",
                    "copy_engine_streams", "copy_engine_max_runs", "consumers_per_readiness")
_READINESS_GRANULARITIES = ("rank", "consumer")


@dataclass(frozen=True)
class KVCachePhysicalization:
    """Everything the compiler decided about how pages move; the runtime only reads it."""

    name: str
    target_profile: str
    pages_per_transfer: int
    direct_destination: bool
    readiness: str
    slot_count: int
    target_batch_bytes: int
    generated_copy_workers: int
    generated_block_elements: int
    copy_engine_threshold_bytes: int
    copy_engine_streams: int
    copy_engine_max_runs: int
    asynchronous_completion: bool
    consumer_layer_pipeline: bool
    consumers_per_readiness: int

    def __post_init__(self) -> None:
        problems = [f"{field} is {getattr(self, field)}, it has to be at least 1"
                    for field in _POSITIVE_FIELDS if getattr(self, field) < 1]
        if not self.target_profile:
            problems.append("no target profile is named")
        if self.readiness not in _READINESS_GRANULARITIES:
            problems.append(f"readiness {self.readiness!r} is not one of {_READINESS_GRANULARITIES}")
        if self.copy_engine_threshold_bytes < 0:
            problems.append("the copy-engine threshold is negative")
        if self.consumer_layer_pipeline and self.copy_engine_streams != 1:
            # layers become ready in order only if their copies are issued in order
            problems.append("layer-by-layer readiness needs exactly one copy stream")
        if problems:
            raise ValueError(f"KV physicalisation {self.name!r}: " + "; ".join(problems))


@dataclass(frozen=True)
class CompiledKVCacheMigrationPlan:
    spec: KVCacheMigrationSpec
    phase: CompiledPhase
    fallback_phase: Optional[CompiledPhase]
    execution: dict
    physicalization: KVCachePhysicalization
    layout_contract: KVCacheLayoutContract

    def select_transfer_engine(self, *, transfer_bytes: int, run_count: int) -> str:
        """``copy_engine`` for few, large runs; ``generated_p2p`` (SM copies) otherwise."""
        ph = self.physicalization
        if transfer_bytes >= ph.copy_engine_threshold_bytes and run_count <= ph.copy_engine_max_runs:
            return "copy_engine"
        return "generated_p2p"

    def validate_batch_layout(self, *, contiguous_page_runs: bool, consumer_partitioned: bool) -> int:
        """Pages per transfer this batch may use (1 when it breaks the layout promise)."""
        if self.physicalization.pages_per_transfer > 1 and not (contiguous_page_runs and consumer_partitioned):
            return 1
        return self.physicalization.pages_per_transfer

    def select_phase(self, *, contiguous_page_runs: bool,
                     consumer_partitioned: bool) -> tuple[CompiledPhase, int]:
        pages = self.validate_batch_layout(contiguous_page_runs=contiguous_page_runs,
                                           consumer_partitioned=consumer_partitioned)
        if pages == self.physicalization.pages_per_transfer or self.fallback_phase is None:
            return self.phase, pages
        return self.fallback_phase, 1

    def describe(self) -> dict:
        return {"name": "kv-cache-migration", "max_pages": self.spec.max_pages,
                "page_bytes": self.spec.page_bytes, "max_consumers": self.spec.max_consumers,
                "physicalization": {**vars(self.physicalization),
                                    "fallback": self.fallback_phase.name if self.fallback_phase else None},
                "layout_contract": dict(vars(self.layout_contract)),
                "execution": self.execution}


def _select_pages_per_transfer(spec: KVCacheMigrationSpec, contract: KVCacheLayoutContract,
                               target_batch_bytes: int) -> int:
    if not contract.contiguous_page_runs:
        return 1
    maximum = min(16, spec.max_pages, max(1, spec.max_pages // spec.max_consumers),
                  max(1, target_batch_bytes // spec.page_bytes))
    return 1 << (maximum.bit_length() - 1)


def compile_kv_cache_migration(
        spec: KVCacheMigrationSpec, *, transports: Optional[tuple[str, ...]] = None,
        layout_contract: Optional[KVCacheLayoutContract] = None,
        execution_contract: Optional[ExecutionContract] = None,
        target_profile: Optional[KVTargetProfile] = None, target_batch_bytes: int = 1 << 20,
        generated_copy_workers: Optional[int] = None, generated_block_elements: Optional[int] = None,
        copy_engine_threshold_bytes: Optional[int] = None, copy_engine_streams: Optional[int] = None,
        copy_engine_max_runs: Optional[int] = None, asynchronous_completion: bool = True,
        consumer_layer_pipeline: Optional[bool] = None, consumers_per_readiness: Optional[int] = None,
        rank: int = 0) -> CompiledKVCacheMigrationPlan:
    if target_batch_bytes <= 0:
        raise ValueError("target_batch_bytes must be positive")
    transports = transports or ("p2p",) * spec.num_ranks
    if len(transports) != spec.num_ranks:
        raise ValueError("KV topology requires one transport per rank")
    layout_contract = layout_contract or KVCacheLayoutContract()
    profile = target_profile or GENERIC_KV_TARGET_PROFILE
    workers = generated_copy_workers if generated_copy_workers is not None else profile.copy_workers
    block = generated_block_elements if generated_block_elements is not None else profile.block_elements
    never = 1 << 62  # a profile without a threshold never hands a run to the copy engine
    threshold = copy_engine_threshold_bytes if copy_engine_threshold_bytes is not None else (
        profile.copy_engine_threshold if profile.copy_engine_threshold is not None else never)
    streams = copy_engine_streams if copy_engine_streams is not None else 1
    max_runs = copy_engine_max_runs if copy_engine_max_runs is not None else 64
    if consumer_layer_pipeline is None:
        consumer_layer_pipeline = (spec.consumer_asynchronous and spec.max_consumers > 1
                                   and layout_contract.consumer_ordered)
    if consumers_per_readiness is None:
        consumers_per_readiness = min(profile.consumers_per_readiness, spec.max_consumers)
    pages = _select_pages_per_transfer(spec, layout_contract, target_batch_bytes)
    execution_contract = execution_contract or ExecutionContract(
        capacity=CapacityContract(max_items=spec.max_pages, dynamic_valid_count=True,
                                  padding=PaddingSemantics.DEAD,
                                  graph_stable_addresses=layout_contract.graph_stable_addresses),
        rank_control=RankControl.DYNAMIC,
        guards=(RuntimeGuard("page_count_within_capacity", ExecutionFallback.ERROR),
                RuntimeGuard("contiguous_batch_layout", ExecutionFallback.EAGER)),
        fallback=ExecutionFallback.EAGER)

    compiled = build_kv_cache_migration_pattern(spec).compile()
    peers = {r: t for r, t in enumerate(transports) if r != rank} or {rank: transports[rank]}
    resources = PhaseResources(peers=peers, buffer_depth=spec.slot_count,
                               realization=KV_CACHE_P2P_REALIZATION)
    plan = compiled.compile_plan(resources)

    def phase_for(pages_per_transfer: int) -> CompiledPhase:
        return compile_phase(plan, "migration.transfer", rank=rank,
                             capacity=max(1, spec.max_pages // pages_per_transfer),
                             width_bytes=spec.page_bytes * pages_per_transfer, reuse=spec.slot_count)

    phase = phase_for(pages)
    fallback_phase = phase_for(1) if pages > 1 else None
    # Unique destinations: the simplifier retargets the transfer at the final storage, so the
    # materialising copy and the staging region are gone from the surviving graph.
    transfer = next(op for op in compiled.dataflow.operations if op["name"] == "migration.transfer")
    direct = (transfer["dst"] == "cache.destination.storage"
              and not compiled.dataflow.has("migration.materialize"))
    if spec.unique_destinations and not direct:
        raise RuntimeError("unique KV pages failed direct-destination proof")
    name = ("parallel-batched-direct-pages" if direct and pages > 1
            else "parallel-direct-pages" if direct else "staged-pages")
    physicalization = KVCachePhysicalization(
        name=name, target_profile=profile.name, pages_per_transfer=pages, direct_destination=direct,
        readiness="consumer" if spec.consumer_asynchronous or spec.max_consumers > 1 else "rank",
        slot_count=spec.slot_count, target_batch_bytes=target_batch_bytes,
        generated_copy_workers=workers, generated_block_elements=block,
        copy_engine_threshold_bytes=threshold, copy_engine_streams=streams,
        copy_engine_max_runs=max_runs, asynchronous_completion=asynchronous_completion,
        consumer_layer_pipeline=consumer_layer_pipeline, consumers_per_readiness=consumers_per_readiness)
    variants = tuple(sorted({max(1, spec.max_pages // pages), spec.max_pages}))
    execution = compile_execution_plan(execution_contract, variants)
    return CompiledKVCacheMigrationPlan(spec, phase, fallback_phase, execution, physicalization,
                                        layout_contract)
