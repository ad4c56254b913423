"""KV-cache page migration around an opaque cache consumer, as a Pattern.

Pages named by a workset (source row, destination peer, destination row, consumer) move
into a staging region on the consumer rank and are materialised into the cache's final
storage, which the consumer's attention kernels read.  When destinations are unique the
dataflow simplification retargets the transfer at the final storage and the staging copy
disappears (reference: python/aboleth/patterns/kv_cache.py:11-185).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

from ..pattern import OpaqueCapabilities, Pattern


@dataclass(frozen=True)
class KVCacheMigrationSpec:
    max_pages: int
    page_bytes: int
    num_ranks: int = 1
    slots: Optional[int] = None
    max_consumers: int = 1
    unique_destinations: bool = True
    consumer_asynchronous: bool = True
    consumer_max_inflight: int = 1

    def __post_init__(self):
        if self.max_pages <= 0:
            raise ValueError("max_pages must be positive")
        if self.page_bytes <= 0:
            raise ValueError("page_bytes must be positive")
        if self.page_bytes % 8:
            raise ValueError("page_bytes must be aligned to eight bytes")
        if self.num_ranks <= 0:
            raise ValueError("num_ranks must be positive")
        if self.slots is not None and self.slots <= 0:
            raise ValueError("slots must be positive")
        if self.max_consumers <= 0:
            raise ValueError("max_consumers must be positive")
        if self.consumer_max_inflight <= 0:
            raise ValueError("consumer_max_inflight must be positive")
        if self.slots is not None and self.slots < self.required_slots:
            raise ValueError("slot count cannot satisfy consumer lifetime")

    @property
    def required_slots(self) -> int:
        """An asynchronous consumer holds ``max_inflight`` slots while the next one fills."""
        return self.consumer_max_inflight + 1 if self.consumer_asynchronous else 1

    @property
    def slot_count(self) -> int:
        return self.slots or self.required_slots


def build_kv_cache_migration_pattern(spec: KVCacheMigrationSpec) -> Pattern:
    flow = Pattern("kv-cache-migration")
    pages, row = spec.max_pages, spec.page_bytes
    flow.region("cache.source.pages", pages, row, immutable=True, registered=True,
                valid_count="migration.count")
    for name, width in (("migration.source_rows", 8), ("migration.destination_peers", 4),
                        ("migration.destination_rows", 8), ("migration.consumer_ids", 4)):
        flow.region(name, pages, width, immutable=True)
    work = flow.workset("migration.work", "cache.source.pages", max_items=pages, item_bytes=row)
    flow.region("cache.destination.staging", pages, row)
    flow.region("cache.destination.storage", pages, row, escapes=True, registered=True,
                donated=spec.unique_destinations, max_inflight=spec.slot_count)
    flow.transfer_each("migration.transfer", work, "cache.destination.staging")
    flow.copy_each_from("migration.materialize", "cache.destination.staging", "cache.destination.storage")
    flow.reads("cache.source.pages", "migration.transfer", (0, pages), prefix=True)
    flow.writes("cache.destination.storage", "migration.materialize", (0, pages))
    flow.opaque_compute("cache.consumer", ["cache.destination.storage"], "cache.destination.storage",
                        capabilities=OpaqueCapabilities(graph_capturable=not spec.consumer_asynchronous))
    flow.use("cache.reader", ["cache.destination.storage"])
    return flow
