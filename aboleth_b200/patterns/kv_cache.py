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
    """Shape of one migration program: up to ``max_pages`` pages of ``page_bytes`` move per step
    between ``num_ranks`` ranks, to at most ``max_consumers`` consumers (layers) per rank."""

    max_pages: int
    page_bytes: int
    num_ranks: int = 1
    slots: Optional[int] = None
    max_consumers: int = 1
    unique_destinations: bool = True
    consumer_asynchronous: bool = True
    consumer_max_inflight: int = 1

    def __post_init__(self):
        counts = {"max_pages": self.max_pages, "page_bytes": self.page_bytes, "num_ranks": self.num_ranks,
                  "max_consumers": self.max_consumers, "consumer_max_inflight": self.consumer_max_inflight}
        if self.slots is not None:
            counts["slots"] = self.slots
        small = [f"{name}={value}" for name, value in counts.items() if value < 1]
        if small:
            raise ValueError("KV migration spec: " + ", ".join(small) + " must be at least 1")
        if self.page_bytes % 8:
            raise ValueError(f"pages are copied in 8-byte words: page_bytes={self.page_bytes} is not a multiple of 8")
        if self.slots is not None and self.slots < self.required_slots:
            raise ValueError(f"{self.slots} slots cannot cover a consumer that keeps {self.consumer_max_inflight} "
                             f"in flight while the next fills (needs {self.required_slots})")

    @property
    def required_slots(self) -> int:
        """Slots a consumer's lifetime demands: those it still reads plus the one being filled."""
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
