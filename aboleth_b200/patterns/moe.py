"""The logical expert-parallel protocol around opaque expert compute, as a Pattern.

route -> dispatch.{values, scales, count} -> experts (opaque) -> return.values -> combine
(opaque) -> output.  Field names and defaults of :class:`MoEPatternSpec` follow the reference
(python/aboleth/patterns/moe.py:21-63); the graph is the one its builder declares
(python/aboleth/patterns/moe.py:66-157, helpers in _moe.py and _exchange.py), written
against this package's region/row model: a region is ``rows x row_bytes`` and a workset is
the unordered set of routed rows.
"""
from __future__ import annotations

from dataclasses import dataclass

from ..pattern import OpaqueCapabilities, Pattern

_ELEMENT_BYTES = {"bf16": 2, "f16": 2, "f32": 4, "fp8": 1, "f8e4m3": 1, "i8": 1, "i32": 4, "i64": 8}


def element_bytes(element_type: str) -> int:
    try:
        return _ELEMENT_BYTES[element_type]
    except KeyError:
        raise ValueError(f"unknown element type {element_type!r}") from None


@dataclass(frozen=True)
class MoEPatternSpec:
    max_tokens: int
    hidden: int
    top_k: int
    num_ranks: int = 1
    slots: int = 4
    value_type: str = "bf16"
    scale_width: int = 0
    output_type: str = "bf16"
    experts_asynchronous: bool = True
    expert_max_inflight: int = 1
    expert_event_ordered: bool = True
    preserve_return_staging: bool = False

    def __post_init__(self):
        sizes = {name: getattr(self, name)
                 for name in ("max_tokens", "hidden", "top_k", "num_ranks", "slots", "expert_max_inflight")}
        wrong = [f"{name}={value}" for name, value in sizes.items() if value < 1]
        if self.scale_width < 0:
            wrong.append(f"scale_width={self.scale_width}")
        if wrong:
            raise ValueError("MoE pattern spec: " + ", ".join(wrong) + " out of range")
        if not self.experts_asynchronous and self.expert_max_inflight != 1:
            raise ValueError("an expert stage that runs synchronously holds exactly one layer in flight")
        for kind in (self.value_type, self.output_type):
            element_bytes(kind)  # raises on an unknown element type

    @property
    def has_scales(self) -> bool:
        return self.scale_width > 0

    @property
    def routes(self) -> int:
        return self.max_tokens * self.top_k

    @property
    def expert_rows(self) -> int:
        return self.routes * self.num_ranks


def build_moe_pattern(spec: MoEPatternSpec) -> Pattern:
    """route -> dispatch -> experts -> return -> combine, with the experts and the combine opaque."""
    p = Pattern("moe")
    routes, expert_rows = spec.routes, spec.expert_rows
    value_row = spec.hidden * element_bytes(spec.value_type)
    output_row = spec.hidden * element_bytes(spec.output_type)

    # What routing produced on this rank (inputs of the protocol, never written by it).
    p.region("route.values", routes, value_row, immutable=True, registered=True, valid_count="route.count")
    p.region("route.source_rows", routes, 8, immutable=True)
    p.region("route.weights", routes, 4, immutable=True)
    p.region("route.peer_counts", spec.num_ranks, 4, immutable=True)
    work = p.workset("dispatch.work", "route.values", max_items=routes, item_bytes=value_row)

    # Dispatch: values (and block scales) to the expert owners, plus one count per peer.
    p.region("expert.values", expert_rows, value_row, max_inflight=spec.slots)
    inputs = [p.transfer_each("dispatch.values", work, "expert.values")]
    p.reads("route.values", "dispatch.values", (0, routes), prefix=True)
    p.writes("expert.values", "dispatch.values", (0, expert_rows))
    if spec.has_scales:
        p.region("route.scales", routes, 4 * spec.scale_width, immutable=True)
        p.region("expert.scales", expert_rows, 4 * spec.scale_width, max_inflight=spec.slots)
        inputs.append(p.transfer("dispatch.scales", "route.scales", "expert.scales"))
    p.region("expert.counts", spec.num_ranks, 4, max_inflight=spec.slots)
    inputs.append(p.transfer("dispatch.count", "route.peer_counts", "expert.counts"))

    # Experts: the client's kernels.  They may write straight into the return source.
    p.region("expert.output", expert_rows, output_row)
    destinations = ["expert.values", "expert.counts"] + (["expert.scales"] if spec.has_scales else [])
    p.opaque_compute("experts", destinations, "expert.output",
                     capabilities=OpaqueCapabilities(accepts_destination_rewrite=True))
    p.reads("expert.values", "experts", (0, expert_rows), through=expert_rows)

    # Return: every expert row back to the rank that routed it.
    p.region("return.source", expert_rows, output_row, registered=True, donated=True)
    p.copy("return.stage", "expert.output", "return.source")
    p.region("returned.values", routes, output_row, max_inflight=spec.slots)
    p.transfer("return.values", "return.source", "returned.values")
    p.writes("returned.values", "return.values", (0, routes))

    # Combine: gate-weighted reduction per token (opaque: a fused kernel of the client).
    p.region("output.values", spec.max_tokens, spec.hidden * 4, escapes=True)
    p.opaque_compute("combine", ["returned.values", "route.source_rows", "route.weights"], "output.values")
    p.reads("returned.values", "combine", (0, routes))
    p.use("output.consumer", ["output.values"])
    return p
