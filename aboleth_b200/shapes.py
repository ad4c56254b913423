"""Shape families: power-of-two capacity variants and the selector that picks one.

The plan itself is computed by the native ``plan-shapes`` pass; this module
builds the request and interprets the thresholds
(reference: python/aboleth/shapes.py:13-123, compiler/lib/Transforms/PlanShapes.cpp:28-116).
"""
from __future__ import annotations

import bisect
from dataclasses import dataclass
from typing import Optional

from .compiler.driver import run_planner
from .compiler.options import current_options


@dataclass(frozen=True)
class ShapeVariant:
    capacity: int
    control_base: int
    control_count: int


@dataclass(frozen=True)
class ShapeFamilyPlan:
    name: str
    maximum_bound: int
    slots: int
    selector: str
    uniform_required: bool
    variants: tuple[ShapeVariant, ...]

    def select(self, bound: int) -> ShapeVariant:
        """Smallest variant whose capacity is at least ``bound`` (the runtime bound must be
        the same on every rank when ``uniform_required``)."""
        if bound > self.variants[-1].capacity:
            raise ValueError(f"bound {bound} exceeds the largest variant {self.variants[-1].capacity}")
        capacities = [v.capacity for v in self.variants]
        return self.variants[bisect.bisect_left(capacities, max(bound, 1))]

    def control_domain(self, variant: ShapeVariant, slot: int) -> int:
        if not 0 <= slot < variant.control_count:
            raise ValueError("slot is outside the variant's control domain")
        return variant.control_base + slot


def plan_shape_family(name: str, *, minimum: int, maximum: int, slots: int = 1,
                      iteration_bound: Optional[int] = None, uniform: bool = True) -> ShapeFamilyPlan:
    passes = ",".join(sorted(current_options().passes))
    request = f"program plan enable={passes or 'none'}\nshape_family name={name} minimum={minimum} " \
              f"maximum={maximum} slots={slots} uniform={int(uniform)}"
    if iteration_bound is not None:
        request += f" iteration={iteration_bound}"
    family = run_planner("plan-shapes", request + "\n")["families"][0]
    return ShapeFamilyPlan(
        name=family["name"], maximum_bound=family["maximum_bound"], slots=family["slots"],
        selector=family["selector"], uniform_required=family["uniform_required"],
        variants=tuple(ShapeVariant(v["capacity"], v["control_base"], v["control_count"])
                       for v in family["variants"]))
