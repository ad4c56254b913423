"""Execution contract: may a phase run at a fixed compiled capacity, and what to do when not.

A fixed-capacity launch (the CUDA-graph friendly form) is legal only when the valid count
is dynamic, the padding is dead, addresses are graph-stable and the ranks run in lockstep;
otherwise the declared fallback applies.  Reference: python/aboleth/execution.py:13-253.
"""
from __future__ import annotations

from dataclasses import dataclass
from enum import Enum


class PaddingSemantics(Enum):
    UNKNOWN = "unknown"
    PRESERVED = "preserved"
    DEAD = "dead"


class RankControl(Enum):
    UNKNOWN = "unknown"
    DYNAMIC = "dynamic"
    LOCKSTEP = "lockstep"


class ExecutionFallback(Enum):
    EXACT_AGREEMENT = "exact_agreement"
    EAGER = "eager"
    ERROR = "error"


@dataclass(frozen=True)
class CapacityContract:
    max_items: int
    dynamic_valid_count: bool
    padding: PaddingSemantics
    graph_stable_addresses: bool

    def __post_init__(self) -> None:
        if self.max_items <= 0:
            raise ValueError("capacity max_items must be positive")
        if not isinstance(self.padding, PaddingSemantics):
            raise TypeError("capacity padding must be PaddingSemantics")


@dataclass(frozen=True)
class RuntimeGuard:
    name: str
    fallback: ExecutionFallback

    def __post_init__(self) -> None:
        if not self.name:
            raise ValueError("runtime guard name cannot be empty")
        if not isinstance(self.fallback, ExecutionFallback):
            raise TypeError("runtime guard fallback must be ExecutionFallback")


@dataclass(frozen=True)
class ExecutionDecision:
    mode: str            # "fixed_capacity" | "exact_agreement" | "eager"
    capacity: int
    reason: str


@dataclass(frozen=True)
class ExecutionContract:
    capacity: CapacityContract
    rank_control: RankControl
    guards: tuple[RuntimeGuard, ...] = ()
    fallback: ExecutionFallback = ExecutionFallback.EXACT_AGREEMENT

    def __post_init__(self) -> None:
        if not isinstance(self.rank_control, RankControl):
            raise TypeError("execution rank_control must be RankControl")
        if not isinstance(self.fallback, ExecutionFallback):
            raise TypeError("execution fallback must be ExecutionFallback")
        names = [g.name for g in self.guards]
        if len(names) != len(set(names)):
            raise ValueError("runtime guard names must be unique")

    @property
    def fixed_capacity_legal(self) -> bool:
        c = self.capacity
        return (c.dynamic_valid_count and c.padding is PaddingSemantics.DEAD
                and c.graph_stable_addresses and self.rank_control is RankControl.LOCKSTEP)

    def describe(self) -> dict:
        c = self.capacity
        return {"capacity": {"max_items": c.max_items, "dynamic_valid_count": c.dynamic_valid_count,
                             "padding": c.padding.value, "graph_stable_addresses": c.graph_stable_addresses},
                "rank_control": self.rank_control.value, "fixed_capacity_legal": self.fixed_capacity_legal,
                "fallback": self.fallback.value,
                "guards": [{"name": g.name, "fallback": g.fallback.value} for g in self.guards]}

    def resolve(self, actual_items: int, *, graph_stable_addresses: bool = True,
                failed_guards: tuple[str, ...] = ()) -> ExecutionDecision:
        """Pick the execution mode for one call with ``actual_items`` live items."""
        if actual_items < 0 or actual_items > self.capacity.max_items:
            raise ValueError(f"{actual_items} items are outside the contract's capacity "
                             f"{self.capacity.max_items}")
        for guard in self.guards:
            if guard.name in failed_guards:
                if guard.fallback is ExecutionFallback.ERROR:
                    raise RuntimeError(f"runtime guard {guard.name!r} failed")
                return ExecutionDecision(guard.fallback.value, actual_items, f"guard {guard.name} failed")
        if self.fixed_capacity_legal and graph_stable_addresses:
            return ExecutionDecision("fixed_capacity", self.capacity.max_items, "contract proven")
        if self.fallback is ExecutionFallback.ERROR:
            raise RuntimeError("fixed-capacity execution is not legal and the contract forbids a fallback")
        return ExecutionDecision(self.fallback.value, actual_items, "fixed capacity not proven")


@dataclass(frozen=True)
class CompiledExecutionPlan:
    """Compiled phases plus the contract they may run under."""

    phases: tuple
    contract: ExecutionContract

    def __post_init__(self) -> None:
        names = tuple(phase.name for phase in self.phases)
        if not names:
            raise ValueError("compiled execution plan requires at least one phase")
        if len(names) != len(set(names)):
            raise ValueError("compiled execution phase names must be unique")

    def phase(self, name: str):
        for phase in self.phases:
            if phase.name == name:
                return phase
        raise KeyError(f"compiled execution has no phase {name!r}")

    def resolve(self, actual_items: int, **kwargs) -> ExecutionDecision:
        return self.contract.resolve(actual_items, **kwargs)

    def describe(self) -> dict:
        return {"contract": self.contract.describe(),
                "phases": [phase.manifest() if hasattr(phase, "manifest") else {"name": phase.name}
                           for phase in self.phases]}


def compile_execution_plan(contract: ExecutionContract, variants: tuple[int, ...]) -> dict:
    """Which compiled capacities a contract may use, smallest first."""
    usable = tuple(v for v in sorted(variants) if v <= contract.capacity.max_items) or \
        (contract.capacity.max_items,)
    return {"contract": contract.describe(), "variants": usable,
            "mode": "fixed_capacity" if contract.fixed_capacity_legal else contract.fallback.value}
