"""Execution contract: may a phase run at a fixed compiled capacity, and what to do when not.

A launch at a fixed capacity (the form a CUDA graph can hold) moves the padding of a partly
filled buffer along with its live prefix and assumes every rank takes the same path.  That is
only sound under four proof obligations, which :meth:`ExecutionContract.unmet` lists by name:
the live count is a run-time value, the padding is dead, the addresses do not change between
replays, and the ranks advance in lockstep.  With an obligation open, the declared fallback
applies (agree on the exact count first, run eagerly, or refuse).  The vocabulary - capacity
contract, padding semantics, rank control, runtime guards, fallbacks - is the reference's
(python/aboleth/execution.py:13-253).
"""
from __future__ import annotations

from dataclasses import dataclass
from enum import Enum


class _Named(Enum):
    """Enumerations here compare by identity and also accept their value as a string."""

    @classmethod
    def of(cls, value):
        if isinstance(value, cls):
            return value
        try:
            return cls(value)
        except ValueError:
            raise TypeError(f"{value!r} is not a {cls.__name__}; expected one of "
                            f"{[member.value for member in cls]}") from None


class PaddingSemantics(_Named):
    UNKNOWN = "unknown"        # nothing is known about the bytes past the live prefix
    PRESERVED = "preserved"    # a reader may look at them: they must not travel or be clobbered
    DEAD = "dead"              # nobody reads them: moving or overwriting them is harmless


class RankControl(_Named):
    UNKNOWN = "unknown"
    DYNAMIC = "dynamic"        # ranks may take different paths (a rank can skip a step)
    LOCKSTEP = "lockstep"      # every rank runs every step with the same shape variant


class ExecutionFallback(_Named):
    EXACT_AGREEMENT = "exact_agreement"   # ranks agree on the live count, then launch exactly that
    EAGER = "eager"                       # leave the graph: launch from the host with the live count
    ERROR = "error"                       # refuse


@dataclass(frozen=True)
class CapacityContract:
    """What is promised about a buffer of ``max_items`` slots of which a prefix is live."""

    max_items: int
    dynamic_valid_count: bool
    padding: PaddingSemantics
    graph_stable_addresses: bool

    def __post_init__(self) -> None:
        if self.max_items < 1:
            raise ValueError(f"a capacity holds at least one item, got max_items={self.max_items}")
        object.__setattr__(self, "padding", PaddingSemantics.of(self.padding))


@dataclass(frozen=True)
class RuntimeGuard:
    """A condition only the running program can check, and what happens when it fails."""

    name: str
    fallback: ExecutionFallback

    def __post_init__(self) -> None:
        if not self.name.strip():
            raise ValueError("a runtime guard needs a name (it is how a failed guard is reported)")
        object.__setattr__(self, "fallback", ExecutionFallback.of(self.fallback))


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
        object.__setattr__(self, "rank_control", RankControl.of(self.rank_control))
        object.__setattr__(self, "fallback", ExecutionFallback.of(self.fallback))
        seen: set[str] = set()
        for guard in self.guards:
            if guard.name in seen:
                raise ValueError(f"two runtime guards are called {guard.name!r}")
            seen.add(guard.name)

    def unmet(self) -> tuple[str, ...]:
        """The proof obligations of a fixed-capacity launch that this contract leaves open."""
        c = self.capacity
        checks = (("the live count is a run-time value", c.dynamic_valid_count),
                  ("the padding is dead", c.padding is PaddingSemantics.DEAD),
                  ("addresses are stable across graph replays", c.graph_stable_addresses),
                  ("ranks run in lockstep", self.rank_control is RankControl.LOCKSTEP))
        return tuple(name for name, holds in checks if not holds)

    @property
    def fixed_capacity_legal(self) -> bool:
        return not self.unmet()

    def describe(self) -> dict:
        c = self.capacity
        return {"capacity": {"max_items": c.max_items, "dynamic_valid_count": c.dynamic_valid_count,
                             "padding": c.padding.value, "graph_stable_addresses": c.graph_stable_addresses},
                "rank_control": self.rank_control.value, "fixed_capacity_legal": self.fixed_capacity_legal,
                "open_obligations": list(self.unmet()), "fallback": self.fallback.value,
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
