"""A compiled phase: one transfer of a pattern plan turned into a Tier-2 program, its
specialised source and the launch geometry.  Reference: python/aboleth/phase.py:39-282,
python/aboleth/planned_phase.py:18-200.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

from .compiler import CompiledProgram, compile_program
from .pattern import CompiledPatternPlan, PhaseSchedule
from .records import await_records, send_records


@dataclass(frozen=True)
class PhaseLaunch:
    name: str
    sender_grid: tuple[int, int]
    receiver_grid: tuple[int, int]
    sender_threads: int
    ready_stride: int
    signal_slots: int


@dataclass(frozen=True)
class CompiledPhase:
    name: str
    schedule: PhaseSchedule
    binding: PhaseLaunch
    sender: CompiledProgram
    receiver: CompiledProgram
    completion_interval: int

    def manifest(self) -> dict:
        return {"name": self.name, "strategy": self.schedule.strategy,
                "publication": self.schedule.publication_strategy,
                "sender_grid": self.binding.sender_grid, "receiver_grid": self.binding.receiver_grid,
                "completion_interval": self.completion_interval,
                "sender_facts": self.sender.facts, "receiver_facts": self.receiver.facts}


def compile_phase(plan: CompiledPatternPlan, name: str, *, rank: int, capacity: int, width_bytes: int,
                  meta_width_words: int = 0, reuse: Optional[int] = None) -> CompiledPhase:
    """Compile the record transport of one planned transfer for the current ``compilation`` options."""
    launches = plan.launches[name]
    if not launches:
        raise ValueError(f"phase {name!r} has no launch partition")
    launch = launches[0]
    schedule = plan.phase_schedule(name)
    sender = compile_program(send_records(
        rank=rank, peer_extent=max(len(launch.peers), 1) + 1, capacity=capacity, width_bytes=width_bytes,
        meta_width_words=meta_width_words, lanes=launch.lanes, row_quotient=launch.slice_quotient,
        row_remainder=launch.slice_remainder, reuse=reuse or schedule.buffer_depth,
        ready_stride=launch.ready_stride, threads=32 * launch.sender_warps))
    receiver = compile_program(await_records(ready_stride=launch.ready_stride,
                                             lanes_per_program=launch.receiver_lanes_per_program))
    binding = PhaseLaunch(name, launch.sender_grid, launch.receiver_grid, 32 * launch.sender_warps,
                           launch.ready_stride, launch.signal_slots)
    return CompiledPhase(name, schedule, binding, sender, receiver,
                         plan.completion_interval_for(name.replace(".", "_")))
