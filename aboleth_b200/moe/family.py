"""A family of MoE slots: power-of-two capacity variants x in-flight slots.

Every (variant, slot) pair owns private payload, flags, epoch and endpoint
reservations, so variants are mutually exclusive within a slot and several slots
can be in flight (dual-batch overlap).  ``select(bound, slot)`` picks the smallest
variant whose capacity covers the rank-uniform token bound.  Reference:
python/aboleth/moe/native.py:663-811, docs/COMPILED_MOE.md:41-48.
"""
from __future__ import annotations

from typing import Optional, Sequence

import torch

from ..shapes import ShapeFamilyPlan, plan_shape_family
from ..world import World
from .compiled_plan import CompiledMoEPlan, compile_moe_plan
from .native import NativeMoESlot
from .spec import MoESpec


class NativeMoEFamily:
    def __init__(self, world: World, *, capacity: int, hidden: int, top_k: int, experts: int,
                 slots: int = 1, owners: Optional[Sequence[int]] = None, tag: str = "moe-family",
                 value_type: str = "bf16", scale_group: int = 128, round_scale: bool = False,
                 quant_amax_floor: float = 1e-4, minimum_capacity: Optional[int] = None,
                 decode_bound: Optional[int] = None, profiles: Optional[dict] = None):
        self.world = world
        self.ranks = world.world_size
        self.capacity, self.hidden, self.top_k, self.experts = capacity, hidden, top_k, experts
        self.slots = slots
        self.family: ShapeFamilyPlan = plan_shape_family(
            tag, minimum=minimum_capacity or capacity, maximum=capacity, slots=slots,
            iteration_bound=decode_bound, uniform=True)
        self.plans: dict[int, CompiledMoEPlan] = {}
        self._slots: dict[tuple[int, int], NativeMoESlot] = {}
        for variant in self.family.variants:
            spec = MoESpec(capacity=variant.capacity, hidden=hidden, top_k=top_k, experts=experts,
                           ranks=self.ranks, value_type=value_type, scale_group=scale_group,
                           round_scale=round_scale, quant_amax_floor=quant_amax_floor)
            self.plans[variant.capacity] = compile_moe_plan(spec, world, profiles=profiles)
            for slot in range(slots):
                domain = self.family.control_domain(variant, slot)
                self._slots[(variant.capacity, slot)] = NativeMoESlot.create(
                    world, spec, tag=f"{tag}.{domain}", plan=self.plans[variant.capacity],
                    placement=list(owners) if owners is not None else "linear")

    def select(self, bound: int, slot: int = 0) -> NativeMoESlot:
        """``bound`` must be the same on every rank (see ``uniform_token_bound``)."""
        variant = self.family.select(bound)
        return self._slots[(variant.capacity, slot)]

    def local_counts(self, expert_counts: torch.Tensor) -> torch.Tensor:
        """Counts of the experts this rank owns, in local expert order."""
        index = getattr(self, "_local_experts", None)
        if index is None or index.device != expert_counts.device:
            any_slot = next(iter(self._slots.values()))
            mine = [e for e, o in enumerate(any_slot.owners_list) if o == self.world.rank]
            # Built once: a host-to-device copy per layer is both slow and illegal under graph capture.
            index = self._local_experts = torch.tensor(mine, device=expert_counts.device)
        return expert_counts[index]

    def manifest(self) -> dict:
        return {"variants": [v.capacity for v in self.family.variants], "slots": self.slots,
                "plans": {c: p.manifest() for c, p in self.plans.items()},
                "slot_manifests": {f"{c}/{s}": slot.manifest() for (c, s), slot in self._slots.items()}}

    def close(self) -> None:
        self._slots.clear()


def uniform_token_bound(tokens: int, group=None) -> int:
    """MAX of ``tokens`` over the ranks of a CPU process group, so that every rank selects
    the same shape variant (the reference's ``_wave_uniform_tokens``,
    integrations/vllm/0001-aboleth-all2all-backend.patch:791-841)."""
    import torch.distributed as dist

    if group is None and not (dist.is_available() and dist.is_initialized()):
        return tokens
    value = torch.tensor([tokens], dtype=torch.int64)
    dist.all_reduce(value, op=dist.ReduceOp.MAX, group=group)
    return int(value.item())
