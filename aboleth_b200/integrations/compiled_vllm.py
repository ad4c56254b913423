"""The fused MoE executor behind the prepare / finalize pair of a serving engine's modular MoE layer.

An engine describes a layer with a dictionary of facts (activation dtype, experts, top-k, hidden
size, token bound, optional fp8 block quantisation).  :class:`LayerContract` validates those facts
once and is the cache key of the slot family that serves every layer with the same contract;
:class:`ModularMoERuntime` is the per-layer object the engine calls: ``prepare`` routes a batch
through the fused dispatch and hands back what the engine's expert kernel consumes, ``finalize``
returns the expert output through the fused combine.  The entry points and their argument names
are those of the reference's adapter (python/aboleth/integrations/compiled_vllm.py:18-188), so an
engine patched for one runs on the other.
"""
from __future__ import annotations

import threading
from dataclasses import dataclass
from typing import Callable, Optional

import torch

from ..moe.family import NativeMoEFamily

_PLACEMENTS = {
    "linear": lambda expert, experts, ranks: expert // (experts // ranks),
    "round_robin": lambda expert, experts, ranks: expert % ranks,
}


@dataclass(frozen=True)
class PreparedExperts:
    """What ``prepare`` returns.  Rows are records: ``[ranks * capacity]``, source rank major."""

    expert_input: torch.Tensor          # [rows, hidden] bf16 or e4m3
    local_counts: torch.Tensor          # int32, (record, choice) pairs per expert this rank owns
    global_ids: torch.Tensor            # [rows, k] int32 expert ids, unused choices name a foreign expert
    expert_weights: torch.Tensor        # [rows, k] fp32 gates (0 for unused choices)
    scales: Optional[torch.Tensor] = None       # [rows, hidden / group] fp32 view, fp8 contracts only
    expert_pos: Optional[torch.Tensor] = None   # [rows, k] position inside the (source, expert) group
    recv_counts: Optional[torch.Tensor] = None  # int64 live records per source rank
    counts_by_source: Optional[torch.Tensor] = None  # [ranks, experts] int32, input of ``expert_offsets``


@dataclass(frozen=True)
class LayerContract:
    """The facts of one MoE layer that decide which kernels and buffers serve it."""

    capacity: int
    minimum_capacity: Optional[int]
    decode_bound: Optional[int]
    hidden: int
    top_k: int
    experts: int
    slots: int
    owners: tuple
    value_type: str
    scale_group: int
    round_scale: bool
    amax_floor: float

    @classmethod
    def from_engine(cls, facts: dict, ranks: int, slots: int, placement: str) -> "LayerContract":
        if facts["dtype"] is not torch.bfloat16:
            raise NotImplementedError(f"the executor moves bf16 activations, the model runs {facts['dtype']}")
        experts = int(facts["num_experts"])
        if experts % ranks != 0 or int(facts["num_local_experts"]) * ranks != experts:
            raise ValueError(f"{experts} experts do not split evenly over {ranks} ranks")
        if placement not in _PLACEMENTS:
            raise ValueError(f"unknown expert placement {placement!r}; choose from {sorted(_PLACEMENTS)}")
        owners = tuple(_PLACEMENTS[placement](e, experts, ranks) for e in range(experts))
        quantised = facts.get("quant_dtype") is not None
        value_type, group, floor = "bf16", 128, 1e-4
        if quantised:
            block = facts.get("quant_block_shape")
            if facts["quant_dtype"] is not torch.float8_e4m3fn or block is None or len(block) != 2:
                raise NotImplementedError("quantised dispatch means e4m3 with one scale per token and K block")
            if "quant_round_scale" not in facts:
                # Power-of-two scales or not changes the bytes on the wire: the engine has to say.
                raise ValueError("an fp8 layer must state quant_round_scale (does its expert kernel want "
                                 "power-of-two scales?)")
            value_type, group, floor = "f8E4M3FN", int(block[1]), 1e-10
        elif facts.get("quant_round_scale"):
            raise ValueError("quant_round_scale was set for a layer that does not quantise")
        return cls(capacity=int(facts["num_max_tokens_per_rank"]),
                   minimum_capacity=facts.get("min_tokens_per_rank"), decode_bound=facts.get("decode_bound"),
                   hidden=int(facts["hidden"]), top_k=int(facts["num_topk"]), experts=experts, slots=slots,
                   owners=owners, value_type=value_type, scale_group=group,
                   round_scale=bool(facts.get("quant_round_scale", False)), amax_floor=floor)

    def build(self, world, tag: str) -> NativeMoEFamily:
        return NativeMoEFamily(world, capacity=self.capacity, hidden=self.hidden, top_k=self.top_k,
                               experts=self.experts, slots=self.slots, owners=self.owners, tag=tag,
                               value_type=self.value_type, scale_group=self.scale_group,
                               round_scale=self.round_scale, quant_amax_floor=self.amax_floor,
                               decode_bound=self.decode_bound, minimum_capacity=self.minimum_capacity)


class AbolethMoERuntimeManager:
    """One per process: layers with equal contracts share one slot family."""

    def __init__(self, *, world, internode: bool = False):
        self.world, self.internode = world, internode
        self.handles: dict[LayerContract, NativeMoEFamily] = {}
        self._guard = threading.Lock()

    def get_handle(self, kwargs: dict, *, num_slots: int = 1,
                   placement_strategy: str = "linear") -> NativeMoEFamily:
        contract = LayerContract.from_engine(kwargs, self.world.world_size, num_slots, placement_strategy)
        with self._guard:
            family = self.handles.get(contract)
            if family is None:
                family = contract.build(self.world, tag=f"compiled-moe-{len(self.handles)}")
                self.handles[contract] = family
            return family

    def close(self) -> None:
        with self._guard:
            families, self.handles = list(self.handles.values()), {}
        for family in families:
            family.close()


class ModularMoERuntime:
    """Per-layer prepare / finalize.  ``slot_provider`` names the in-flight slot of the calling
    micro-batch (dual-batch overlap runs two); a slot carries one layer from prepare to finalize."""

    def __init__(self, handle: NativeMoEFamily, *, layer_name: str = "",
                 slot_provider: Optional[Callable[[], int]] = None):
        self.family, self.layer_name = handle, layer_name
        self.slot_provider = slot_provider if slot_provider is not None else (lambda: 0)
        self.has_decode_sibling = len(handle.family.variants) > 1
        self.selected: dict = {}     # slot -> the NativeMoESlot (shape variant) its last prepare chose
        self.routed: set = set()     # slots between prepare and finalize

    # -- facts the engine asks for ---------------------------------------------------------
    def num_dispatchers(self) -> int:
        return self.family.ranks

    def output_is_reduced(self) -> bool:
        return True     # finalize leaves the gate-weighted sum over all experts

    def max_num_tokens_per_rank(self) -> int:
        return self.family.capacity

    def topk_indices_dtype(self):
        return torch.int32

    def expert_output_alias(self, expert_input: torch.Tensor) -> torch.Tensor:
        """The buffer an expert kernel may write directly so that finalize copies nothing."""
        executor = self.selected[self.slot_provider()]
        if executor.expert_output.shape[0] != expert_input.shape[0]:
            raise RuntimeError(f"{self.layer_name}: expert input has {expert_input.shape[0]} rows, the "
                               f"selected variant holds {executor.expert_output.shape[0]}")
        return executor.expert_output

    # -- the two calls per layer -------------------------------------------------------------
    def prepare(self, a1: torch.Tensor, topk_weights: torch.Tensor, topk_ids: torch.Tensor, *,
                num_experts: int, expert_map=None, apply_router_weight_on_input: bool = False,
                required_tokens: int = 0, quantized_input: bool = False,
                defer_input_quant: bool = False) -> PreparedExperts:
        if num_experts != self.family.experts:
            raise ValueError(f"{self.layer_name}: the layer has {num_experts} experts, its contract "
                             f"{self.family.experts}")
        slot = self.slot_provider()
        if slot in self.routed:
            raise RuntimeError(f"{self.layer_name}: slot {slot} already carries a layer that was not finalized")
        if apply_router_weight_on_input:
            if topk_ids.shape[1] != 1:
                raise ValueError("gates can only be folded into the input of a top-1 layer")
            a1, topk_weights = a1 * topk_weights.to(a1.dtype), torch.ones_like(topk_weights)
        executor = self.family.select(max(int(a1.shape[0]), int(required_tokens)), slot)
        wants_fp8 = bool(quantized_input) and not defer_input_quant
        if executor.spec.fp8 != wants_fp8:
            raise ValueError(f"{self.layer_name}: the expert kernel asks for "
                             f"{'quantised' if wants_fp8 else 'unquantised'} input, the contract dispatches "
                             f"{executor.spec.value_type}")
        self.selected[slot] = executor
        result = executor.dispatch(a1.contiguous(), topk_ids.to(torch.int32).contiguous(),
                                   topk_weights.float().contiguous())
        self.routed.add(slot)
        return PreparedExperts(expert_input=result.expert_input,
                               local_counts=self.family.local_counts(result.expert_counts),
                               global_ids=result.expert_ids, expert_weights=result.expert_weights,
                               scales=result.expert_scales, expert_pos=result.expert_pos,
                               recv_counts=result.recv_counts,
                               counts_by_source=result.expert_counts_by_source)

    def finalize(self, output: torch.Tensor, fused_expert_output: torch.Tensor,
                 expert_offsets: Optional[torch.Tensor] = None) -> None:
        slot = self.slot_provider()
        if slot not in self.routed:
            raise RuntimeError(f"{self.layer_name}: finalize on slot {slot}, which has nothing prepared")
        executor = self.selected[slot]
        tokens = output.shape[0]
        direct = output.is_contiguous()
        executor.combine(fused_expert_output, expert_offsets=expert_offsets,
                         out=output if direct else None, num_tokens=tokens)
        if not direct:
            output.copy_(executor.final_output[:tokens])
        self.routed.discard(slot)
