"""Prepare/finalize around the fused MoE executor, in the shape a serving engine's
modular-MoE layer expects.

``AbolethMoERuntimeManager.get_handle`` turns the engine's layer facts into a
:class:`NativeMoEFamily` (cached per fact tuple); ``ModularMoERuntime.prepare``
dispatches a layer's tokens and returns what the expert kernel consumes,
``finalize`` combines the expert output.  Interface and checks follow the reference
(python/aboleth/integrations/compiled_vllm.py:18-188).
"""
from __future__ import annotations

from dataclasses import dataclass
from threading import Lock
from typing import Callable, Optional

import torch

from ..moe.family import NativeMoEFamily


@dataclass(frozen=True)
class PreparedExperts:
    expert_input: torch.Tensor          # [ranks*capacity, hidden] bf16 or e4m3 records
    local_counts: torch.Tensor          # int32 counts of this rank's experts
    global_ids: torch.Tensor            # [ranks*capacity, k] int32
    expert_weights: torch.Tensor        # [ranks*capacity, k] fp32
    scales: Optional[torch.Tensor] = None
    expert_pos: Optional[torch.Tensor] = None   # position of each (record, choice) in its expert
    recv_counts: Optional[torch.Tensor] = None  # live records per source rank


class AbolethMoERuntimeManager:
    def __init__(self, *, world, internode: bool = False):
        self.world = world
        self.internode = internode
        self.handles: dict = {}
        self.lock = Lock()

    def get_handle(self, kwargs: dict, *, num_slots: int = 1,
                   placement_strategy: str = "linear") -> NativeMoEFamily:
        if kwargs["dtype"] != torch.bfloat16:
            raise NotImplementedError("compiled MoE requires BF16 model activations")
        quant = kwargs.get("quant_dtype")
        group, value_type, floor = 128, "bf16", 1e-4
        rounded = kwargs.get("quant_round_scale", False)
        if quant is not None:
            block = kwargs.get("quant_block_shape")
            if "quant_round_scale" not in kwargs:
                raise ValueError("FP8 requires the optimized consumer scale-rounding fact")
            if quant != torch.float8_e4m3fn or block is None or len(block) != 2:
                raise NotImplementedError("FP8 dispatch requires E4M3 per-token K-block scales")
            group, value_type, floor = block[1], "f8E4M3FN", 1e-10
        elif rounded:
            raise ValueError("unquantized dispatch has no rounding contract")
        e, r = kwargs["num_experts"], self.world.world_size
        if e % r or kwargs["num_local_experts"] != e // r:
            raise ValueError("expert counts must be balanced")
        if placement_strategy == "linear":
            owners = tuple(i // (e // r) for i in range(e))
        elif placement_strategy == "round_robin":
            owners = tuple(i % r for i in range(e))
        else:
            raise ValueError("expert placement must be linear or round_robin")
        key = (kwargs["num_max_tokens_per_rank"], kwargs["hidden"], kwargs["num_topk"], e, num_slots,
               owners, value_type, group, rounded, floor, kwargs.get("decode_bound"))
        with self.lock:
            if key not in self.handles:
                self.handles[key] = NativeMoEFamily(
                    self.world, capacity=key[0], hidden=key[1], top_k=key[2], experts=e,
                    slots=num_slots, owners=owners, tag=f"compiled-moe-{len(self.handles)}",
                    value_type=value_type, scale_group=group, round_scale=rounded,
                    quant_amax_floor=floor, decode_bound=kwargs.get("decode_bound"),
                    minimum_capacity=kwargs.get("min_tokens_per_rank"))
            return self.handles[key]

    def close(self) -> None:
        for handle in self.handles.values():
            handle.close()
        self.handles.clear()


class ModularMoERuntime:
    def __init__(self, handle: NativeMoEFamily, *, layer_name: str = "",
                 slot_provider: Optional[Callable[[], int]] = None):
        self.family = handle
        self.layer_name = layer_name
        self.slot_provider = slot_provider or (lambda: 0)
        self.has_decode_sibling = len(handle.family.variants) > 1
        self.selected: dict = {}
        self.routed: set = set()

    def num_dispatchers(self) -> int:
        return self.family.ranks

    def output_is_reduced(self) -> bool:
        return True

    def max_num_tokens_per_rank(self) -> int:
        return self.family.capacity

    def topk_indices_dtype(self):
        return torch.int32

    def expert_output_alias(self, expert_input: torch.Tensor) -> torch.Tensor:
        """The buffer the expert kernel should write so that combine needs no copy."""
        handle = self.selected[self.slot_provider()]
        if handle.expert_output.shape[0] != expert_input.shape[0]:
            raise RuntimeError("expert binding shape mismatch")
        return handle.expert_output

    def prepare(self, a1: torch.Tensor, topk_weights: torch.Tensor, topk_ids: torch.Tensor, *,
                num_experts: int, expert_map=None, apply_router_weight_on_input: bool = False,
                required_tokens: int = 0, quantized_input: bool = False,
                defer_input_quant: bool = False) -> PreparedExperts:
        if num_experts != self.family.experts:
            raise ValueError("missing or mismatched expert contract")
        if apply_router_weight_on_input:
            if topk_ids.shape[1] != 1:
                raise ValueError("router weight on input requires top-k one")
            a1 = a1 * topk_weights.to(a1.dtype)
            topk_weights = torch.ones_like(topk_weights)
        slot = self.slot_provider()
        if slot in self.routed:
            raise RuntimeError("same in-flight slot prepared twice before finalize")
        handle = self.family.select(max(int(a1.shape[0]), int(required_tokens)), slot)
        if bool(handle.spec.scale_cols) != bool(quantized_input and not defer_input_quant):
            raise ValueError("expert quantization request disagrees with the compiled dispatch contract")
        self.selected[slot] = handle
        result = handle.dispatch(a1.contiguous(), topk_ids.to(torch.int32).contiguous(),
                                 topk_weights.float().contiguous())
        self.routed.add(slot)
        return PreparedExperts(result.expert_input, self.family.local_counts(result.expert_counts),
                               result.expert_ids, result.expert_weights, result.expert_scales,
                               result.expert_pos, result.recv_counts)

    def finalize(self, output: torch.Tensor, fused_expert_output: torch.Tensor,
                 expert_offsets: Optional[torch.Tensor] = None) -> None:
        slot = self.slot_provider()
        if slot not in self.routed:
            raise RuntimeError("finalize without a matching prepared slot")
        handle = self.selected[slot]
        handle.combine(fused_expert_output, expert_offsets=expert_offsets,
                       out=output if output.is_contiguous() else None,
                       num_tokens=output.shape[0])
        if not output.is_contiguous():
            output.copy_(handle.final_output[: output.shape[0]])
        self.routed.remove(slot)
