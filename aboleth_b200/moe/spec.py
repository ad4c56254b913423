"""Shape contract of one expert-parallel MoE layer.

Fields and limits follow the reference's ``MoESpec``
(python/aboleth/moe/compiled_plan.py:31-107).
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

VALUE_TYPES = ("bf16", "f8E4M3FN")


@dataclass(frozen=True)
class MoESpec:
    capacity: int            # max tokens per rank per dispatch
    hidden: int
    top_k: int
    experts: int
    ranks: int
    value_type: str = "f8E4M3FN"
    scale_group: int = 128
    round_scale: bool = False
    quant_amax_floor: float = 1e-4

    def __post_init__(self):
        if self.ranks < 1:
            raise ValueError("ranks must be >= 1")
        if self.experts % self.ranks:
            raise ValueError("experts must divide evenly over ranks")
        if self.value_type not in VALUE_TYPES:
            raise ValueError(f"value_type must be one of {VALUE_TYPES}")
        if self.scale_group < 16 or self.scale_group & (self.scale_group - 1):
            raise ValueError("scale_group must be a power of two >= 16")
        if self.hidden % self.scale_group or self.hidden % 16:
            raise ValueError("hidden must be a multiple of scale_group and of 16")
        if not 1 <= self.top_k <= 16 or self.top_k > self.experts:
            raise ValueError("top_k must be in [1, 16] and <= experts")
        if self.experts >= 2 ** 31 or self.experts > 512:
            raise ValueError("at most 512 experts are supported")
        if self.capacity < 1 or self.capacity * self.hidden * 2 >= 2 ** 31:
            raise ValueError("capacity * hidden * 2 must stay below 2^31")
        if self.ranks > 32:
            raise ValueError("at most 32 ranks are supported")

    @property
    def fp8(self) -> bool:
        return self.value_type == "f8E4M3FN"

    @property
    def scale_cols(self) -> int:
        return self.hidden // self.scale_group if self.fp8 else 0

    @property
    def metadata_words(self) -> int:
        return 2 + 2 * self.top_k + self.scale_cols

    @property
    def row_bytes(self) -> int:
        return self.hidden * (1 if self.fp8 else 2)

    @property
    def payload_dtype(self) -> torch.dtype:
        return torch.float8_e4m3fn if self.fp8 else torch.bfloat16

    @property
    def experts_per_rank(self) -> int:
        return self.experts // self.ranks

    def owners(self, placement: str = "linear") -> list[int]:
        """Expert -> owning rank (``linear`` blocks or ``round_robin``)."""
        if placement == "linear":
            return [e // self.experts_per_rank for e in range(self.experts)]
        if placement == "round_robin":
            return [e % self.ranks for e in range(self.experts)]
        raise ValueError("placement must be 'linear' or 'round_robin'")
