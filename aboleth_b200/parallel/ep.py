"""Expert parallelism: one MoE layer's dispatch -> experts -> combine over a World.

This is the call a user of the framework makes.  ``ExpertParallelLayer`` owns
one :class:`~aboleth_b200.moe.NativeMoESlot` and runs two communication
launches per layer around a caller-supplied expert stage.
"""
from __future__ import annotations

from typing import Callable, Optional

import torch

from ..moe import DispatchResult, MoESpec, NativeMoESlot
from ..moe.compiled_plan import compile_moe_plan
from ..ops import expert_offsets, standin_expert
from ..utils import host_range
from ..world import World

ExpertFn = Callable[[DispatchResult, torch.Tensor], object]


class ExpertParallelLayer:
    def __init__(self, world: World, spec: MoESpec, *, tag: str = "ep", grid: Optional[int] = None):
        self.world, self.spec = world, spec
        # The compiled plan of this shape decides the launch geometry (latency or throughput path,
        # sender warps, readiness block) and confirms that inputs and expert output need no copy.
        self.plan = compile_moe_plan(spec, world)
        self.slot = NativeMoESlot.create(world, spec, tag=tag, grid=grid, plan=self.plan)
        self._host_result = torch.zeros(4, dtype=torch.int64).pin_memory()
        self._staging: Optional[list] = None
        self._grouped: Optional[torch.Tensor] = None

    def standin_experts(self, result: DispatchResult, y: torch.Tensor) -> None:
        """The benchmark's expert stage, ``f_e(x) = x * (1 + (e mod 7)/8)``, gate-weighted here:
        one partial row per received record, which the combine sums unweighted."""
        s = self.spec
        standin_expert(result.expert_input, result.expert_scales, y, result.expert_ids,
                       result.expert_weights, result.expert_pos, result.recv_counts,
                       world=s.ranks, capacity=s.capacity, group=s.scale_group)
        return None

    def standin_experts_grouped(self, result: DispatchResult, y: torch.Tensor):
        """The same experts behind an expert-contiguous output, as a grouped expert GEMM leaves it:
        one UNWEIGHTED row per (record, choice) at ``offsets[expert] + position``.  Returns the
        offsets, so the combine kernel gathers each record's rows and applies the gates itself."""
        s = self.spec
        offsets, _ = expert_offsets(result.expert_counts_by_source)
        rows = s.ranks * s.capacity * min(s.top_k, s.experts_per_rank)
        if self._grouped is None or self._grouped.shape[0] < rows:
            self._grouped = torch.empty(rows, s.hidden, dtype=torch.bfloat16, device=y.device)
        standin_expert(result.expert_input, result.expert_scales, self._grouped, result.expert_ids,
                       result.expert_weights, result.expert_pos, result.recv_counts,
                       world=s.ranks, capacity=s.capacity, group=s.scale_group, offsets=offsets)
        return offsets, self._grouped

    def forward(self, tokens: torch.Tensor, logits: torch.Tensor, experts: Optional[ExpertFn] = None,
                *, renormalize: bool = False, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``tokens`` bf16 ``[n, hidden]`` and router ``logits`` fp32 ``[n, experts]`` on the device.

        ``experts(result, y)`` either fills ``y`` (one gate-weighted partial row per
        received record) and returns None, or returns int32 ``[experts]`` offsets when
        it wrote ``y`` in expert-contiguous order and wants the combine kernel to apply
        the gates, or ``(offsets, rows)`` when it wrote its own buffer ``rows`` that way.
        """
        with host_range("ep.dispatch"):
            result = self.slot.dispatch(tokens, logits=logits, renormalize=renormalize)
        y = self.slot.expert_output
        with host_range("ep.experts"):
            offsets = (experts or self.standin_experts)(result, y)
        if isinstance(offsets, tuple):  # (offsets, rows): the stage owns its output buffer
            offsets, y = offsets
        with host_range("ep.combine"):
            return self.slot.combine(y, expert_offsets=offsets, out=out)

    def forward_from_host(self, tokens_host: torch.Tensor, logits_host: torch.Tensor,
                          experts: Optional[ExpertFn] = None, *,
                          prefetch: Optional[tuple[torch.Tensor, torch.Tensor]] = None) -> torch.Tensor:
        """Same, from pinned host tensors; returns a pinned int64[4] summary
        (status, detail, overflow, output checksum bits).  The caller synchronises the
        stream before reading it.

        ``prefetch=(tokens, logits)`` names the inputs of the NEXT call: their host-to-device
        copy is enqueued on a side stream before this call's kernels, so it runs under them
        (two staging buffers alternate).  The next call must then pass those same tensors.
        """
        dev = self.world.torch_device
        if self._staging is None or self._staging[0][0].shape != tokens_host.shape:
            self._staging = [(torch.empty_like(tokens_host, device=dev),
                              torch.empty_like(logits_host, device=dev)) for _ in range(2)]
            self._summary = torch.zeros(4, dtype=torch.int64, device=dev)
            self._copy_stream = torch.cuda.Stream(device=dev)
            self._copied = [torch.cuda.Event() for _ in range(2)]
            self._consumed = [None, None]
            self._current, self._prefetched = 0, None
        main = torch.cuda.current_stream()
        cur = self._current
        x_dev, l_dev = self._staging[cur]
        if self._prefetched == (tokens_host.data_ptr(), logits_host.data_ptr()):
            main.wait_event(self._copied[cur])          # copied by the previous call's prefetch
        else:
            x_dev.copy_(tokens_host, non_blocking=True)
            l_dev.copy_(logits_host, non_blocking=True)
        self._prefetched = None
        if prefetch is not None:
            nxt = cur ^ 1
            if self._consumed[nxt] is not None:
                self._copy_stream.wait_event(self._consumed[nxt])  # its last reader has finished
            with torch.cuda.stream(self._copy_stream):
                self._staging[nxt][0].copy_(prefetch[0], non_blocking=True)
                self._staging[nxt][1].copy_(prefetch[1], non_blocking=True)
                self._copied[nxt].record(self._copy_stream)
            self._prefetched = (prefetch[0].data_ptr(), prefetch[1].data_ptr())
        out = self.forward(x_dev, l_dev, experts)
        self._consumed[cur] = torch.cuda.Event()
        self._consumed[cur].record(main)
        self._current = cur ^ 1
        self._summary[:2].copy_(self.slot.status)
        self._summary[2:3].copy_(self.slot.overflow)
        self._summary[3:4].copy_(out.view(torch.int16).to(torch.int64).sum().view(1))
        self._host_result.copy_(self._summary, non_blocking=True)
        return self._host_result

    @property
    def h2d_bytes(self) -> int:
        s = self.spec
        return 0 if self._staging is None else (
            self._staging[0][0].numel() * 2 + self._staging[0][1].numel() * 4)

    def check(self) -> None:
        self.slot.check()
