"""Standalone MoE pieces: fp8 1xG quantisation, router top-k, permute/unpermute.

Kernels: csrc/kernels/moe_kernels.cu.  The fused dispatch and combine live in
``aboleth_b200.moe``.
"""
from __future__ import annotations

from typing import Optional

import torch

from ._kernels import call, ptr, stream_ptr


def quant_fp8(x: torch.Tensor, *, group: int = 128, amax_floor: float = 1e-4,
              round_scale: bool = False) -> tuple[torch.Tensor, torch.Tensor]:
    """bf16 ``[rows, hidden]`` -> (e4m3 ``[rows, hidden]``, fp32 scales ``[rows, hidden/group]``).

    ``scale = max(amax, floor) / 448`` (rounded up to a power of two on request),
    ``q = clamp(x / scale, +-448)`` rounded to nearest even.
    """
    assert x.dtype == torch.bfloat16 and x.is_cuda and x.is_contiguous() and x.dim() == 2
    rows, hidden = x.shape
    q = torch.empty(rows, hidden, dtype=torch.float8_e4m3fn, device=x.device)
    scales = torch.empty(rows, hidden // group, dtype=torch.float32, device=x.device)
    call("ab_quant_fp8", ptr(x), ptr(q), ptr(scales), rows, hidden, group, amax_floor,
         int(round_scale), stream_ptr())
    return q, scales


def router_topk(logits: torch.Tensor, top_k: int, *, renormalize: bool = False
                ) -> tuple[torch.Tensor, torch.Tensor]:
    """fp32 ``[tokens, experts]`` -> (int32 ids ``[tokens, k]``, fp32 softmax weights)."""
    assert logits.dtype == torch.float32 and logits.is_cuda and logits.is_contiguous()
    tokens, experts = logits.shape
    ids = torch.empty(tokens, top_k, dtype=torch.int32, device=logits.device)
    weights = torch.empty(tokens, top_k, dtype=torch.float32, device=logits.device)
    call("ab_router_topk", ptr(logits), ptr(ids), ptr(weights), tokens, experts, top_k,
         int(renormalize), stream_ptr())
    return ids, weights


def expert_offsets(counts: torch.Tensor, *, align: int = 1) -> tuple[torch.Tensor, torch.Tensor]:
    """Row offsets of the expert-contiguous layout -> (offsets, total rows).

    ``counts`` is int32 ``[sources, experts]`` (``DispatchResult.expert_counts_by_source``) or
    ``[experts]``.  The group of expert ``e`` starts at the exclusive scan of the experts' totals
    (each rounded up to ``align``); inside it the rows of source ``s`` follow those of the sources
    before it.  ``offsets`` has the shape of ``counts``; ``offsets[0]`` (or ``offsets`` itself for
    1-D counts) is the start of every expert's group, which is what a grouped GEMM needs.
    """
    assert counts.dtype == torch.int32 and counts.is_contiguous() and counts.dim() in (1, 2)
    sources = counts.shape[0] if counts.dim() == 2 else 1
    offsets = torch.empty_like(counts)
    total = torch.empty(1, dtype=torch.int32, device=counts.device)
    call("ab_expert_offsets", ptr(counts), ptr(offsets), ptr(total), sources, counts.shape[-1], align,
         stream_ptr())
    return offsets, total


def _offset_stride(offsets: Optional[torch.Tensor]) -> int:
    """0 for one offset per expert, ``experts`` for one per (source rank, expert)."""
    if offsets is None or offsets.dim() == 1:
        return 0
    assert offsets.dim() == 2 and offsets.is_contiguous()
    return int(offsets.shape[1])


def permute(src: torch.Tensor, dst: torch.Tensor, expert_ids: torch.Tensor,
            expert_pos: torch.Tensor, offsets: torch.Tensor, recv_counts: torch.Tensor, *,
            world: int, capacity: int, src_scales: Optional[torch.Tensor] = None,
            dst_scales: Optional[torch.Tensor] = None,
            perm_row: Optional[torch.Tensor] = None) -> None:
    """Gather received rows into expert-contiguous order (``dst[offsets[source, e] + pos] = src[row]``;
    ``offsets`` from :func:`expert_offsets` over the per-source counts)."""
    top_k = expert_ids.shape[-1]
    row_bytes = src.shape[-1] * src.element_size()
    cols = 0 if src_scales is None else src_scales.shape[-1]
    stride = 0 if src_scales is None else _row_stride(src_scales)
    call("ab_permute", ptr(src), ptr(dst), ptr(src_scales), ptr(dst_scales), ptr(expert_ids),
         ptr(expert_pos), ptr(offsets), ptr(recv_counts), ptr(perm_row), world, capacity, top_k,
         row_bytes, cols, stride, _offset_stride(offsets), stream_ptr())


def unpermute(y: torch.Tensor, out: torch.Tensor, expert_ids: torch.Tensor,
              expert_pos: torch.Tensor, expert_weights: torch.Tensor, offsets: torch.Tensor,
              recv_counts: torch.Tensor, *, world: int, capacity: int) -> None:
    """``out[row] = sum_j w[row, j] * y[offsets[id] + pos]`` in fp32, bf16 result."""
    call("ab_unpermute", ptr(y), ptr(out), ptr(expert_ids), ptr(expert_pos), ptr(expert_weights),
         ptr(offsets), ptr(recv_counts), world, capacity, expert_ids.shape[-1], y.shape[-1],
         _offset_stride(offsets), stream_ptr())


def _row_stride(scales: torch.Tensor) -> int:
    """Row stride (elements) of a 2-D scale tensor whose rows are contiguous.  The scales of a
    dispatch are a strided view of the received metadata rows, not a packed array."""
    if scales.dim() != 2 or scales.stride(1) != 1:
        raise ValueError("scales must be 2-D with contiguous rows")
    return int(scales.stride(0))


def standin_expert(payload: torch.Tensor, scales: Optional[torch.Tensor], y: torch.Tensor,
                   expert_ids: torch.Tensor, expert_weights: torch.Tensor,
                   expert_pos: torch.Tensor, recv_counts: torch.Tensor, *, world: int,
                   capacity: int, group: int, offsets: Optional[torch.Tensor] = None) -> None:
    """Benchmark expert ``f_e(x) = x * (1 + (e mod 7) / 8)``.

    Without ``offsets``: record layout, gate-weighted (one partial row per received record).
    With ``offsets`` (int32 ``[ranks, experts]``): expert-contiguous layout, one unweighted row per
    (record, choice) at ``offsets[source, id] + pos`` - what a grouped expert GEMM leaves behind.
    """
    fp8 = payload.dtype == torch.float8_e4m3fn
    stride = 0 if scales is None else _row_stride(scales)
    call("ab_standin_expert", ptr(payload), ptr(scales), stride, ptr(y), ptr(expert_ids),
         ptr(expert_weights), ptr(expert_pos), ptr(offsets), ptr(recv_counts), world, capacity,
         expert_ids.shape[-1], y.shape[-1], group, int(fp8), _offset_stride(offsets), stream_ptr())
