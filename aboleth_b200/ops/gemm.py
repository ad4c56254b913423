"""bf16 and e4m3 GEMMs on tcgen05 / TMEM / TMA (kernels: csrc/kernels/gemm_kernels.cu)."""
from __future__ import annotations

from typing import Optional

import torch

import ctypes

from ._kernels import _I, _VP, call, declare, ptr, stream_ptr

declare("ab_gemm_bf16", [_VP, _VP, _VP] + [_I] * 6 + [_VP, _VP])
declare("ab_grouped_gemm_bf16", [_VP] * 5 + [_I] * 4 + [_VP, _VP])
declare("ab_gemm_e4m3", [_VP, _VP, _VP] + [_I] * 6 + [ctypes.c_float, _VP, _VP])

_status: dict[torch.device, torch.Tensor] = {}


def gemm_status(device) -> torch.Tensor:
    """int64 status words shared by the GEMM launches on ``device`` (word 0: status, 0 = ok; word 1: detail;
    words 2..15: cycle counters the kernels fill when built with ``-DAB_GEMM_TRACE``)."""
    device = torch.device(device)
    if device.type == "cuda" and device.index is None:  # "cuda" means the current device
        device = torch.device("cuda", torch.cuda.current_device())
    if device not in _status:
        _status[device] = torch.zeros(16, dtype=torch.int64, device=device)
    return _status[device]


def check_gemm_status(device) -> None:
    status = gemm_status(device)[:2].tolist()
    if status[0]:
        raise RuntimeError(f"GEMM kernel gave up waiting (status {status[0]}, detail {status[1]:#x})")


def gemm_bf16(a: torch.Tensor, b: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``out[M, N] = a[M, K] @ b[N, K].T`` with fp32 accumulation in tensor memory."""
    assert a.dtype == b.dtype == torch.bfloat16 and a.is_cuda and a.dim() == b.dim() == 2
    assert a.stride(1) == 1 and b.stride(1) == 1 and a.shape[1] == b.shape[1]
    m, k = a.shape
    n = b.shape[0]
    if out is None:
        out = torch.empty(m, n, dtype=torch.bfloat16, device=a.device)
    assert out.stride(1) == 1 and out.shape == (m, n)
    call("ab_gemm_bf16", ptr(a), ptr(b), ptr(out), m, n, k, a.stride(0), b.stride(0), out.stride(0),
         ptr(gemm_status(a.device)), stream_ptr())
    return out


def gemm_e4m3(a: torch.Tensor, b: torch.Tensor, out: Optional[torch.Tensor] = None, *,
              alpha: float = 1.0) -> torch.Tensor:
    """``out[M, N] = alpha * a[M, K] @ b[N, K].T`` for ``torch.float8_e4m3fn`` operands (per-tensor
    scaling: pass the product of the two dequantisation scales as ``alpha``); bf16 output, fp32
    accumulation in tensor memory, ``kind::f8f6f4`` on CTA pairs."""
    assert a.dtype == b.dtype == torch.float8_e4m3fn and a.is_cuda and a.dim() == b.dim() == 2
    assert a.stride(1) == 1 and b.stride(1) == 1 and a.shape[1] == b.shape[1]
    m, k = a.shape
    n = b.shape[0]
    if out is None:
        out = torch.empty(m, n, dtype=torch.bfloat16, device=a.device)
    assert out.dtype == torch.bfloat16 and out.stride(1) == 1 and out.shape == (m, n)
    call("ab_gemm_e4m3", ptr(a), ptr(b), ptr(out), m, n, k, a.stride(0), b.stride(0), out.stride(0),
         float(alpha), ptr(gemm_status(a.device)), stream_ptr())
    return out


def grouped_gemm_bf16(a: torch.Tensor, w: torch.Tensor, counts: torch.Tensor,
                      offsets: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Per-expert GEMM: rows ``[offsets[e], offsets[e]+counts[e])`` of ``a`` times ``w[e].T``.

    ``a`` is bf16 ``[rows, K]`` in expert-contiguous order, ``w`` bf16 ``[E, N, K]``,
    ``counts`` / ``offsets`` int32 ``[E]`` on the device (never read by the host).
    """
    assert a.dtype == w.dtype == torch.bfloat16 and a.is_contiguous() and w.is_contiguous()
    experts, n, k = w.shape
    assert a.shape[1] == k and counts.dtype == offsets.dtype == torch.int32
    if out is None:
        out = torch.empty(a.shape[0], n, dtype=torch.bfloat16, device=a.device)
    call("ab_grouped_gemm_bf16", ptr(a), ptr(w), ptr(out), ptr(counts), ptr(offsets), experts,
         a.shape[0], n, k, ptr(gemm_status(a.device)), stream_ptr())
    return out


declare("ab_dequant_block_scaled", [_VP, _VP, _VP] + [_I] * 4 + [ctypes.c_longlong] * 2 + [_I, _VP])


def dequant_block_scaled(q: torch.Tensor, scales: torch.Tensor, *, block: tuple[int, int] = (1, 128),
                         out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``out[r, c] = q[r, c] * scales[r // block[0], c // block[1]]`` as bf16.

    ``q`` is ``torch.float8_e4m3fn`` ``[rows, cols]``; ``scales`` is fp32
    ``[ceil(rows / block[0]), cols / block[1]]``: ``(1, 128)`` for activations (what
    :func:`aboleth_b200.ops.moe_ops.quant_fp8` and the dispatch kernel produce), ``(128, 128)``
    for weights.  Exact when the scales are powers of two.
    """
    assert q.dtype == torch.float8_e4m3fn and q.is_cuda and q.dim() == 2 and q.stride(1) == 1
    assert scales.dtype == torch.float32 and scales.dim() == 2 and scales.stride(1) == 1
    rows, cols = q.shape
    row_block, col_block = block
    assert scales.shape[0] == -(-rows // row_block) and scales.shape[1] == -(-cols // col_block), \
        f"scales {tuple(scales.shape)} do not cover {tuple(q.shape)} in blocks of {block}"
    if out is None:
        out = torch.empty(rows, cols, dtype=torch.bfloat16, device=q.device)
    assert out.dtype == torch.bfloat16 and out.shape == (rows, cols) and out.stride(1) == 1
    call("ab_dequant_block_scaled", ptr(q), ptr(scales), ptr(out), rows, cols, row_block, col_block,
         q.stride(0), out.stride(0), scales.stride(0), stream_ptr())
    return out


def gemm_e4m3_block_scaled(a: torch.Tensor, a_scales: torch.Tensor, b: torch.Tensor, b_scales: torch.Tensor, *,
                           a_block: tuple[int, int] = (1, 128), b_block: tuple[int, int] = (128, 128),
                           out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``out[M, N] = (a * a_scales) @ (b * b_scales).T`` for block-scaled e4m3 operands (1 x 128
    activation scales, 128 x 128 weight scales by default); bf16 output, fp32 accumulation.

    The operands are expanded to bf16 by :func:`dequant_block_scaled` and multiplied by the
    tcgen05 bf16 GEMM: the result carries the block scales exactly (for power-of-two scales) at
    bf16 tensor-core rate and fp8 storage.  A weight that is used repeatedly should be expanded
    once with :func:`dequant_block_scaled` and passed to :func:`gemm_bf16`.
    """
    assert a.shape[1] == b.shape[1]
    return gemm_bf16(dequant_block_scaled(a, a_scales, block=a_block),
                     dequant_block_scaled(b, b_scales, block=b_block), out)
