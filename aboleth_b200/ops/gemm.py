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


declare("ab_mx_pack_scales", [_VP, ctypes.c_longlong, _VP, _I, _I, _I, _VP, _VP])
declare("ab_gemm_e4m3_mx", [_VP] * 5 + [_I] * 6 + [_VP, _VP])
declare("ab_grouped_gemm_e4m3_mx", [_VP] * 7 + [_I] * 4 + [_VP, _VP])


def pack_scales_mx(scales: torch.Tensor, rows: int, k: int, *, weight: bool) -> torch.Tensor:
    """Power-of-two fp32 block scales -> the ue8m0 scale-factor atoms the block-scaled MMA reads.

    ``weight=False``: ``scales`` is ``[rows, k / 128]`` (one scale per row and 128-K block, what
    ``quant_fp8(round_scale=True)`` and the dispatch kernel produce; a strided view is fine).
    ``weight=True``: ``scales`` is ``[ceil(rows / 128), k / 128]`` (one per 128 x 128 block).  A weight's
    packed scales can be kept and reused.  A scale that is not a positive power of two is reported
    through :func:`check_gemm_status` (status 3), because ue8m0 cannot carry it.
    """
    assert scales.dtype == torch.float32 and scales.dim() == 2 and scales.stride(1) == 1 and k % 128 == 0
    assert scales.shape == ((-(-rows // 128) if weight else rows), k // 128), tuple(scales.shape)
    lib_bytes = _mx_scale_bytes(rows, rows, k, 1 if weight else 0)
    out = torch.empty(lib_bytes, dtype=torch.uint8, device=scales.device)
    call("ab_mx_pack_scales", ptr(scales), scales.stride(0), ptr(out), rows, k, int(weight),
         ptr(gemm_status(scales.device)), stream_ptr())
    return out


def _mx_scale_bytes(m: int, n: int, k: int, which: int) -> int:
    from ._kernels import lib
    fn = lib().ab_mx_scale_bytes
    fn.restype, fn.argtypes = ctypes.c_longlong, [ctypes.c_int] * 4
    return int(fn(m, n, k, which))


def gemm_e4m3_mx(a: torch.Tensor, a_packed: torch.Tensor, b: torch.Tensor, b_packed: torch.Tensor,
                 out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``out[M, N] = (a * sa) @ (b * sb).T`` for e4m3 operands with packed ue8m0 scales
    (:func:`pack_scales_mx`): ``tcgen05.mma.kind::mxf8f6f4.block_scale``, the scales are applied by the
    tensor core, nothing is expanded.  K must be a multiple of 128."""
    assert a.dtype == b.dtype == torch.float8_e4m3fn and a.is_cuda and a.dim() == b.dim() == 2
    assert a.stride(1) == 1 and b.stride(1) == 1 and a.shape[1] == b.shape[1] and a.shape[1] % 128 == 0
    m, k = a.shape
    n = b.shape[0]
    assert a_packed.numel() == _mx_scale_bytes(m, n, k, 0) and b_packed.numel() == _mx_scale_bytes(m, n, k, 1)
    if out is None:
        out = torch.empty(m, n, dtype=torch.bfloat16, device=a.device)
    assert out.dtype == torch.bfloat16 and out.stride(1) == 1 and out.shape == (m, n)
    call("ab_gemm_e4m3_mx", ptr(a), ptr(b), ptr(out), ptr(a_packed), ptr(b_packed), m, n, k, a.stride(0),
         b.stride(0), out.stride(0), ptr(gemm_status(a.device)), stream_ptr())
    return out


def grouped_gemm_e4m3_mx(a: torch.Tensor, a_packed: torch.Tensor, w: torch.Tensor, w_packed: torch.Tensor,
                         counts: torch.Tensor, offsets: torch.Tensor,
                         out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Per-expert block-scaled GEMM on ``tcgen05.mma.kind::mxf8f6f4.block_scale``: rows
    ``[offsets[e], offsets[e] + counts[e])`` of ``a`` times ``w[e].T``, bf16 output.

    ``a`` is e4m3 ``[rows, K]`` in expert-contiguous order with every expert's first row on a multiple
    of 128 (``expert_offsets(..., align=128)``), ``a_packed = pack_scales_mx(a_scales, rows, K,
    weight=False)``; ``w`` is e4m3 ``[E, N, K]`` (N a multiple of 128) and ``w_packed =
    pack_scales_mx(w_scales.view(E * N // 128, K // 128), E * N, K, weight=True)``.  ``counts`` /
    ``offsets`` are int32 ``[E]`` on the device and never read by the host.
    """
    fp8 = torch.float8_e4m3fn
    assert a.dtype == w.dtype == fp8 and a.is_contiguous() and w.is_contiguous()
    experts, n, k = w.shape
    rows = a.shape[0]
    assert a.shape[1] == k and k % 128 == 0 and n % 128 == 0 and counts.dtype == offsets.dtype == torch.int32
    assert a_packed.numel() == _mx_scale_bytes(rows, experts * n, k, 0)
    assert w_packed.numel() == _mx_scale_bytes(rows, experts * n, k, 1)
    if out is None:
        out = torch.empty(rows, n, dtype=torch.bfloat16, device=a.device)
    assert out.dtype == torch.bfloat16 and out.is_contiguous() and out.shape == (rows, n)
    call("ab_grouped_gemm_e4m3_mx", ptr(a), ptr(a_packed), ptr(w), ptr(w_packed), ptr(out), ptr(counts),
         ptr(offsets), experts, rows, n, k, ptr(gemm_status(a.device)), stream_ptr())
    return out


def gemm_e4m3_block_scaled(a: torch.Tensor, a_scales: torch.Tensor, b: torch.Tensor, b_scales: torch.Tensor, *,
                           a_block: tuple[int, int] = (1, 128), b_block: tuple[int, int] = (128, 128),
                           out: Optional[torch.Tensor] = None, path: str = "mx",
                           b_packed: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``out[M, N] = (a * a_scales) @ (b * b_scales).T`` for block-scaled e4m3 operands (1 x 128
    activation scales, 128 x 128 weight scales); bf16 output, fp32 accumulation.

    ``path="mx"`` (default): the scales go to the tensor core as ue8m0 and the product runs at the
    fp8 rate (:func:`gemm_e4m3_mx`).  It needs power-of-two scales (``quant_fp8(round_scale=True)``),
    the default block shapes and K a multiple of 128; pass a weight's ``b_packed`` scales to skip its
    packing.  ``path="expand"``: the operands are expanded to bf16 by :func:`dequant_block_scaled` and
    multiplied by the bf16 GEMM - any positive scales, any block shape, bf16 rate and one more pass
    over the operands.
    """
    assert a.shape[1] == b.shape[1]
    if path == "expand":
        return gemm_bf16(dequant_block_scaled(a, a_scales, block=a_block),
                         dequant_block_scaled(b, b_scales, block=b_block), out)
    if path != "mx":
        raise ValueError("path must be 'mx' or 'expand'")
    if tuple(a_block) != (1, 128) or tuple(b_block) != (128, 128) or a.shape[1] % 128:
        raise ValueError("the tensor-core path takes 1 x 128 activation and 128 x 128 weight scales and K % 128 == 0")
    m, k = a.shape
    n = b.shape[0]
    a_packed = pack_scales_mx(a_scales, m, k, weight=False)
    if b_packed is None:
        b_packed = pack_scales_mx(b_scales, n, k, weight=True)
    return gemm_e4m3_mx(a, a_packed, b, b_packed, out)
