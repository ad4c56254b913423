"""Plain PyTorch fp32 restatements of the MoE kernels, used as test oracles.

Quantisation rule and tolerances follow the reference
(python/aboleth/moe/kernels.py:78-102; experiments/dsl/moe/moe_common.py:72-140).
"""
from __future__ import annotations

import torch

FP8_MAX = 448.0


def quant_fp8_reference(x: torch.Tensor, group: int = 128, amax_floor: float = 1e-4,
                        round_scale: bool = False) -> tuple[torch.Tensor, torch.Tensor]:
    rows, hidden = x.shape
    xf = x.float().view(rows, hidden // group, group)
    amax = xf.abs().amax(dim=-1).clamp_min(amax_floor)
    # IEEE division (torch would multiply by a rounded reciprocal for a scalar divisor).
    scale = (amax.double() / FP8_MAX).float()
    if round_scale:
        bits = scale.view(torch.int32)
        bumped = (bits & ~0x7FFFFF) + 0x800000
        scale = torch.where((bits & 0x7FFFFF) != 0, bumped, bits).view(torch.float32)
    q = (xf / scale.unsqueeze(-1)).clamp(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn)
    return q.view(rows, hidden), scale


def dequant_fp8_reference(q: torch.Tensor, scales: torch.Tensor, group: int = 128) -> torch.Tensor:
    rows, hidden = q.shape
    return (q.float().view(rows, hidden // group, group) * scales.unsqueeze(-1)).view(rows, hidden)


def router_reference(logits: torch.Tensor, top_k: int, renormalize: bool = False):
    probs = torch.softmax(logits.float(), dim=-1)
    weights, ids = torch.topk(probs, top_k, dim=-1)
    if renormalize:
        weights = weights / weights.sum(dim=-1, keepdim=True)
    return ids.to(torch.int32), weights


def standin_layer_reference(x: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor, *,
                            fp8: bool, group: int = 128, amax_floor: float = 1e-4,
                            round_scale: bool = False) -> tuple[torch.Tensor, torch.Tensor]:
    """Output of dispatch -> stand-in experts -> combine for one rank's tokens.

    Returns (expected fp32 ``[n, hidden]``, per-row tolerance).  The stand-in
    expert is ``f_e(x) = x * (1 + (e mod 7) / 8)``; invalid ids (< 0) are skipped.
    The expectation is computed from the UNQUANTISED activations; the tolerance
    (``coefficient * amax / 16`` for e4m3, ``/ 128`` for bf16, plus 1e-3) is what
    absorbs the quantisation, as in the reference's benchmark oracle.
    """
    xf = x.float()
    valid = ids >= 0
    coef = (weights * (1.0 + (ids.clamp_min(0) % 7).float() / 8.0) * valid).sum(dim=-1)
    expected = xf * coef.unsqueeze(-1)
    amax = x.float().abs().amax(dim=-1)
    tolerance = coef.abs() * amax * (1.0 / 16 if fp8 else 1.0 / 128) + 1e-3
    return expected, tolerance
