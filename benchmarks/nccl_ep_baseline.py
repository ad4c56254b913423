"""Baseline arm of the expert-parallel layer: the same dispatch -> experts -> combine written
with PyTorch operators and NCCL collectives only.  It exists to be measured against, never to be
used: none of the framework's kernels or transports is on this path.

Dispatch: per-group fp8 e4m3 quantisation with torch operators, records deduplicated per
(token, destination rank), one ``all_to_all_single`` for the record counts (read back on the
host, as the split sizes of the next calls), one for the payload rows and one for the metadata
rows (token index, expert ids, gate weights, scales).  Experts: the stand-in
``f_e(x) = x * (1 + (e mod 7) / 8)`` with the gates applied on the expert side.  Combine: one
``all_to_all_single`` of bf16 partial rows back to the source ranks and an ``index_add_`` per
token.  Same shapes, same timing rules and the same fp32 oracle as the fused kernels.
"""
from __future__ import annotations

import statistics

import torch
import torch.distributed as dist

FP8_MAX = 448.0


class NcclEpLayer:
    def __init__(self, *, rank: int, world: int, hidden: int, experts: int, top_k: int, group: int,
                 amax_floor: float = 1e-4):
        self.rank, self.world = rank, world
        self.hidden, self.experts, self.top_k, self.group = hidden, experts, top_k, group
        self.amax_floor = amax_floor
        self.per_rank = experts // world
        self.cols = hidden // group

    # -- dispatch ---------------------------------------------------------------------------
    def dispatch(self, x: torch.Tensor, logits: torch.Tensor) -> dict:
        t, dev = x.shape[0], x.device
        probs = torch.softmax(logits.float(), dim=-1)
        weights, ids = torch.topk(probs, self.top_k, dim=-1)
        xf = x.float().view(t, self.cols, self.group)
        scale = xf.abs().amax(dim=-1).clamp_min(self.amax_floor) / FP8_MAX
        q = (xf / scale.unsqueeze(-1)).clamp(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn).view(t, self.hidden)
        owner = ids // self.per_rank                                   # [t, k]
        hit = torch.zeros(t, self.world, dtype=torch.bool, device=dev)
        hit.scatter_(1, owner, True)
        dest, token = hit.t().nonzero(as_tuple=True)                    # sorted by destination, then token
        send_counts = hit.sum(dim=0).to(torch.int64)
        recv_counts = torch.empty_like(send_counts)
        dist.all_to_all_single(recv_counts, send_counts)
        send_split, recv_split = send_counts.tolist(), recv_counts.tolist()   # host read-back
        n_recv = sum(recv_split)
        # metadata row: token, expert ids (-1 where another rank owns the choice), weights, scales
        mine = owner[token] == dest.unsqueeze(-1)                       # [records, k]
        meta = torch.cat([token.view(-1, 1).float(),
                          torch.where(mine, ids[token], torch.full_like(ids[token], -1)).float(),
                          torch.where(mine, weights[token], torch.zeros_like(weights[token])),
                          scale[token]], dim=1).contiguous()
        payload = q[token].view(torch.uint8).contiguous()
        got_payload = torch.empty(n_recv, self.hidden, dtype=torch.uint8, device=dev)
        got_meta = torch.empty(n_recv, meta.shape[1], dtype=torch.float32, device=dev)
        dist.all_to_all_single(got_payload, payload, recv_split, send_split)
        dist.all_to_all_single(got_meta, meta, recv_split, send_split)
        return {"payload": got_payload.view(torch.float8_e4m3fn), "meta": got_meta, "token": token,
                "send_split": send_split, "recv_split": recv_split, "ids": ids, "weights": weights,
                "tokens": t}

    # -- stand-in experts (gate applied here) ----------------------------------------------------
    def experts_standin(self, state: dict) -> torch.Tensor:
        k = self.top_k
        meta = state["meta"]
        ids = meta[:, 1:1 + k]
        w = meta[:, 1 + k:1 + 2 * k]
        scales = meta[:, 1 + 2 * k:]
        coef = (w * (1.0 + torch.remainder(ids.clamp_min(0), 7) / 8.0) * (ids >= 0)).sum(dim=-1)
        xq = state["payload"].float().view(-1, self.cols, self.group) * scales.unsqueeze(-1)
        return (xq.view(-1, self.hidden) * coef.unsqueeze(-1)).to(torch.bfloat16)

    # -- combine ---------------------------------------------------------------------------------
    def combine(self, state: dict, y: torch.Tensor) -> torch.Tensor:
        back = torch.empty(sum(state["send_split"]), self.hidden, dtype=torch.bfloat16, device=y.device)
        dist.all_to_all_single(back, y, state["send_split"], state["recv_split"])
        out = torch.zeros(state["tokens"], self.hidden, dtype=torch.float32, device=y.device)
        out.index_add_(0, state["token"], back.float())
        return out.to(torch.bfloat16)


def measure(x_list, logits_list, *, rank: int, world: int, hidden: int, experts: int, top_k: int,
            group: int, steps: int, sync_ranks, device_max_vector, oracle) -> dict:
    """Phase times (median, max over ranks) of the NCCL arm on the given inputs, and the number of
    output rows outside the oracle's tolerance."""
    layer = NcclEpLayer(rank=rank, world=world, hidden=hidden, experts=experts, top_k=top_k, group=group)
    ev = lambda: torch.cuda.Event(enable_timing=True)  # noqa: E731
    d_ms, c_ms, s_ms = [], [], []
    out = None
    for it in range(steps + 2):
        i = it % len(x_list)
        sync_ranks(True)
        e0, e1, e2, e3 = ev(), ev(), ev(), ev()
        e0.record()
        state = layer.dispatch(x_list[i], logits_list[i])
        e1.record()
        y = layer.experts_standin(state)
        e2.record()
        out = layer.combine(state, y)
        e3.record()
        torch.cuda.synchronize()
        if it >= 2:
            d_ms.append(e0.elapsed_time(e1))
            c_ms.append(e2.elapsed_time(e3))
            s_ms.append(e0.elapsed_time(e3))
    state = layer.dispatch(x_list[0], logits_list[0])
    out = layer.combine(state, layer.experts_standin(state)).float()
    expected, tol = oracle(x_list[0], state["ids"], state["weights"])
    bad = int((~((out - expected).abs().amax(dim=-1) <= tol)).sum().item())
    med = lambda v: statistics.median(device_max_vector(v, True))  # noqa: E731
    return {"impl": "torch operators + NCCL all_to_all_single (baseline only)",
            "dispatch_us": med(d_ms) * 1e3, "combine_us": med(c_ms) * 1e3, "step_us": med(s_ms) * 1e3,
            "verify_errors": bad, "steps": steps,
            "note": "dispatch includes the torch fp8 quantisation, the count exchange and its host "
                    "read-back; combine includes the per-token index_add"}
