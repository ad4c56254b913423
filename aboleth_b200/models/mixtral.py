"""Mixtral-style sparse-MoE decoder served with expert parallelism (EP == DP, TP 1).

Attention, norms and the router are replicated; every rank keeps ``experts / ranks``
experts.  A MoE layer is: router logits -> top-k (own kernel) -> fused dispatch ->
permute -> grouped expert GEMMs on tcgen05 (gate/up, SiLU-mul, down) -> fused combine
with the gate weights applied inside the kernel.  With ``fp8_experts=True`` the tokens are
dispatched as e4m3 with 1 x 128 power-of-two scales, the expert weights are e4m3 with 128 x 128
scales, and both grouped GEMMs run on the block-scaled tensor-core path (DeepSeek-V3's recipe);
nothing is expanded to bf16 on the way.  Attention uses PyTorch's
scaled-dot-product attention with a static KV cache; it is not one of this
framework's kernels.

Weights are random-init from a seed (there are no checkpoints on an offline box).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch
import torch.nn.functional as F

from ..integrations.vllm_all2all import AbolethAll2AllManager, AbolethPrepareAndFinalize
from ..ops import (expert_offsets, grouped_gemm_bf16, grouped_gemm_e4m3_mx, pack_scales_mx, permute, quant_fp8,
                   router_topk)
from ..world import World


@dataclass(frozen=True)
class MixtralConfig:
    layers: int = 32
    hidden: int = 4096
    experts: int = 8
    top_k: int = 2
    ffn: int = 14336
    heads: int = 32
    kv_heads: int = 8
    vocab: int = 32000
    rope_theta: float = 1e6
    rms_eps: float = 1e-5
    max_seq: int = 2048

    @property
    def head_dim(self) -> int:
        return self.hidden // self.heads


def _rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)).to(x.dtype) * weight


_ROPE_INV: dict = {}


def _rope(x: torch.Tensor, positions: torch.Tensor, theta: float) -> torch.Tensor:
    # x: [B, heads, S, D]; positions: [B, S]
    d = x.shape[-1]
    key = (d, theta, x.device)
    inv = _ROPE_INV.get(key)
    if inv is None:
        inv = _ROPE_INV[key] = 1.0 / (theta ** (torch.arange(0, d, 2, device=x.device,
                                                                 dtype=torch.float32) / d))
    ang = positions[:, None, :, None].float() * inv
    cos, sin = ang.cos(), ang.sin()
    x1, x2 = x[..., 0::2].float(), x[..., 1::2].float()
    out = torch.stack((x1 * cos - x2 * sin, x1 * sin + x2 * cos), dim=-1).flatten(-2)
    return out.to(x.dtype)


class MixtralEP:
    def __init__(self, config: MixtralConfig, world: World, *, max_batch: int, max_prompt: int,
                 seed: int = 0, manager: Optional[AbolethAll2AllManager] = None, cpu_group=None,
                 fp8_experts: bool = False):
        c = self.config = config
        self.fp8_experts = fp8_experts
        if fp8_experts and (c.hidden % 128 or c.ffn % 128):
            raise ValueError("fp8 experts need hidden and ffn sizes that are multiples of 128")
        self.world = world
        dev = self.device = world.torch_device
        ranks = world.world_size
        if c.experts % ranks:
            raise ValueError("experts must divide evenly over ranks")
        self.local_experts = c.experts // ranks
        self.first_expert = world.rank * self.local_experts
        g = torch.Generator(device=dev).manual_seed(seed)  # same seed: replicated weights agree

        def w(*shape, scale=0.02, gen=g):
            return (torch.randn(*shape, generator=gen, device=dev) * scale).to(torch.bfloat16)

        qkv = (c.heads + 2 * c.kv_heads) * c.head_dim
        self.embed = w(c.vocab, c.hidden)
        self.lm_head = w(c.vocab, c.hidden)
        self.final_norm = torch.ones(c.hidden, dtype=torch.bfloat16, device=dev)
        ge = torch.Generator(device=dev).manual_seed(seed * 1000 + 17 + world.rank)  # experts differ per rank
        self.layers = []
        for _ in range(c.layers):
            self.layers.append({
                "attn_norm": torch.ones(c.hidden, dtype=torch.bfloat16, device=dev),
                "wqkv": w(qkv, c.hidden), "wo": w(c.hidden, c.heads * c.head_dim),
                "ffn_norm": torch.ones(c.hidden, dtype=torch.bfloat16, device=dev),
                "router": w(c.experts, c.hidden),
                "w13": w(self.local_experts, 2 * c.ffn, c.hidden, gen=ge),
                "w2": w(self.local_experts, c.hidden, c.ffn, gen=ge),
            })
        self.max_batch, self.max_prompt = max_batch, max_prompt
        self.capacity = max_batch * max_prompt
        self.manager = manager or AbolethAll2AllManager(cpu_group, world=world)
        facts = dict(dtype=torch.bfloat16, num_experts=c.experts, num_local_experts=self.local_experts,
                     num_max_tokens_per_rank=self.capacity, hidden=c.hidden, num_topk=c.top_k,
                     decode_bound=max_batch, min_tokens_per_rank=max_batch)
        if fp8_experts:
            facts.update(quant_dtype=torch.float8_e4m3fn, quant_block_shape=[128, 128], quant_round_scale=True)
        self.moe = AbolethPrepareAndFinalize(self.manager, facts, layer_name="moe")
        rows = ranks * self.capacity * min(c.top_k, self.local_experts)
        if fp8_experts:
            # Every expert's group starts on a 128-row boundary (a scale-factor atom covers 128 rows).
            rows = (rows + self.local_experts * 127 + 127) // 128 * 128
            for layer in self.layers:
                for name in ("w13", "w2"):
                    layer[name + "_q"], layer[name + "_scales"], layer[name + "_packed"] = \
                        self._quantise_weight(layer[name])
            self.x_perm = torch.zeros(rows, c.hidden, dtype=torch.float8_e4m3fn, device=dev)
            # Padding rows are never written; ones / zeros keep their scales and activations finite.
            self.x_scales = torch.ones(rows, c.hidden // 128, dtype=torch.float32, device=dev)
            self.h13 = torch.zeros(rows, 2 * c.ffn, dtype=torch.bfloat16, device=dev)
        else:
            self.x_perm = torch.zeros(rows, c.hidden, dtype=torch.bfloat16, device=dev)
            self.h13 = torch.empty(rows, 2 * c.ffn, dtype=torch.bfloat16, device=dev) \
                if rows * c.ffn < 2 ** 31 else None
        self.y_perm = torch.empty(rows, c.hidden, dtype=torch.bfloat16, device=dev)
        self.kv = torch.zeros(c.layers, 2, max_batch, c.kv_heads, c.max_seq, c.head_dim,
                              dtype=torch.bfloat16, device=dev)

    @staticmethod
    def _quantise_weight(w: torch.Tensor):
        """bf16 ``[E, N, K]`` -> (e4m3 weights, fp32 128 x 128 power-of-two scales ``[E, N/128, K/128]``,
        the scales packed for the tensor core)."""
        experts, n, k = w.shape
        blocks = w.float().view(experts, n // 128, 128, k // 128, 128)
        scales = torch.exp2(torch.ceil(torch.log2(blocks.abs().amax(dim=(2, 4)).clamp_min(1e-10) / 448.0)))
        q = (blocks / scales[:, :, None, :, None]).view(experts, n, k).to(torch.float8_e4m3fn).contiguous()
        packed = pack_scales_mx(scales.view(experts * n // 128, k // 128).contiguous(), experts * n, k, weight=True)
        return q, scales, packed

    def dequantised_experts(self, layer: dict):
        """The bf16 weights the fp8 experts stand for (tests)."""
        out = []
        for name in ("w13", "w2"):
            q, scales = layer[name + "_q"], layer[name + "_scales"]
            full = scales.repeat_interleave(128, dim=1).repeat_interleave(128, dim=2)
            out.append((q.float() * full).to(torch.bfloat16))
        return out

    # -- one MoE layer --------------------------------------------------------------------
    def _moe_layer_fp8(self, x: torch.Tensor, layer: dict, ids: torch.Tensor, weights: torch.Tensor) -> torch.Tensor:
        c = self.config
        prepared = self.moe.prepare(x, weights, ids, quantized_input=True)
        slot = self.moe.runtime.selected[0]
        spec = slot.spec
        offsets, _ = expert_offsets(slot.expert_counts_by_source, align=128)
        permute(prepared.expert_input, self.x_perm, prepared.global_ids, prepared.expert_pos, offsets,
                prepared.recv_counts, world=spec.ranks, capacity=spec.capacity, src_scales=prepared.scales,
                dst_scales=self.x_scales)
        lo, hi = self.first_expert, self.first_expert + self.local_experts
        # Experts of other ranks hold no rows here, so the scan over all experts leaves the local groups packed.
        counts, offs = slot.expert_counts[lo:hi], offsets[0, lo:hi]
        live = spec.ranks * spec.capacity * min(c.top_k, self.local_experts)
        rows = min(self.x_perm.shape[0], (live + self.local_experts * 127 + 127) // 128 * 128)
        xp, h13 = self.x_perm[:rows], self.h13[:rows]
        grouped_gemm_e4m3_mx(xp, pack_scales_mx(self.x_scales[:rows], rows, c.hidden, weight=False),
                             layer["w13_q"], layer["w13_packed"], counts, offs, h13)
        act = (F.silu(h13[:, : c.ffn]) * h13[:, c.ffn:]).contiguous()
        act_q, act_s = quant_fp8(act, round_scale=True)
        grouped_gemm_e4m3_mx(act_q, pack_scales_mx(act_s, rows, c.ffn, weight=False), layer["w2_q"],
                             layer["w2_packed"], counts, offs, self.y_perm[:rows])
        out = torch.empty(x.shape[0], c.hidden, dtype=torch.bfloat16, device=x.device)
        self.moe.finalize(out, self.y_perm, expert_offsets=offsets)
        return out

    def moe_layer(self, x: torch.Tensor, layer: dict) -> torch.Tensor:
        c = self.config
        tokens = x.shape[0]
        logits = (x @ layer["router"].t()).float().contiguous()
        ids, weights = router_topk(logits, c.top_k, renormalize=True)
        if self.fp8_experts:
            return self._moe_layer_fp8(x, layer, ids, weights)
        prepared = self.moe.prepare(x, weights, ids)
        slot = self.moe.runtime.selected[0]
        spec = slot.spec
        # One offset per (source rank, expert); row 0 is where each expert's group starts.
        offsets, total = expert_offsets(slot.expert_counts_by_source)
        permute(prepared.expert_input, self.x_perm, prepared.global_ids, prepared.expert_pos, offsets,
                prepared.recv_counts, world=spec.ranks, capacity=spec.capacity)
        lo, hi = self.first_expert, self.first_expert + self.local_experts
        counts, offs = slot.expert_counts[lo:hi], offsets[0, lo:hi]
        # Rows that can be live under the selected variant's (rank-uniform) token bound.
        rows = min(self.x_perm.shape[0], spec.ranks * spec.capacity * min(c.top_k, self.local_experts))
        xp = self.x_perm[:rows]
        h13 = self.h13[:rows] if self.h13 is not None else torch.empty(
            rows, 2 * c.ffn, dtype=torch.bfloat16, device=x.device)
        grouped_gemm_bf16(xp, layer["w13"], counts, offs, h13)
        act = F.silu(h13[:, : c.ffn]) * h13[:, c.ffn:]
        grouped_gemm_bf16(act.contiguous(), layer["w2"], counts, offs, self.y_perm[:rows])
        out = torch.empty(tokens, c.hidden, dtype=torch.bfloat16, device=x.device)
        self.moe.finalize(out, self.y_perm, expert_offsets=offsets)
        return out

    # -- attention ---------------------------------------------------------------------------
    def attention(self, x: torch.Tensor, layer: dict, index: int, positions: torch.Tensor,
                  start: int) -> torch.Tensor:
        c = self.config
        b, s, _ = x.shape
        qkv = x @ layer["wqkv"].t()
        q, k, v = qkv.split([c.heads * c.head_dim, c.kv_heads * c.head_dim, c.kv_heads * c.head_dim], -1)
        q = _rope(q.view(b, s, c.heads, c.head_dim).transpose(1, 2), positions, c.rope_theta)
        k = _rope(k.view(b, s, c.kv_heads, c.head_dim).transpose(1, 2), positions, c.rope_theta)
        v = v.view(b, s, c.kv_heads, c.head_dim).transpose(1, 2)
        self.kv[index, 0, :b, :, start:start + s] = k
        self.kv[index, 1, :b, :, start:start + s] = v
        keys, values = self.kv[index, 0, :b, :, : start + s], self.kv[index, 1, :b, :, : start + s]
        if s == 1:
            # Decode: one query per head.  Batched matmuls over the cache slice; the library's fused
            # attention takes a slow generic path for a strided cache with grouped heads.
            group = c.heads // c.kv_heads
            qg = q.reshape(b, c.kv_heads, group, c.head_dim)
            scores = torch.matmul(qg, keys.transpose(-1, -2)).float() * (c.head_dim ** -0.5)
            out = torch.matmul(torch.softmax(scores, -1).to(values.dtype), values)
            out = out.reshape(b, 1, c.heads * c.head_dim)
            return out @ layer["wo"].t()
        out = F.scaled_dot_product_attention(q, keys, values, is_causal=(s > 1 and start == 0),
                                             enable_gqa=True)
        return out.transpose(1, 2).reshape(b, s, c.heads * c.head_dim) @ layer["wo"].t()

    def forward(self, token_ids: torch.Tensor, start: int = 0) -> torch.Tensor:
        """``token_ids`` int64 ``[B, S]`` at positions ``start .. start+S``; logits of the last position."""
        c = self.config
        b, s = token_ids.shape
        positions = torch.arange(start, start + s, device=self.device).expand(b, s)
        x = self.embed[token_ids]
        with self.moe.wave(b * s):  # one agreement on the shape variant per forward, not per layer
            for index, layer in enumerate(self.layers):
                x = x + self.attention(_rms_norm(x, layer["attn_norm"], c.rms_eps), layer, index,
                                       positions, start)
                h = _rms_norm(x, layer["ffn_norm"], c.rms_eps).reshape(b * s, c.hidden).contiguous()
                x = x + self.moe_layer(h, layer).view(b, s, c.hidden)
        x = _rms_norm(x[:, -1], self.final_norm, c.rms_eps)
        return (x @ self.lm_head.t()).float()

    # -- decode step as a CUDA graph ------------------------------------------------------------
    def _attention_static(self, x: torch.Tensor, layer: dict, index: int) -> torch.Tensor:
        """One-token attention whose position is a DEVICE scalar (``self._g_pos``): the new key and
        value are scattered into the cache with ``index_copy_`` and the scores run over the whole
        cache under a mask, so the launch sequence does not depend on the position."""
        c = self.config
        b = x.shape[0]
        positions = self._g_pos.expand(b, 1)
        qkv = x @ layer["wqkv"].t()
        q, k, v = qkv.split([c.heads * c.head_dim, c.kv_heads * c.head_dim, c.kv_heads * c.head_dim], -1)
        q = _rope(q.view(b, 1, c.heads, c.head_dim).transpose(1, 2), positions, c.rope_theta)
        k = _rope(k.view(b, 1, c.kv_heads, c.head_dim).transpose(1, 2), positions, c.rope_theta)
        v = v.view(b, 1, c.kv_heads, c.head_dim).transpose(1, 2)
        self.kv[index, 0, :b].index_copy_(2, self._g_pos, k)
        self.kv[index, 1, :b].index_copy_(2, self._g_pos, v)
        keys, values = self.kv[index, 0, :b], self.kv[index, 1, :b]          # [b, kv, max_seq, d]
        group = c.heads // c.kv_heads
        qg = q.reshape(b, c.kv_heads, group, c.head_dim)
        scores = torch.matmul(qg, keys.transpose(-1, -2)).float() * (c.head_dim ** -0.5)
        scores = scores.masked_fill(self._g_steps > self._g_pos, float("-inf"))
        out = torch.matmul(torch.softmax(scores, -1).to(values.dtype), values)
        return out.reshape(b, 1, c.heads * c.head_dim) @ layer["wo"].t()

    def _decode_static(self) -> torch.Tensor:
        c = self.config
        b = self._g_tokens.shape[0]
        x = self.embed[self._g_tokens]
        for index, layer in enumerate(self.layers):
            x = x + self._attention_static(_rms_norm(x, layer["attn_norm"], c.rms_eps), layer, index)
            h = _rms_norm(x, layer["ffn_norm"], c.rms_eps).reshape(b, c.hidden).contiguous()
            x = x + self.moe_layer(h, layer).view(b, 1, c.hidden)
        x = _rms_norm(x[:, -1], self.final_norm, c.rms_eps)
        return (x @ self.lm_head.t()).float()

    @torch.no_grad()
    def enable_decode_graph(self, batch: Optional[int] = None) -> None:
        """Capture one decode step (all layers: attention, router, fused dispatch, grouped expert
        GEMMs, fused combine) into a CUDA graph.  Every rank must call this at the same point: the
        warm-up and the capture run the MoE collectives.  Afterwards :meth:`decode` replays the graph;
        the token ids and the position travel through device tensors."""
        b = self.max_batch if batch is None else int(batch)
        self._g_tokens = torch.zeros(b, 1, dtype=torch.int64, device=self.device)
        self._g_pos = torch.zeros(1, dtype=torch.int64, device=self.device)
        self._g_steps = torch.arange(self.config.max_seq, device=self.device)
        self.moe.set_wave_bound(self.max_batch)  # decode: every rank has at most max_batch tokens
        side = torch.cuda.Stream(device=self.device)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(3):  # first-use initialisation of the launchers must not be captured
                self._decode_static()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        self._graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self._graph):
            self._g_logits = self._decode_static()
        self.moe.set_wave_bound(None)

    @torch.no_grad()
    def decode(self, token_ids: torch.Tensor, position: int) -> torch.Tensor:
        """One decode step for ``token_ids`` int64 ``[B, 1]`` at ``position``; logits ``[B, vocab]``."""
        if getattr(self, "_graph", None) is None or token_ids.shape != self._g_tokens.shape:
            return self.forward(token_ids, position)
        self._g_tokens.copy_(token_ids)
        self._g_pos.fill_(position)
        self._graph.replay()
        return self._g_logits

    @torch.no_grad()
    def generate(self, prompts: torch.Tensor, new_tokens: int) -> torch.Tensor:
        """Greedy decoding: prefill the prompts, then ``new_tokens`` single-token steps."""
        b, s = prompts.shape
        out = torch.empty(b, new_tokens, dtype=torch.int64, device=self.device)
        nxt = self.forward(prompts, 0).argmax(-1)
        for i in range(new_tokens):
            out[:, i] = nxt
            if i + 1 < new_tokens:
                nxt = self.decode(nxt[:, None], s + i).argmax(-1)
        return out

    def check(self) -> None:
        for slot in self.moe.runtime.family._slots.values():
            slot.check()

    def reference_moe_layer(self, x: torch.Tensor, layer: dict, all_w13, all_w2) -> torch.Tensor:
        """fp32 restatement of one MoE layer given every expert's weights (tests, tiny sizes)."""
        c = self.config
        probs = torch.softmax((x @ layer["router"].t()).float(), -1)
        w, ids = torch.topk(probs, c.top_k, -1)
        w = w / w.sum(-1, keepdim=True)
        out = torch.zeros_like(x, dtype=torch.float32)
        for e in range(c.experts):
            mask = (ids == e)
            rows = mask.any(-1)
            if not rows.any():
                continue
            h = x[rows].float() @ all_w13[e].float().t()
            act = (F.silu(h[:, : c.ffn]) * h[:, c.ffn:]).to(torch.bfloat16).float()
            y = (act @ all_w2[e].float().t()).to(torch.bfloat16).float()
            out[rows] += y * (w * mask)[rows].sum(-1, keepdim=True)
        return out
