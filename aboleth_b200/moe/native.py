"""Executor of the fused expert-parallel dispatch and combine.

``NativeMoESlot`` owns one set of buffers (one in-flight layer) on one rank:
the peer-visible receive/return segments and flags, registered with the World
and exchanged once, plus the local routing state.  ``dispatch`` and ``combine``
are one kernel launch each (csrc/kernels/moe_kernels.cu); the epoch lives in
device memory and is advanced by the combine kernel, so the pair can be
captured in a CUDA graph.  API shape follows the reference's executor
(python/aboleth/moe/native.py:34-178,433-615).

The SENDER unpacks: besides the payload row and the wire-format metadata row it
writes each record's expert ids, gate weights and positions into the
destination's ``recv_ids`` / ``recv_weights`` / ``recv_pos`` arrays, so the
receiving rank runs no per-record pass.  A position counts the record among
ITS SOURCE RANK's records for that expert; each source also sends its
per-expert totals (``recv_expert_counts[source, expert]``), and
``expert_offsets`` turns that table into the first row of every (source,
expert) group in the expert-contiguous layout.  The
combine publishes returned records in blocks of ``return_block`` rows
(``return_flags[peer, block]``) and reduces a token as soon as the blocks that
hold its partial rows are there.

``LocalMoEGroup`` runs several ranks on ONE device inside one process by
launching every rank's send half before any rank's receive half; it exists for
tests and single-GPU development, not for performance.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import Optional, Sequence

import torch

from ..ops._kernels import call, ptr, stream_ptr
from ..world import World
from .spec import MoESpec

PHASE_SEND, PHASE_RECV = 1, 2
_REGIONS = ("recv_payload", "recv_meta", "recv_counts", "dispatch_flags", "returned", "return_flags",
            "recv_ids", "recv_weights", "recv_pos", "recv_expert_counts")
RETURN_BLOCK = 64          # records per readiness block of the combine (every rank must use the same)
MIN_RETURN_BLOCK = 16      # the flag arrays are sized for blocks this small
MAX_DISPATCH_CTAS = 2048   # rows of the per-CTA record-count table (token-ordered slots)


def return_blocks(spec: MoESpec, block: int = MIN_RETURN_BLOCK) -> int:
    return (spec.capacity + block - 1) // block


def _region_sizes(spec: MoESpec) -> dict[str, int]:
    s, rows = spec, spec.ranks * spec.capacity
    return {
        "recv_payload": rows * s.row_bytes,
        "recv_meta": rows * s.metadata_words * 4,
        "recv_counts": s.ranks * 8,
        "dispatch_flags": s.ranks * 8,
        "returned": rows * s.hidden * 2,
        # [ranks, blocks + 1] int64: one flag per block of returned records, then "finished sending"
        "return_flags": s.ranks * (return_blocks(s) + 1) * 8,
        "recv_ids": rows * s.top_k * 4,
        "recv_weights": rows * s.top_k * 4,
        "recv_pos": rows * s.top_k * 4,
        "recv_expert_counts": s.ranks * s.experts * 4,
    }


def _align(n: int, a: int = 256) -> int:
    return (n + a - 1) // a * a


@dataclass(frozen=True)
class LaunchBinding:
    """What the compiled plan of a shape variant decides about the executor's launches
    (the reference binds grids, lanes, row slices, REUSE and the ready stride the same way:
    python/aboleth/moe/native.py:193-289; in-place inputs :451-477; forwarded output :594-597).

    The fused kernels are token-parallel rather than (peer, lane) programs, so a lane plan maps to
    them as follows.  A dispatch that the planner fans out over every lane of its endpoint profile
    is bandwidth-bound: one warp per token, token-ordered slots.  One that needs fewer lanes is
    latency-bound: one CTA per token.  The combine gives ``sender_warps - 1`` warps of each CTA to
    sending (the rest reduce) and publishes returned records in blocks of half a lane's row slice.
    """

    by_warp: bool
    dispatch_lanes: int
    return_lanes: int
    send_warps: int
    return_block: int
    received_rows: int
    borrow_tokens: bool          # the storage plan proved a prefix binding: read the caller's tensor in place
    forward_expert_output: bool  # the expert stage writes the return source itself: no copy before the combine
    profile: str

    @classmethod
    def from_plan(cls, spec: MoESpec, plan) -> "LaunchBinding":
        dispatch, back = plan.dispatch_launches[0], plan.return_launches[0]
        profile = dispatch.profile_identity
        max_lanes = dict(plan.profile_max_lanes).get(dispatch.backend, dispatch.lanes)
        rows_per_lane = max(1, spec.capacity // max(back.lanes, 1))
        block = max(64, min(128, rows_per_lane // 2))
        return cls(by_warp=dispatch.lanes >= max_lanes and dispatch.lanes > 1,
                   dispatch_lanes=dispatch.lanes, return_lanes=back.lanes,
                   send_warps=max(1, min(7, back.sender_warps - 1)),
                   return_block=1 << (block.bit_length() - 1),
                   received_rows=int(plan.storage["received_payload"]["physical_rows"]),
                   borrow_tokens=bool(plan.storage.get("tokens", {}).get("prefix_binding", False)),
                   forward_expert_output=bool(plan.forwarded_expert_output), profile=profile)


@dataclass
class DispatchResult:
    """What the expert stage consumes.  Rows are ``[ranks * capacity]``; rows of
    source rank ``r`` start at ``r * capacity`` and ``recv_counts[r]`` are live."""

    expert_input: torch.Tensor      # [ranks*capacity, hidden] e4m3 or bf16
    expert_scales: Optional[torch.Tensor]  # [ranks*capacity, hidden/group] fp32
    expert_ids: torch.Tensor        # [ranks*capacity, k] int32
    expert_weights: torch.Tensor    # [ranks*capacity, k] fp32
    expert_pos: torch.Tensor        # [ranks*capacity, k] int32 position inside its (source, expert) group, -1 unused
    expert_counts: torch.Tensor     # [experts] int32 totals
    expert_counts_by_source: torch.Tensor  # [ranks, experts] int32: what ``expert_offsets`` consumes
    recv_counts: torch.Tensor       # [ranks] int64
    topk_ids: torch.Tensor          # [capacity, k] int32 (this rank's tokens)
    topk_weights: torch.Tensor      # [capacity, k] fp32


def _last_grid(which: int) -> int:
    """CTAs of the last dispatch (0) or combine (1) launch of this thread."""
    from ..ops._kernels import lib
    fn = lib().ab_ep_last_grid
    fn.restype, fn.argtypes = ctypes.c_int, [ctypes.c_int]
    return int(fn(which))


class MoEBuffers:
    """Carves one rank's arena.  ``arena`` must be zero-initialised."""

    def __init__(self, spec: MoESpec, arena: torch.Tensor):
        sizes = _region_sizes(spec)
        self.offsets, cursor = {}, 0
        for name in _REGIONS:
            self.offsets[name] = (cursor, sizes[name])
            cursor += _align(sizes[name])
        self.nbytes = cursor
        if arena.numel() < cursor:
            raise ValueError(f"arena holds {arena.numel()} bytes, {cursor} are needed")
        self.arena = arena

    @staticmethod
    def arena_bytes(spec: MoESpec) -> int:
        return sum(_align(x) for x in _region_sizes(spec).values())

    def view(self, name: str) -> torch.Tensor:
        start, size = self.offsets[name]
        return self.arena[start:start + size]


class NativeMoESlot:
    def __init__(self, spec: MoESpec, rank: int, arena: torch.Tensor,
                 peer_tables: dict[str, torch.Tensor], *, placement="linear", grid: Optional[int] = None,
                 plan=None):
        self.spec, self.rank = spec, int(rank)
        dev = arena.device
        self.device = dev
        self.buffers = MoEBuffers(spec, arena)
        s, rows = spec, spec.ranks * spec.capacity
        b = self.buffers
        self.recv_payload = b.view("recv_payload").view(spec.payload_dtype).view(rows, s.hidden)
        self.recv_meta = b.view("recv_meta").view(torch.int32).view(rows, s.metadata_words)
        self.recv_counts = b.view("recv_counts").view(torch.int64)
        self.dispatch_flags = b.view("dispatch_flags").view(torch.int64)
        self.returned = b.view("returned").view(torch.bfloat16).view(rows, s.hidden)
        self.return_block = RETURN_BLOCK
        self.return_flags = b.view("return_flags").view(torch.int64)   # [ranks, blocks + 1] at run time
        self.peer_tables = peer_tables  # name -> int64 [ranks] addresses
        owners = placement if isinstance(placement, (list, tuple)) else spec.owners(placement)
        self.owners_list = list(owners)
        self.owners = torch.tensor(self.owners_list, dtype=torch.int32, device=dev)
        # Unused choice slots of a record name an expert its destination does not own, at weight 0.
        foreign = [next((e for e, o in enumerate(self.owners_list) if o != d), -1)
                   for d in range(s.ranks)]
        self.placeholder = foreign[self.rank]
        self.placeholders = torch.tensor(foreign, dtype=torch.int32, device=dev)
        z = lambda *shape, dtype: torch.zeros(*shape, dtype=dtype, device=dev)  # noqa: E731
        self.source_slots = torch.full((s.capacity, s.ranks), -1, dtype=torch.int32, device=dev)
        self.send_counts = z(s.ranks, dtype=torch.int64)
        self.done = z(8 + 32, dtype=torch.int32)   # arrival counters, then one record cursor per destination
        self.block_counts = z(MAX_DISPATCH_CTAS, s.ranks, dtype=torch.int32)
        self.block_done = z(s.ranks, return_blocks(s), dtype=torch.int32)
        self.overflow = z(1, dtype=torch.int32)
        self.epoch = torch.ones(1, dtype=torch.int64, device=dev)
        self.status = z(2, dtype=torch.int64)
        # Written by the SENDING ranks (peer-visible); the expert stage reads them as they are.
        self.expert_ids = b.view("recv_ids").view(torch.int32).view(rows, s.top_k)
        self.expert_weights = b.view("recv_weights").view(torch.float32).view(rows, s.top_k)
        self.expert_pos = b.view("recv_pos").view(torch.int32).view(rows, s.top_k)
        self.expert_counts_by_source = b.view("recv_expert_counts").view(torch.int32).view(s.ranks, s.experts)
        self.send_expert_counts = z(s.experts, dtype=torch.int32)
        self.expert_counts = z(s.experts, dtype=torch.int32)
        # The scales travel inside the metadata row; this is a strided view of them (row stride =
        # metadata_words), not a copy.
        self.expert_scales = (self.recv_meta.view(torch.float32)[:, 2 + 2 * s.top_k:]
                              if s.fp8 else None)
        self.topk_ids = z(s.capacity, s.top_k, dtype=torch.int32)
        self.topk_weights = z(s.capacity, s.top_k, dtype=torch.float32)
        self.expert_output = z(rows, s.hidden, dtype=torch.bfloat16)
        self.final_output = z(s.capacity, s.hidden, dtype=torch.bfloat16)
        # 0 lets the launcher size the grid from the token count.  `by_warp`
        # selects one warp per token / row (throughput) over one CTA per token
        # (latency); None decides per call from the token count.
        self.grid = int(grid) if grid else 0
        self.by_warp: Optional[bool] = None
        self.by_warp_threshold = 512
        # Optional device trace: %globaltimer stamps (ns) of kernel phases, see trace().
        self.trace_buffer: Optional[torch.Tensor] = None
        # Warps per CTA that send in a fused warp-per-row combine; the others reduce.
        self.send_warps = 6
        self._ints = (ctypes.c_int * 24)()
        self._ptrs = (ctypes.c_uint64 * 32)()
        self._table = None
        self.launched: dict[str, dict] = {}   # what the last dispatch / combine actually launched
        self.binding: Optional[LaunchBinding] = None
        self._token_staging: Optional[torch.Tensor] = None
        self._return_source: Optional[torch.Tensor] = None
        if plan is not None:
            self.bind_plan(plan)

    def bind_plan(self, plan) -> LaunchBinding:
        """Take the launch geometry and the buffer decisions from a compiled plan of this shape."""
        binding = LaunchBinding.from_plan(self.spec, plan)
        rows = self.spec.ranks * self.spec.capacity
        if binding.received_rows != rows:
            raise ValueError(f"the plan keeps {binding.received_rows} received rows, the slot was built for {rows}")
        self.binding = binding
        self.by_warp = binding.by_warp
        self.send_warps, self.return_block = binding.send_warps, binding.return_block
        return binding

    # -- construction over a World ------------------------------------------------
    @classmethod
    def create(cls, world: World, spec: MoESpec, *, tag: str = "moe", **kwargs) -> "NativeMoESlot":
        """Allocate, register and exchange one slot's buffers over ``world``."""
        if spec.ranks != world.world_size:
            raise ValueError("spec.ranks must equal the world size")
        arena = world.runtime.allocate(MoEBuffers.arena_bytes(spec))
        registration = world.register(arena, network=False)
        layout = MoEBuffers(spec, arena)
        regions = [world.region(name, registration, offset=layout.offsets[name][0],
                                length=layout.offsets[name][1]) for name in _REGIONS]
        table = world.exchange_regions(regions, tag=tag)
        slot = cls(spec, world.rank, arena, {name: table.addresses(name) for name in _REGIONS},
                   **kwargs)
        slot._table = table
        return slot

    # -- launches ---------------------------------------------------------------------
    def _geometry(self, num_tokens: int, routing: int, renormalize: bool, phases: int,
                  weighted: int = 0):
        s, i = self.spec, self._ints
        if self.return_block < MIN_RETURN_BLOCK:
            raise ValueError(f"return_block must be at least {MIN_RETURN_BLOCK}")
        by_warp = (num_tokens > self.by_warp_threshold) if self.by_warp is None else self.by_warp
        values = [self.rank, s.ranks, s.experts, s.top_k, s.hidden, s.scale_group, s.capacity,
                  int(s.fp8), int(s.round_scale), 0, num_tokens, routing,
                  int(renormalize), phases, weighted, int(by_warp), self.return_block,
                  self.send_warps, self.block_counts.shape[0]]
        self.last_launch = {"by_warp": bool(by_warp), "requested_grid": self.grid, "phases": phases,
                            "send_warps": self.send_warps, "return_block": self.return_block}
        for k, v in enumerate(values):
            i[k] = v
        return i

    def _fill(self, pointers: Sequence) -> ctypes.Array:
        for k, p in enumerate(pointers):
            self._ptrs[k] = p if isinstance(p, int) else ptr(p)
        return self._ptrs

    def dispatch(self, tokens: torch.Tensor, ids: Optional[torch.Tensor] = None,
                 weights: Optional[torch.Tensor] = None, *, logits: Optional[torch.Tensor] = None,
                 num_tokens: Optional[int] = None, renormalize: bool = False,
                 phases: int = PHASE_SEND | PHASE_RECV) -> DispatchResult:
        """Route, quantise and send this rank's tokens; receive and unpack the peers'.

        Give either ``logits`` (fp32 ``[n, experts]``: the router softmax and
        top-k run inside the kernel) or ``ids`` (int32 ``[n, k]``, -1 = unused)
        with ``weights`` (fp32 ``[n, k]``).
        """
        s = self.spec
        n = tokens.shape[0] if num_tokens is None else int(num_tokens)
        if n > s.capacity:
            raise ValueError(f"{n} tokens exceed the slot capacity {s.capacity}")
        if tokens.dtype != torch.bfloat16 or tokens.shape[-1] != s.hidden or not tokens.is_contiguous():
            raise ValueError("tokens must be contiguous bf16 [n, hidden]")
        if self.binding is not None and not self.binding.borrow_tokens:
            # No prefix binding was proven for the token region: the kernel may not read the caller's
            # tensor while the caller is free to overwrite it, so it gets a private copy.
            if self._token_staging is None:
                self._token_staging = torch.empty(s.capacity, s.hidden, dtype=torch.bfloat16, device=self.device)
            self._token_staging[:n].copy_(tokens[:n])
            tokens = self._token_staging
        routing = 1 if logits is not None else 0
        if routing:
            if logits.dtype != torch.float32 or logits.shape[-1] != s.experts:
                raise ValueError("logits must be fp32 [n, experts]")
        elif ids is None or weights is None or ids.dtype != torch.int32 or weights.dtype != torch.float32:
            raise ValueError("ids (int32) and weights (fp32) are required without logits")
        t = self.peer_tables
        pointers = [tokens, logits, ids, weights, self.topk_ids, self.topk_weights, self.owners,
                    self.placeholders, self.source_slots, self.send_counts, self.done, self.overflow,
                    self.epoch, self.status, self.block_counts, t["recv_payload"], t["recv_meta"],
                    t["recv_counts"], t["dispatch_flags"], t["recv_ids"], t["recv_weights"],
                    t["recv_pos"], t["recv_expert_counts"], self.send_expert_counts, self.recv_counts,
                    self.dispatch_flags, self.expert_counts_by_source, self.expert_counts,
                    self.trace_buffer]
        call("ab_ep_dispatch", self._geometry(n, routing, renormalize, phases),
             ctypes.c_float(s.quant_amax_floor), self._fill(pointers), self.grid, stream_ptr())
        self.launched["dispatch"] = {**self.last_launch, "tokens": n, "grid": _last_grid(0)}
        self._last_tokens = n
        return DispatchResult(self.recv_payload, self.expert_scales, self.expert_ids,
                              self.expert_weights, self.expert_pos, self.expert_counts,
                              self.expert_counts_by_source, self.recv_counts, self.topk_ids,
                              self.topk_weights)

    def combine(self, expert_output: Optional[torch.Tensor] = None, *,
                expert_offsets: Optional[torch.Tensor] = None, num_tokens: Optional[int] = None,
                out: Optional[torch.Tensor] = None,
                phases: int = PHASE_SEND | PHASE_RECV) -> torch.Tensor:
        """Return expert results to their source ranks and reduce them per token.

        Without ``expert_offsets`` the rows of ``expert_output`` are one partial
        per received record (``[ranks*capacity, hidden]``, already gate-weighted)
        and are summed over ranks.  With ``expert_offsets`` (int32 ``[ranks, experts]``
        from :func:`aboleth_b200.ops.expert_offsets` over ``expert_counts_by_source``)
        ``expert_output`` is in expert-contiguous order and the gate-weighted
        sum over each record's experts is taken inside the kernel.
        """
        s = self.spec
        n = getattr(self, "_last_tokens", s.capacity) if num_tokens is None else int(num_tokens)
        y = self.expert_output if expert_output is None else expert_output
        if y.dtype != torch.bfloat16 or y.shape[-1] != s.hidden or not y.is_contiguous():
            raise ValueError("expert_output must be contiguous bf16 [rows, hidden]")
        out = self.final_output if out is None else out
        if self.binding is not None and not self.binding.forward_expert_output:
            # The plan could not forward the expert stage's destination into the return source:
            # the residual copy the reference calls ``residual_expert_copy``.
            if self._return_source is None or self._return_source.shape != y.shape:
                self._return_source = torch.empty_like(y)
            self._return_source.copy_(y)
            y = self._return_source
        if expert_offsets is not None and tuple(expert_offsets.shape) != (s.ranks, s.experts):
            raise ValueError("expert_offsets must be int32 [ranks, experts] (one row per source rank)")
        t = self.peer_tables
        pointers = [y, self.expert_ids, self.expert_pos, self.expert_weights, expert_offsets,
                    self.recv_meta, self.recv_counts, t["returned"], t["return_flags"],
                    self.return_flags, self.returned, self.source_slots, out, self.done,
                    self.block_done, self.epoch, self.status, self.trace_buffer]
        call("ab_ep_combine", self._geometry(n, 0, False, phases, int(expert_offsets is not None)),
             ctypes.c_float(s.quant_amax_floor), self._fill(pointers), self.grid, stream_ptr())
        self.launched["combine"] = {**self.last_launch, "tokens": n, "grid": _last_grid(1),
                                    "weighted": expert_offsets is not None}
        return out[:n]

    def enable_trace(self) -> None:
        """Record phase stamps of the next kernels (CTA 0 and the publishing CTA)."""
        self.trace_buffer = torch.zeros(8, dtype=torch.int64, device=self.device)

    def trace(self) -> dict:
        """Phase stamps (us after CTA 0 started) of the last traced kernel.

        Dispatch: ``first_cta_sent``, ``all_sent`` (the last CTA arrived and publishes),
        ``peers_seen`` (every peer's flag observed), ``end``.  Combine: ``first_cta_sent``,
        ``first_cta_reduced``, ``all_reduced`` (last CTA arrived), ``end`` (every peer said it
        finished sending)."""
        t = self.trace_buffer.tolist()
        us = lambda b: (t[b] - t[0]) / 1e3 if t[0] and t[b] else None  # noqa: E731
        return {"first_cta_sent": us(1), "all_sent_or_first_reduced": us(2), "peers_seen_or_all_reduced": us(3),
                "end": us(4)}

    def reset(self) -> None:
        """Clear per-layer counters (only needed when a dispatch is not followed by a combine)."""
        self.expert_counts.zero_()
        self.send_expert_counts.zero_()
        self.send_counts.zero_()
        self.done.zero_()
        self.block_done.zero_()

    def check(self) -> None:
        """Raise if a kernel recorded a timeout / malformed record, or a segment overflowed."""
        status = self.status.tolist()
        if status[0]:
            names = {1: "timeout", 2: "completion failure", 3: "malformed record"}
            raise RuntimeError(f"MoE transport {names.get(status[0], status[0])} "
                               f"(detail {status[1]:#x}) on rank {self.rank}")
        if int(self.overflow.item()):
            raise RuntimeError(f"a destination segment overflowed on rank {self.rank}")

    def manifest(self) -> dict:
        s = self.spec
        return {"rank": self.rank, "ranks": s.ranks, "capacity": s.capacity, "hidden": s.hidden,
                "top_k": s.top_k, "experts": s.experts, "value_type": s.value_type,
                "metadata_words": s.metadata_words, "arena_bytes": self.buffers.nbytes,
                "launches_per_layer": 2, "requested_grid": self.grid, "return_block": self.return_block,
                "send_warps": self.send_warps,
                "plan_binding": None if self.binding is None else vars(self.binding),
                "launched": self.launched}


class LocalMoEGroup:
    """``ranks`` slots on one device in one process (tests, single-GPU development)."""

    def __init__(self, spec: MoESpec, device="cuda:0", **kwargs):
        device = torch.device(device)
        self.spec = spec
        arenas = [torch.zeros(MoEBuffers.arena_bytes(spec), dtype=torch.uint8, device=device)
                  for _ in range(spec.ranks)]
        layouts = [MoEBuffers(spec, a) for a in arenas]
        tables = {name: torch.tensor([l.view(name).data_ptr() for l in layouts], dtype=torch.int64,
                                     device=device) for name in _REGIONS}
        self.slots = [NativeMoESlot(spec, r, arenas[r], tables, **kwargs) for r in range(spec.ranks)]

    def dispatch(self, tokens: Sequence[torch.Tensor], **per_rank) -> list[DispatchResult]:
        kw = lambda r: {k: (v[r] if v is not None else None) for k, v in per_rank.items()}  # noqa: E731
        for r, slot in enumerate(self.slots):
            slot.dispatch(tokens[r], phases=PHASE_SEND, **kw(r))
        return [slot.dispatch(tokens[r], phases=PHASE_RECV, **kw(r))
                for r, slot in enumerate(self.slots)]

    def combine(self, expert_outputs: Sequence[Optional[torch.Tensor]], *,
                expert_offsets: Optional[Sequence[torch.Tensor]] = None) -> list[torch.Tensor]:
        off = lambda r: None if expert_offsets is None else expert_offsets[r]  # noqa: E731
        for r, slot in enumerate(self.slots):
            slot.combine(expert_outputs[r], expert_offsets=off(r), phases=PHASE_SEND)
        return [slot.combine(expert_outputs[r], expert_offsets=off(r), phases=PHASE_RECV)
                for r, slot in enumerate(self.slots)]

    def check(self) -> None:
        for slot in self.slots:
            slot.check()
