"""Tensor parallelism: GEMMs fused with their collective over NVLink peer memory.

``AllGatherGemm``       ``C[world*Ml, Nl] = all_gather(A_local) @ B_local.T`` in one launch
``GemmReduceScatter``   ``out[Ml, N] = reduce_scatter(A_local @ B_local.T)`` in one launch

Kernels: csrc/kernels/tp_kernels.cu (tcgen05 / TMEM main loop, TMA from local memory
only, peer stores and release flags for the collective half).  Each object owns two
sets of peer-visible buffers and alternates between them, so a rank may run one call
ahead of its slowest peer; any collective between two calls keeps ranks that close.

``LocalTpGroup`` runs several ranks on ONE device by launching every rank's producing
half before any rank's consuming half (tests, single-GPU development).
"""
from __future__ import annotations

import ctypes
from typing import Optional, Sequence

import torch

from ..ops._kernels import _I, _U64, _VP, call, declare, lib, ptr, stream_ptr
from ..world import World

declare("ab_ag_gemm_bf16", [_VP] * 9 + [_U64] + [_I] * 7 + [_U64, _VP])
declare("ab_gemm_rs_bf16", [_VP] * 9 + [_U64] + [_I] * 6 + [_VP])
declare("ab_ag_gemm_e4m3_mx", [_VP] * 11 + [_U64] + [_I] * 7 + [_U64, _VP])
declare("ab_gemm_rs_e4m3_mx", [_VP] * 11 + [_U64] + [_I] * 6 + [_VP])

PRODUCE, CONSUME = 1, 2
BM = 256  # rows per tile / chunk of the fused kernels


def _align(n: int, a: int = 256) -> int:
    return (n + a - 1) // a * a


class _Buffers:
    """Two alternating (data, flags) sets carved from one arena."""

    def __init__(self, arena: torch.Tensor, data_bytes: int, flag_count: int):
        self.data_bytes, self.flag_count = data_bytes, flag_count
        stride = _align(data_bytes) + _align(flag_count * 8)
        self.offsets = [(i * stride, i * stride + _align(data_bytes)) for i in range(2)]
        self.arena = arena

    @staticmethod
    def nbytes(data_bytes: int, flag_count: int) -> int:
        return 2 * (_align(data_bytes) + _align(flag_count * 8))

    def data(self, i: int) -> torch.Tensor:
        start = self.offsets[i][0]
        return self.arena[start:start + self.data_bytes]

    def flags(self, i: int) -> torch.Tensor:
        start = self.offsets[i][1]
        return self.arena[start:start + self.flag_count * 8].view(torch.int64)


def _exchange(world: World, buffers: _Buffers, tag: str):
    registration = world.register(buffers.arena, network=False)
    regions = []
    for i in range(2):
        regions.append(world.region(f"data{i}", registration, offset=buffers.offsets[i][0],
                                    length=buffers.data_bytes))
        regions.append(world.region(f"flags{i}", registration, offset=buffers.offsets[i][1],
                                    length=buffers.flag_count * 8))
    table = world.exchange_regions(regions, tag=tag)
    return [(table.addresses(f"data{i}"), table.addresses(f"flags{i}")) for i in range(2)], table


class AllGatherGemm:
    """Column-parallel linear layer whose input is sharded by rows across ranks."""

    def __init__(self, rank: int, world_size: int, m_local: int, k: int, buffers: _Buffers,
                 tables, *, push_parts: int = 0, multicast: Optional[Sequence[int]] = None):
        if m_local % BM:
            raise ValueError("rows per rank must be a multiple of 256")
        self.rank, self.world_size, self.m_local, self.k = rank, world_size, m_local, k
        self.buffers, self.tables, self.push_parts = buffers, tables, push_parts  # 0: items of ~64 KiB
        # Multicast address of each of the two staging buffers (0: push with one store per peer).
        self.multicast = tuple(multicast) if multicast is not None else (0, 0)
        self.status = torch.zeros(2, dtype=torch.int64, device=buffers.arena.device)
        # Sender-side arrival counters of the push, one per (peer, chunk); the kernel resets them.
        self.arrivals = torch.zeros(world_size * (m_local // BM), dtype=torch.int32,
                                    device=buffers.arena.device)
        self.epoch = 0

    @staticmethod
    def arena_bytes(world_size: int, m_local: int, k: int) -> int:
        return _Buffers.nbytes(world_size * m_local * k * 2, world_size * (m_local // BM))

    @classmethod
    def create_multicast(cls, world: World, m_local: int, k: int, *, group=None, **kw) -> "AllGatherGemm":
        """Like :meth:`create`, with the staging buffers in symmetric memory bound to an NVLink
        multicast object (:class:`aboleth_b200.symmetric.SymmetricArena`): the shard is pushed with
        ``multimem.st`` and leaves this GPU once instead of ``world - 1`` times.  Needs an
        initialised ``torch.distributed`` group over the same ranks; falls back to peer stores
        through the symmetric mappings when the fabric offers no multicast."""
        from ..symmetric import SymmetricArena
        n = world.world_size
        arena = SymmetricArena(cls.arena_bytes(n, m_local, k), world.torch_device, group)
        if arena.rank != world.rank or arena.world_size != n:
            raise ValueError("the process group and the world disagree on rank or size")
        buffers = _Buffers(arena.tensor, n * m_local * k * 2, n * (m_local // BM))
        tables = [(arena.addresses(buffers.offsets[i][0]), arena.addresses(buffers.offsets[i][1])) for i in range(2)]
        obj = cls(world.rank, n, m_local, k, buffers, tables,
                  multicast=[arena.multicast(buffers.offsets[i][0]) for i in range(2)], **kw)
        obj._arena = arena
        return obj

    @classmethod
    def create(cls, world: World, m_local: int, k: int, *, tag: str = "ag_gemm", **kw) -> "AllGatherGemm":
        n = world.world_size
        arena = world.runtime.allocate(cls.arena_bytes(n, m_local, k))
        buffers = _Buffers(arena, n * m_local * k * 2, n * (m_local // BM))
        tables, table = _exchange(world, buffers, tag)
        obj = cls(world.rank, n, m_local, k, buffers, tables, **kw)
        obj._table = table
        return obj

    def __call__(self, a_local: torch.Tensor, b_local: torch.Tensor, out: Optional[torch.Tensor] = None,
                 *, phases: int = PRODUCE | CONSUME, advance: bool = True) -> torch.Tensor:
        """``a_local`` bf16 ``[m_local, k]``, ``b_local`` bf16 ``[n_local, k]`` ->
        bf16 ``[world*m_local, n_local]`` (rows of rank r at ``r*m_local``)."""
        assert a_local.dtype == b_local.dtype == torch.bfloat16
        assert a_local.shape == (self.m_local, self.k) and b_local.shape[1] == self.k
        assert a_local.is_contiguous() and b_local.is_contiguous()
        n = b_local.shape[0]
        if out is None:
            out = torch.empty(self.world_size * self.m_local, n, dtype=torch.bfloat16,
                              device=a_local.device)
        if advance and (phases & PRODUCE):
            self.epoch += 1
        which = self.epoch & 1
        peer_data, peer_flags = self.tables[which]
        call("ab_ag_gemm_bf16", ptr(a_local), ptr(self.buffers.data(which)), ptr(b_local), ptr(out),
             ptr(peer_data), ptr(peer_flags), ptr(self.buffers.flags(which)), ptr(self.status),
             ptr(self.arrivals), (self.epoch + 1) // 2, self.rank, self.world_size, self.m_local, n,
             self.k, self.push_parts, phases, self.multicast[which], stream_ptr())
        return out

    def mx(self, a_q: torch.Tensor, a_packed: torch.Tensor, b_q: torch.Tensor, b_packed: torch.Tensor,
           out: Optional[torch.Tensor] = None, *, phases: int = PRODUCE | CONSUME,
           advance: bool = True) -> torch.Tensor:
        """The fused kernel on block-scaled e4m3 operands: ``a_q`` ``[m_local, k]`` and ``b_q``
        ``[n_local, k]`` with scale factors packed by :func:`aboleth_b200.ops.pack_scales_mx`.  The
        shard crosses NVLink as e4m3 (half the bytes of the bf16 form) with its scale-factor atoms
        and the product runs on ``tcgen05.mma.kind::mxf8f6f4.block_scale``; bf16 output."""
        from ..ops.gemm import _mx_scale_bytes
        fp8 = torch.float8_e4m3fn
        assert a_q.dtype == b_q.dtype == fp8 and a_q.is_contiguous() and b_q.is_contiguous()
        assert a_q.shape == (self.m_local, self.k) and b_q.shape[1] == self.k and self.k % 128 == 0
        n = b_q.shape[0]
        assert a_packed.numel() == _mx_scale_bytes(self.m_local, n, self.k, 0)
        assert b_packed.numel() == _mx_scale_bytes(self.m_local, n, self.k, 1)
        rows = self.world_size * self.m_local
        assert rows * self.k + rows // 128 * (self.k // 128) * 512 <= self.buffers.data_bytes
        if out is None:
            out = torch.empty(rows, n, dtype=torch.bfloat16, device=a_q.device)
        if advance and (phases & PRODUCE):
            self.epoch += 1
        which = self.epoch & 1
        peer_data, peer_flags = self.tables[which]
        call("ab_ag_gemm_e4m3_mx", ptr(a_q), ptr(a_packed), ptr(self.buffers.data(which)), ptr(b_q),
             ptr(b_packed), ptr(out), ptr(peer_data), ptr(peer_flags), ptr(self.buffers.flags(which)),
             ptr(self.status), ptr(self.arrivals), (self.epoch + 1) // 2, self.rank, self.world_size,
             self.m_local, n, self.k, self.push_parts, phases, self.multicast[which], stream_ptr())
        return out

    def block_scaled(self, a_q: torch.Tensor, a_scales: torch.Tensor, b_local: torch.Tensor,
                     out: Optional[torch.Tensor] = None, *, b_scales: Optional[torch.Tensor] = None,
                     b_packed: Optional[torch.Tensor] = None, **kw) -> torch.Tensor:
        """Block-scaled e4m3 activations (``a_q`` with 1 x 128 fp32 ``a_scales``).

        With an e4m3 ``b_local`` and its 128 x 128 ``b_scales`` (or their packed form ``b_packed``) and
        power-of-two scales everywhere, both operands stay e4m3 end to end (:meth:`mx`).  With a bf16
        ``b_local`` this rank's shard is expanded to bf16 by
        :func:`aboleth_b200.ops.dequant_block_scaled` and then gathered and multiplied as in
        :meth:`__call__` (any positive scales)."""
        from ..ops.gemm import dequant_block_scaled, pack_scales_mx
        if b_local.dtype == torch.float8_e4m3fn:
            if b_packed is None:
                b_packed = pack_scales_mx(b_scales, b_local.shape[0], self.k, weight=True)
            a_packed = pack_scales_mx(a_scales, self.m_local, self.k, weight=False)
            return self.mx(a_q, a_packed, b_local, b_packed, out, **kw)
        return self(dequant_block_scaled(a_q, a_scales), b_local, out, **kw)

    def check(self) -> None:
        status = self.status.tolist()
        if status[0]:
            raise RuntimeError(f"all-gather GEMM wait gave up (status {status[0]}, detail {status[1]:#x})")


class GemmReduceScatter:
    """Row-parallel linear layer whose output is reduced and scattered by rows."""

    def __init__(self, rank: int, world_size: int, m_local: int, n: int, buffers: _Buffers, tables):
        if m_local % BM or n % 8:
            raise ValueError("rows per rank must be a multiple of 256 and n a multiple of 8")
        self.rank, self.world_size, self.m_local, self.n = rank, world_size, m_local, n
        self.buffers, self.tables = buffers, tables
        self.status = torch.zeros(2, dtype=torch.int64, device=buffers.arena.device)
        # One 256x256 bf16 staging tile per CTA: the epilogue parks a tile here (it stays in L2) and
        # pushes it to its owner while the next tile's main loop runs.
        with torch.cuda.device(buffers.arena.device):
            query = lib().ab_gemm_rs_stage_bytes
            query.restype, query.argtypes = ctypes.c_longlong, []
            stage_bytes = int(query())
        self.stage = torch.empty(stage_bytes, dtype=torch.uint8, device=buffers.arena.device)
        self.epoch = 0

    @staticmethod
    def _tiles(m_local: int, n: int) -> int:
        # one flag per tile and source; the block-scaled kernel's tiles are 192 columns wide, the
        # bf16 kernel's 256: sized for the narrower
        return (m_local // BM) * ((n + 191) // 192)

    @staticmethod
    def arena_bytes(world_size: int, m_local: int, n: int) -> int:
        return _Buffers.nbytes(world_size * m_local * n * 2,
                               world_size * GemmReduceScatter._tiles(m_local, n))

    @classmethod
    def create(cls, world: World, m_local: int, n: int, *, tag: str = "gemm_rs") -> "GemmReduceScatter":
        w = world.world_size
        arena = world.runtime.allocate(cls.arena_bytes(w, m_local, n))
        buffers = _Buffers(arena, w * m_local * n * 2, w * cls._tiles(m_local, n))
        tables, table = _exchange(world, buffers, tag)
        obj = cls(world.rank, w, m_local, n, buffers, tables)
        obj._table = table
        return obj

    def __call__(self, a: torch.Tensor, b_local: torch.Tensor, out: Optional[torch.Tensor] = None, *,
                 phases: int = PRODUCE | CONSUME, advance: bool = True) -> torch.Tensor:
        """``a`` bf16 ``[world*m_local, k_local]``, ``b_local`` bf16 ``[n, k_local]`` ->
        bf16 ``[m_local, n]``: this rank's rows of the sum over ranks."""
        assert a.dtype == b_local.dtype == torch.bfloat16 and a.is_contiguous() and b_local.is_contiguous()
        assert a.shape[0] == self.world_size * self.m_local and b_local.shape == (self.n, a.shape[1])
        if out is None:
            out = torch.empty(self.m_local, self.n, dtype=torch.bfloat16, device=a.device)
        if advance and (phases & PRODUCE):
            self.epoch += 1
        which = self.epoch & 1
        peer_data, peer_flags = self.tables[which]
        call("ab_gemm_rs_bf16", ptr(a), ptr(b_local), ptr(self.buffers.data(which)), ptr(out),
             ptr(self.stage), ptr(peer_data), ptr(peer_flags), ptr(self.buffers.flags(which)), ptr(self.status),
             (self.epoch + 1) // 2, self.rank, self.world_size, self.m_local, self.n, a.shape[1],
             phases, stream_ptr())
        return out

    def mx(self, a_q: torch.Tensor, a_packed: torch.Tensor, b_q: torch.Tensor, b_packed: torch.Tensor,
           out: Optional[torch.Tensor] = None, *, phases: int = PRODUCE | CONSUME,
           advance: bool = True) -> torch.Tensor:
        """The fused kernel on block-scaled e4m3 operands (scale factors packed by
        :func:`aboleth_b200.ops.pack_scales_mx`): the partial products come off
        ``tcgen05.mma.kind::mxf8f6f4.block_scale`` and are exchanged and reduced as in the bf16 form."""
        from ..ops.gemm import _mx_scale_bytes
        fp8 = torch.float8_e4m3fn
        assert a_q.dtype == b_q.dtype == fp8 and a_q.is_contiguous() and b_q.is_contiguous()
        rows, k = a_q.shape
        assert rows == self.world_size * self.m_local and b_q.shape == (self.n, k) and k % 128 == 0
        assert a_packed.numel() == _mx_scale_bytes(rows, self.n, k, 0)
        assert b_packed.numel() == _mx_scale_bytes(rows, self.n, k, 1)
        if out is None:
            out = torch.empty(self.m_local, self.n, dtype=torch.bfloat16, device=a_q.device)
        if advance and (phases & PRODUCE):
            self.epoch += 1
        which = self.epoch & 1
        peer_data, peer_flags = self.tables[which]
        call("ab_gemm_rs_e4m3_mx", ptr(a_q), ptr(a_packed), ptr(b_q), ptr(b_packed),
             ptr(self.buffers.data(which)), ptr(out), ptr(self.stage), ptr(peer_data), ptr(peer_flags),
             ptr(self.buffers.flags(which)), ptr(self.status), (self.epoch + 1) // 2, self.rank,
             self.world_size, self.m_local, self.n, k, phases, stream_ptr())
        return out

    def block_scaled(self, a_q: torch.Tensor, a_scales: torch.Tensor, b_local: torch.Tensor,
                     out: Optional[torch.Tensor] = None, *, b_scales: Optional[torch.Tensor] = None,
                     b_packed: Optional[torch.Tensor] = None, **kw) -> torch.Tensor:
        """As :meth:`__call__` for block-scaled e4m3 activations (1 x 128 fp32 scales).  An e4m3
        ``b_local`` with 128 x 128 ``b_scales`` (or ``b_packed``) and power-of-two scales keeps both
        operands e4m3 (:meth:`mx`); a bf16 ``b_local`` takes the expansion of ``a_q`` to bf16."""
        from ..ops.gemm import dequant_block_scaled, pack_scales_mx
        if b_local.dtype == torch.float8_e4m3fn:
            k = a_q.shape[1]
            if b_packed is None:
                b_packed = pack_scales_mx(b_scales, self.n, k, weight=True)
            a_packed = pack_scales_mx(a_scales, a_q.shape[0], k, weight=False)
            return self.mx(a_q, a_packed, b_local, b_packed, out, **kw)
        return self(dequant_block_scaled(a_q, a_scales), b_local, out, **kw)

    def check(self) -> None:
        status = self.status.tolist()
        if status[0]:
            raise RuntimeError(f"GEMM reduce-scatter wait gave up (status {status[0]}, detail {status[1]:#x})")


class LocalTpGroup:
    """Emulates ``world_size`` tensor-parallel ranks on one device in one process."""

    def __init__(self, world_size: int, m_local: int, k_or_n_ag: int, n_rs: int, device="cuda:0"):
        device = torch.device(device)
        self.world_size = world_size

        def build(kind, data_bytes, flag_count, make):
            arenas = [torch.zeros(_Buffers.nbytes(data_bytes, flag_count), dtype=torch.uint8, device=device)
                      for _ in range(world_size)]
            bufs = [_Buffers(a, data_bytes, flag_count) for a in arenas]
            tables = [(torch.tensor([b.data(i).data_ptr() for b in bufs], dtype=torch.int64, device=device),
                       torch.tensor([b.flags(i).data_ptr() for b in bufs], dtype=torch.int64, device=device))
                      for i in range(2)]
            return [make(r, bufs[r], tables) for r in range(world_size)]

        k = k_or_n_ag
        self.ag = build("ag", world_size * m_local * k * 2, world_size * (m_local // BM),
                        lambda r, b, t: AllGatherGemm(r, world_size, m_local, k, b, t))
        self.rs = build("rs", world_size * m_local * n_rs * 2,
                        world_size * GemmReduceScatter._tiles(m_local, n_rs),
                        lambda r, b, t: GemmReduceScatter(r, world_size, m_local, n_rs, b, t))

    def ag_gemm(self, a_shards: Sequence[torch.Tensor], b_shards: Sequence[torch.Tensor]) -> list[torch.Tensor]:
        outs = [None] * self.world_size
        for r, op in enumerate(self.ag):
            outs[r] = op(a_shards[r], b_shards[r], phases=PRODUCE)
        return [op(a_shards[r], b_shards[r], outs[r], phases=CONSUME, advance=False)
                for r, op in enumerate(self.ag)]

    def ag_gemm_mx(self, a_q, a_packed, b_q, b_packed) -> list[torch.Tensor]:
        """:meth:`ag_gemm` on block-scaled e4m3 shards (lists per rank, scales already packed)."""
        outs = [op.mx(a_q[r], a_packed[r], b_q[r], b_packed[r], phases=PRODUCE) for r, op in enumerate(self.ag)]
        return [op.mx(a_q[r], a_packed[r], b_q[r], b_packed[r], outs[r], phases=CONSUME, advance=False)
                for r, op in enumerate(self.ag)]

    def gemm_rs_mx(self, a_q, a_packed, b_q, b_packed) -> list[torch.Tensor]:
        """:meth:`gemm_rs` on block-scaled e4m3 operands (lists per rank, scales already packed)."""
        outs = [op.mx(a_q[r], a_packed[r], b_q[r], b_packed[r], phases=PRODUCE) for r, op in enumerate(self.rs)]
        return [op.mx(a_q[r], a_packed[r], b_q[r], b_packed[r], outs[r], phases=CONSUME, advance=False)
                for r, op in enumerate(self.rs)]

    def gemm_rs(self, a_parts: Sequence[torch.Tensor], b_shards: Sequence[torch.Tensor]) -> list[torch.Tensor]:
        outs = [None] * self.world_size
        for r, op in enumerate(self.rs):
            outs[r] = op(a_parts[r], b_shards[r], phases=PRODUCE)
        return [op(a_parts[r], b_shards[r], outs[r], phases=CONSUME, advance=False)
                for r, op in enumerate(self.rs)]
