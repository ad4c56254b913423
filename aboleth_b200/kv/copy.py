"""Page runs and the push launch (kernel: csrc/kernels/kv_kernels.cu)."""
from __future__ import annotations

import struct
from typing import Iterable, Sequence

import torch

from ..ops._kernels import _I, _U64, _VP, call, declare, ptr, stream_ptr

declare("ab_kv_push", [_VP, _VP, _VP, _VP, _I, _U64, _I, _I, _VP, _VP])
declare("ab_kv_push_observed", [_VP, _VP, _VP, _VP, _I, _U64, _I, _I, _VP, _VP, _U64, _VP, _VP])
declare("ab_kv_wait", [_VP, _I, _U64, _U64, _VP, _VP])
declare("ab_memcpy_async", [_VP, _VP, _U64, _VP])


def canonicalize_block_runs(src_blocks: Sequence[int], dst_blocks: Sequence[int]) -> list[tuple[int, int, int]]:
    """Merge (src, dst) block pairs into maximal runs ``(src_start, dst_start, length)`` where
    both sides are consecutive (reference: python/aboleth/kv/copy.py ``canonicalize_block_runs``)."""
    if len(src_blocks) != len(dst_blocks):
        raise ValueError("source and destination block lists differ in length")
    runs: list[tuple[int, int, int]] = []
    for s, d in zip(src_blocks, dst_blocks):
        if runs and runs[-1][0] + runs[-1][2] == s and runs[-1][1] + runs[-1][2] == d:
            runs[-1] = (runs[-1][0], runs[-1][1], runs[-1][2] + 1)
        else:
            runs.append((int(s), int(d), 1))
    return runs


def pack_batches(batches: Iterable[tuple[int, int, int, int]], device) -> torch.Tensor:
    """``(src address, dst address, bytes, readiness cell address)`` records as a device tensor."""
    blob = b"".join(struct.pack("<QQQQ", *b) for b in batches)
    return torch.frombuffer(bytearray(blob), dtype=torch.uint8).to(device)


def pack_groups(cells: Sequence[int], workers: int, device) -> tuple[torch.Tensor, torch.Tensor, int]:
    """Group the batches of one launch by the readiness cell they publish.

    Returns ``(group_of int32 [batches], group_target int32 [groups], groups)``: batches that name
    the same cell share one arrival counter whose target is their worker total, so the cell is
    published by the last worker of the whole group and never while a sibling batch still copies
    (reference: python/aboleth/frontends/triton/kv_cache.py:225-290 counts finished batches per
    consumer for the same reason)."""
    index: dict[int, int] = {}
    group_of = [index.setdefault(int(c), len(index)) for c in cells]
    sizes = [0] * len(index)
    for g in group_of:
        sizes[g] += 1
    both = torch.tensor(group_of + [n * workers for n in sizes], dtype=torch.int32).to(device)
    return both[: len(group_of)], both[len(group_of):], len(index)


def push(batches: torch.Tensor, arrivals: torch.Tensor, count: int, epoch: int, *, workers: int,
         threads: int, status: torch.Tensor, group_of: torch.Tensor | None = None,
         group_target: torch.Tensor | None = None) -> None:
    """Launch the push.  Without ``group_of`` every batch must publish a cell of its own."""
    call("ab_kv_push", ptr(batches), ptr(arrivals), ptr(group_of), ptr(group_target), count, epoch,
         workers, threads, ptr(status), stream_ptr())


def push_observed(batches: torch.Tensor, arrivals: torch.Tensor, count: int, epoch: int, *, workers: int,
                  threads: int, status: torch.Tensor, cell: torch.Tensor, observed: torch.Tensor,
                  group_of: torch.Tensor | None = None, group_target: torch.Tensor | None = None,
                  timeout_ns: int = 1_000_000_000) -> None:
    """Self-check form of :func:`push`: one consumer CTA of the same launch waits for ``cell`` and
    sums the destinations' 8-byte words into ``observed[0]`` the moment the epoch shows."""
    call("ab_kv_push_observed", ptr(batches), ptr(arrivals), ptr(group_of), ptr(group_target), count,
         epoch, workers, threads, ptr(cell), ptr(observed), timeout_ns, ptr(status), stream_ptr())


def wait_ready(cells: torch.Tensor, epoch: int, status: torch.Tensor, *, timeout_ns: int = 2_000_000_000) -> None:
    """Enqueue a bounded device-side wait for every int64 readiness cell in ``cells``."""
    call("ab_kv_wait", ptr(cells), cells.numel(), epoch, timeout_ns, ptr(status), stream_ptr())


def cuda_memcpy_async(dst: int, src: int, nbytes: int, stream: int) -> None:
    """One copy-engine transfer between two device addresses (either may be a peer mapping)."""
    call("ab_memcpy_async", dst, src, nbytes, stream)
