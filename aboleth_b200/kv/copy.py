"""Page runs and the push launch (kernel: csrc/kernels/kv_kernels.cu)."""
from __future__ import annotations

import struct
from typing import Iterable, Sequence

import torch

from ..ops._kernels import _I, _U64, _VP, call, declare, ptr, stream_ptr

declare("ab_kv_push", [_VP, _VP, _I, _U64, _I, _I, _VP, _VP])
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


def push(batches: torch.Tensor, arrivals: torch.Tensor, count: int, epoch: int, *, workers: int,
         threads: int, status: torch.Tensor) -> None:
    call("ab_kv_push", ptr(batches), ptr(arrivals), count, epoch, workers, threads, ptr(status), stream_ptr())


def wait_ready(cells: torch.Tensor, epoch: int, status: torch.Tensor, *, timeout_ns: int = 2_000_000_000) -> None:
    """Enqueue a bounded device-side wait for every int64 readiness cell in ``cells``."""
    call("ab_kv_wait", ptr(cells), cells.numel(), epoch, timeout_ns, ptr(status), stream_ptr())


def cuda_memcpy_async(dst: int, src: int, nbytes: int, stream: int) -> None:
    """One copy-engine transfer between two device addresses (either may be a peer mapping)."""
    call("ab_memcpy_async", dst, src, nbytes, stream)
