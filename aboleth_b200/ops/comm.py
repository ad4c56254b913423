"""All-to-all, ping-pong and Tier-1 exercise launchers (kernels: csrc/kernels/comm_kernels.cu)."""
from __future__ import annotations

from typing import Optional

import torch

from ._kernels import call, ptr, stream_ptr


def alltoall(send: torch.Tensor, peer_recv: torch.Tensor, peer_flags: torch.Tensor,
             my_flags: torch.Tensor, status: torch.Tensor, *, stride: int, nbytes: int,
             epoch0: int, rank: int, world: int, lanes: int = 8, chain: int = 1,
             batched: bool = True, rounds: int = 1, include_self: bool = False,
             wait: bool = True, mode: str = "vector", threads: int = 512) -> None:
    """One or more all-to-all rounds.

    ``send`` holds ``world`` slices of ``stride`` bytes; slice ``p`` goes to rank
    ``p``'s receive buffer at offset ``rank * stride``.  ``peer_recv`` /
    ``peer_flags`` are int64 ``[world]`` address tables (PeerRegionTable.addresses).
    Flags are int64 ``[world * lanes]``; round ``r`` publishes ``epoch0 + 1 + r``.
    ``chain`` splits each lane's slice into that many puts; ``batched`` closes
    them with one signal, otherwise each put is signalled.  ``mode`` is
    ``"vector"`` (ld/st by the CTA) or ``"bulk"`` (bulk-async copies through
    shared memory, 16-byte granularity).  ``wait=False`` sends without
    waiting for the peers (used to emulate several ranks on one device).
    """
    call("ab_alltoall", ptr(send), ptr(peer_recv), ptr(peer_flags), ptr(my_flags), ptr(status),
         stride, nbytes, epoch0, rank, world, lanes, chain, int(batched), rounds,
         int(include_self), int(wait), {"vector": 0, "bulk": 1}[mode], threads, stream_ptr())


def fill_payload(buf: torch.Tensor, nbytes: int, seed: int, sender: int, receiver: int) -> None:
    call("ab_fill_payload", ptr(buf), nbytes, seed, sender, receiver, stream_ptr())


def check_payload(buf: torch.Tensor, nbytes: int, seed: int, sender: int, receiver: int,
                  errors: torch.Tensor) -> None:
    """Add the number of wrong 8-byte words to ``errors`` (uint64/int64 scalar tensor)."""
    call("ab_check_payload", ptr(buf), nbytes, seed, sender, receiver, ptr(errors), stream_ptr())


def pingpong(src: torch.Tensor, peer_dst: int, peer_flag: int, my_flag: torch.Tensor,
             status: torch.Tensor, samples: Optional[torch.Tensor], *, nbytes: int, epoch0: int,
             leader: bool, chain: int = 1, rounds: int = 1, batched: bool = True,
             threads: int = 256) -> None:
    call("ab_pingpong", ptr(src), peer_dst, peer_flag, ptr(my_flag), ptr(status), ptr(samples),
         nbytes, epoch0, int(leader), chain, rounds, int(batched), threads, stream_ptr())


def tier1_exercise(endpoints: torch.Tensor, status: torch.Tensor, *, dst: int, src: int, flag: int,
                   inline_dst: int, wait_flag: int = 0, epoch: int = 1, wait_epoch: int = 0,
                   timeout_ns: int = 200_000_000, nbytes: int = 0, peer: int = 0,
                   pieces: int = 1) -> None:
    """One thread drives put_inline, put_signal / put_many_signal, quiet and a bounded wait."""
    call("ab_tier1_exercise", ptr(endpoints), ptr(status), dst, src, flag, inline_dst, wait_flag,
         epoch, wait_epoch, timeout_ns, nbytes, peer, pieces, stream_ptr())
