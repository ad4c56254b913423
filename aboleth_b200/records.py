"""Semantic record transport as Tier-2 programs: a rank sends the valid prefix of a
per-peer record segment (payload rows, metadata rows, a count) and publishes one flag per
(peer, lane); the receiver waits for every lane's flag.

These are the reference's ``send_record_slice`` / ``send_records`` / ``await_records``
(python/aboleth/records.py:13-228) written with this package's program builder: grid
``(peers, lanes)``; lane ``l`` owns rows ``[Q*l + R*l//L, Q*(l+1) + R*(l+1)//L)`` of the
``capacity`` segment; sources are ``.valid(count, capacity, row_bytes)`` so dead padding
never travels; lane 0 alone sends the count; the wait is planned over ``reuse`` buffers.
The fused MoE kernels do the same work in one launch; these programs are the generic form
for clients that bring their own pack/unpack kernels.
"""
from __future__ import annotations

from .compiler.language import ProgramBuilder


def send_records(*, rank: int, peer_extent: int, capacity: int, width_bytes: int, meta_width_words: int,
                 lanes: int, row_quotient: int, row_remainder: int, reuse: int, ready_stride: int,
                 threads: int = 256) -> ProgramBuilder:
    """One program per (peer, lane): ``grid = peers * lanes`` with ``pid = lane * peers + p``."""
    b = ProgramBuilder("send_records", threads=threads, args=[
        ("endpoints", "table"), ("peers", "table"), ("payload", "ptr"), ("metadata", "ptr"),
        ("destination_data", "table"), ("destination_meta", "table"), ("destination_counts", "table"),
        ("destination_flags", "table"), ("counts", "ptr"), ("epoch_pointer", "ptr"), ("npeers", "i64")])
    b.let("slot", "pid % npeers")
    b.let("lane", "pid / npeers")
    b.let("peer", "(long long)peers[slot]")
    b.let("count", "((const long long*)counts)[peer]")
    b.let("epoch", "*(const long long*)epoch_pointer")
    b.let("begin", f"{row_quotient}*lane + {row_remainder}*lane/{lanes}")
    b.let("end", f"{row_quotient}*(lane+1) + {row_remainder}*(lane+1)/{lanes}")
    e = b.endpoint("endpoints", f"lane*{peer_extent} + peer")
    src = b.local(f"payload + peer*{capacity * width_bytes}", at=f"begin*{width_bytes}",
                  valid=("count", capacity, width_bytes))
    header = b.put(e, b.remote("destination_data", "peer", offset=f"({rank * capacity} + begin)*{width_bytes}"),
                   src, bytes=f"(end - begin)*{width_bytes}")
    if meta_width_words > 0:
        meta_bytes = meta_width_words * 4
        meta = b.local(f"metadata + peer*{capacity * meta_bytes}", at=f"begin*{meta_bytes}",
                       valid=("count", capacity, meta_bytes))
        header = b.put(e, b.remote("destination_meta", "peer", offset=f"({rank * capacity} + begin)*{meta_bytes}"),
                       meta, bytes=f"(end - begin)*{meta_bytes}", after=header)
    count = b.put_inline(e, b.remote("destination_counts", "peer", offset=rank * 8), [("count", 64)],
                         after=header, predicate="lane == 0")
    published = b.signal(e, b.remote("destination_flags", "peer", offset=f"({rank * ready_stride} + lane)*8"),
                         epoch="epoch", after=count)
    b.wait(published, iteration="epoch", reuse=reuse)
    return b


def await_records(*, ready_stride: int, lanes_per_program: int, threads: int = 32) -> ProgramBuilder:
    """One program per (peer, lane group): wait until every lane of the group published ``epoch``."""
    b = ProgramBuilder("await_records", threads=threads, args=[
        ("flags", "ptr"), ("peers", "table"), ("epoch_pointer", "ptr"), ("npeers", "i64")])
    b.let("slot", "pid % npeers")
    b.let("group", "pid / npeers")
    b.let("peer", "(long long)peers[slot]")
    b.let("epoch", "*(const long long*)epoch_pointer")
    for lane in range(lanes_per_program):
        b.wait_signal(f"flags + (peer*{ready_stride} + group*{lanes_per_program} + {lane})*8", "epoch")
    return b
