"""Stock Tier-2 programs: the ones the benchmarks, goldens and docs use.

Each function returns a :class:`ProgramBuilder`.  They restate, in this
builder, the reference's example and benchmark kernels: the README all-to-all
(README.md:91-105, experiments/bench/tier2.py:128-171), the chain modes of the
stream benchmark (experiments/bench/stream.py:40-124) and the FP8 dispatch of
the paper's Listing 2 (experiments/python/aboleth_tier2_dispatch.py:46-83).
"""
from __future__ import annotations

from .language import ProgramBuilder

_A2A_ARGS = [("send", "ptr"), ("endpoints", "table"), ("recv_table", "table"),
             ("flag_table", "table"), ("my_flags", "ptr"), ("epoch", "u64")]


def alltoall(nbytes: int = 4096, *, threads: int = 32) -> ProgramBuilder:
    """One program per peer: put -> signal(epoch) -> wait_signal -> wait."""
    b = ProgramBuilder("alltoall", args=_A2A_ARGS, threads=threads)
    peer = b.let("peer", "pid + (pid >= RANK)")
    e = b.endpoint("endpoints", peer)
    t = b.put(e, b.remote("recv_table", peer, offset=f"RANK*{nbytes}"),
              b.local(f"send + {peer}*{nbytes}"), bytes=nbytes)
    s = b.signal(e, b.remote("flag_table", peer, offset="RANK*8"), epoch="epoch", after=t)
    b.wait_signal(f"my_flags + {peer}*8", "epoch")
    b.wait(s)
    return b


_STREAM_ARGS = [("payload", "ptr"), ("endpoints", "table"), ("remote_table", "table"),
                ("rounds", "i64")]


def stream(mode: str, chains: int, nbytes: int, *, reuse: int = 4, threads: int = 32) -> ProgramBuilder:
    """``chains`` puts of ``nbytes`` per round to one peer, in one of the stream modes.

    ``chains``    K independent put+signal chains, all waits at the round's end;
    ``serial``    wait after each chain;
    ``fused``     K puts chained by ``after`` and closed by ONE signal;
    ``pipelined`` like chains, with planned waits (``reuse``) and a final drain.
    Flags live right after the K payload slots on the peer.
    """
    if mode not in ("chains", "serial", "fused", "pipelined"):
        raise ValueError("mode must be chains, serial, fused or pipelined")
    b = ProgramBuilder(f"stream_{mode}", args=_STREAM_ARGS, threads=threads, grid=1)
    e = b.endpoint("endpoints", 1)
    with b.for_range("round", 0, "rounds"):
        tokens = []
        previous = None
        for k in range(chains):
            src = b.local(f"payload + {k * nbytes}")
            dst = b.remote("remote_table", 1, offset=k * nbytes)
            if mode == "fused":
                previous = b.put(e, dst, src, bytes=nbytes, after=previous)
                continue
            t = b.put(e, dst, src, bytes=nbytes)
            s = b.signal(e, b.remote("remote_table", 1, offset=chains * nbytes + 8 * k),
                         epoch="round + 1", after=t)
            if mode == "serial":
                b.wait(s)
            else:
                tokens.append(s)
        if mode == "fused":
            s = b.signal(e, b.remote("remote_table", 1, offset=chains * nbytes), epoch="round + 1",
                         after=previous)
            b.wait(s)
        for s in tokens:
            if mode == "pipelined":
                b.wait(s, iteration="round", reuse=reuse, final="round == rounds - 1")
            else:
                b.wait(s)
    if mode == "pipelined":
        b.drain(e)
    return b


def fp8_dispatch(chunks: int = 4, rows: int = 16, cols: int = 128, slots: int = 2) -> ProgramBuilder:
    """Per peer: ``chunks`` x (quantise a rows x cols bf16 tile into a send slot, put it),
    then an inline count, one signal, and a planned wait over ``slots`` reused buffers."""
    chunk_bytes = rows * cols + rows * 4
    b = ProgramBuilder("fp8_dispatch", threads=128, args=[
        ("tokens", "ptr"), ("staging", "ptr"), ("endpoints", "table"), ("slot_table", "table"),
        ("count_table", "table"), ("flag_table", "table"), ("live", "ptr"), ("iteration", "i64")])
    peer = b.let("peer", "pid")
    e = b.endpoint("endpoints", peer)
    previous = None
    for c in range(chunks):
        b.stmt(f"quantize_tile(tokens, staging, peer, {c});")
        b.tensor_store("staging")
        previous = b.put(e, b.remote("slot_table", peer, offset=f"(iteration % {slots})*{chunks * chunk_bytes} + {c * chunk_bytes}"),
                         b.local(f"staging + (peer*{chunks} + {c})*{chunk_bytes}"), bytes=chunk_bytes,
                         after=previous, predicate=f"((const int*)live)[peer*{chunks} + {c}]")
    count = b.put_inline(e, b.remote("count_table", peer, offset="RANK*8"),
                         [(f"((const int*)live)[peer*{chunks}]", 64)], after=previous)
    s = b.signal(e, b.remote("flag_table", peer, offset="RANK*8"), epoch="iteration + 1", after=count)
    b.wait(s, iteration="iteration", reuse=slots)
    return b


_LADDER_ARGS = [("payload", "ptr"), ("endpoints", "table"), ("remote_table", "table"), ("my_flag", "ptr"),
                ("rounds", "i64"), ("epoch0", "i64")]


def pingpong(nbytes: int, *, chain: int = 1, leader: bool = True, threads: int = 32) -> ProgramBuilder:
    """Latency ladder (reference: experiments/bench/tier2.py ``_pingpong``): per round the leader
    sends ``chain`` puts closed by ONE signal and waits for the echo; the follower waits first and
    echoes.  Payload at offset 0 of the peer's region, its flag right after the payload."""
    b = ProgramBuilder("pingpong_leader" if leader else "pingpong_follower", args=_LADDER_ARGS,
                       threads=threads, grid=1)
    e = b.endpoint("endpoints", 1)
    piece = max(nbytes // chain, 8)
    with b.for_range("round", 0, "rounds"):
        if not leader:
            b.wait_signal("my_flag", "epoch0 + round + 1")
        previous = None
        for c in range(chain):
            previous = b.put(e, b.remote("remote_table", 1, offset=c * piece), b.local(f"payload + {c * piece}"),
                             bytes=piece, after=previous)
        s = b.signal(e, b.remote("remote_table", 1, offset=chain * piece), epoch="epoch0 + round + 1",
                     after=previous)
        b.wait(s)
        if leader:
            b.wait_signal("my_flag", "epoch0 + round + 1")
    return b


def windowed(nbytes: int, *, window: int = 16, reuse: int = 4, threads: int = 32) -> ProgramBuilder:
    """Bandwidth ladder (``_windowed``): ``window`` independent puts per round and one completion
    for the round (planned over ``reuse`` buffers), a drain at the end.  One program per CTA; CTA
    ``pid`` owns the span ``pid * window * nbytes`` of both buffers."""
    b = ProgramBuilder("windowed", args=[("payload", "ptr"), ("endpoints", "table"), ("remote_table", "table"),
                                         ("rounds", "i64")], threads=threads)
    e = b.endpoint("endpoints", 1)
    span = window * nbytes
    with b.for_range("round", 0, "rounds"):
        previous = None
        for k in range(window):
            previous = b.put(e, b.remote("remote_table", 1, offset=f"pid*{span} + {k * nbytes}"),
                             b.local(f"payload + pid*{span} + {k * nbytes}"), bytes=nbytes, after=previous)
        b.wait(previous, iteration="round", reuse=reuse, final="round == rounds - 1")
    b.drain(e)
    return b
