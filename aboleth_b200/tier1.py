"""The Tier-1 operations as Tier-2 programs, one program per operation.

The hand-written header ``aboleth/device.cuh`` is what device code includes.  This module
states the same operations as programs of the specializer, so that the pass pipeline can
show - per transport - what each of them costs (reservations, doorbells, fences, flag
writes): ``tier1_facts("proxy")["put_many_8_signal"]`` is one reservation and one strong
signal, on ``p2p`` one CTA barrier-free chain closed by a single release store.  The
reference builds its Tier-1 library from per-op programs of this kind
(python/aboleth/tier1.py:164-675); here they document and test the header's contracts.
"""
from __future__ import annotations

from typing import Callable

from .compiler.driver import CompileError, compile_program
from .compiler.language import ProgramBuilder
from .compiler.options import compilation

_PUT_ARGS = [("endpoints", "table"), ("peer", "i32"), ("dst", "u64"), ("dst_key", "i32"), ("src", "u64"),
             ("src_key", "i32"), ("bytes", "i32")]
_FLAG_ARGS = [("flag", "u64"), ("flag_key", "i32"), ("value", "u64")]


def _put() -> ProgramBuilder:
    b = ProgramBuilder("tier1_put", args=_PUT_ARGS, threads=32)
    ep = b.endpoint("endpoints", "peer")
    b.wait(b.put(ep, b.remote_at("dst", key="dst_key"), b.local("src", key="src_key"), bytes="bytes"))
    return b


def _put_inline(bits: int) -> Callable[[], ProgramBuilder]:
    def build() -> ProgramBuilder:
        b = ProgramBuilder(f"tier1_put_inline{bits}", threads=32,
                           args=[("endpoints", "table"), ("peer", "i32"), ("dst", "u64"), ("dst_key", "i32"),
                                 ("value", "u64")])
        ep = b.endpoint("endpoints", "peer")
        b.wait(b.put_inline(ep, b.remote_at("dst", key="dst_key"), [("value", bits)]))
        return b
    return build


def _signal() -> ProgramBuilder:
    b = ProgramBuilder("tier1_signal", args=[("endpoints", "table"), ("peer", "i32")] + _FLAG_ARGS, threads=32)
    ep = b.endpoint("endpoints", "peer")
    b.wait(b.signal(ep, b.remote_at("flag", key="flag_key"), epoch="value"))
    return b


def _put_signal() -> ProgramBuilder:
    b = ProgramBuilder("tier1_put_signal", args=_PUT_ARGS + _FLAG_ARGS, threads=32)
    ep = b.endpoint("endpoints", "peer")
    data = b.put(ep, b.remote_at("dst", key="dst_key"), b.local("src", key="src_key"), bytes="bytes")
    b.wait(b.signal(ep, b.remote_at("flag", key="flag_key"), epoch="value", after=data))
    return b


def _put_many(count: int, closing: str) -> Callable[[], ProgramBuilder]:
    def build() -> ProgramBuilder:
        name = f"tier1_put_many_{count}" + (f"_{closing}" if closing else "")
        b = ProgramBuilder(name, args=_PUT_ARGS + [("stride", "i32")] + (_FLAG_ARGS if closing == "signal" else []),
                           threads=32)
        ep = b.endpoint("endpoints", "peer")
        previous = None
        for i in range(count):
            previous = b.put(ep, b.remote_at(f"dst + {i} * stride", key="dst_key"),
                             b.local(f"src + {i} * stride", key="src_key"), bytes="bytes", after=previous)
        if closing == "signal":
            b.wait(b.signal(ep, b.remote_at("flag", key="flag_key"), epoch="value", after=previous))
        elif closing == "flush":
            b.wait(previous)
            b.drain(ep)
        else:
            b.wait(previous)
        return b
    return build


def _quiet() -> ProgramBuilder:
    b = ProgramBuilder("tier1_quiet", args=[("endpoints", "table"), ("peer", "i32")], threads=32)
    b.drain(b.endpoint("endpoints", "peer"))
    return b


def _wait_signal() -> ProgramBuilder:
    b = ProgramBuilder("tier1_wait_signal", args=[("flag", "u64"), ("value", "u64")], threads=32)
    b.wait_signal("flag", "value")
    return b


PROGRAMS: dict[str, Callable[[], ProgramBuilder]] = {
    "put": _put, "put_inline8": _put_inline(8), "put_inline16": _put_inline(16), "put_inline24": _put_inline(24),
    "put_inline64": _put_inline(64), "signal": _signal, "put_signal": _put_signal,
    "put_many_8": _put_many(8, ""), "put_many_8_signal": _put_many(8, "signal"),
    "put_many_8_flush": _put_many(8, "flush"), "put_many_32": _put_many(32, ""),
    "put_many_32_signal": _put_many(32, "signal"), "put_many_32_flush": _put_many(32, "flush"),
    "quiet": _quiet, "wait_signal": _wait_signal,
}


def tier1_program(name: str) -> ProgramBuilder:
    try:
        return PROGRAMS[name]()
    except KeyError:
        raise KeyError(f"unknown Tier-1 operation {name!r}; known: {', '.join(sorted(PROGRAMS))}") from None


def tier1_facts(backend: str, **settings) -> dict[str, dict]:
    """Pipeline facts of every Tier-1 operation on ``backend``."""
    if backend != "p2p":
        settings.setdefault("queue_capacity", 64)
    facts: dict[str, dict] = {}
    with compilation(backend, **settings):
        for name, build in PROGRAMS.items():
            try:
                facts[name] = compile_program(build()).facts
            except CompileError as error:  # e.g. the ring carries only 64-bit inline values
                facts[name] = {"unsupported": str(error)}
    return facts
