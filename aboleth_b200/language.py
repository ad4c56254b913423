"""Free-function form of the Tier-2 semantic operations.

The reference exposes ``put``, ``signal``, ``wait`` ... as functions callable inside a kernel
body (python/aboleth/language.py:204-566).  Here a kernel body is a
:class:`~aboleth_b200.compiler.language.ProgramBuilder`; the functions below apply to the
builder opened by ``building(...)`` so that client code reads the same way::

    with building("ring", args=[("endpoints", "ptr"), ("buf", "u64")]) as program:
        ep = endpoint("endpoints", 0)
        data = put(ep, remote_at("buf"), local("buf"), bytes=4096)
        ready = signal(ep, remote_at("buf + 4096"), epoch="it + 1", after=data)
        wait(ready)
    compiled = compile_program(program)
"""
from __future__ import annotations

import contextlib
import threading
from typing import Iterator, Optional

from .compiler.language import ProgramBuilder, Token, Value
from .transport_binding import invoke_transport_program  # noqa: F401  (re-exported)

token = Token


class token_type:  # noqa: N801  (name kept from the reference)
    """Type tag of a completion token: what ``put`` / ``signal`` return and ``after=`` / ``wait`` accept."""

    name = "token"

    def __eq__(self, other) -> bool:
        return isinstance(other, token_type)

    def __hash__(self) -> int:
        return hash("aboleth.token")

    @staticmethod
    def of(value) -> bool:
        return isinstance(value, Token)


_state = threading.local()


def current_builder() -> ProgramBuilder:
    builder = getattr(_state, "builder", None)
    if builder is None:
        raise RuntimeError("semantic operations need an open program: use `with building(...)`")
    return builder


@contextlib.contextmanager
def building(name: str, **kwargs) -> Iterator[ProgramBuilder]:
    previous = getattr(_state, "builder", None)
    _state.builder = ProgramBuilder(name, **kwargs)
    try:
        yield _state.builder
    finally:
        _state.builder = previous


def endpoint(table: str, index) -> Value:
    return current_builder().endpoint(table, index)


def local(address, **kwargs) -> Value:
    return current_builder().local(address, **kwargs)


def remote(table: str, peer, **kwargs) -> Value:
    return current_builder().remote(table, peer, **kwargs)


def remote_at(address, **kwargs) -> Value:
    return current_builder().remote_at(address, **kwargs)


def put(endpoint_value: Value, destination: Value, source: Value, byte_count=None, *, bytes=None,
        after: Optional[Token] = None, predicate=None) -> Token:
    size = bytes if bytes is not None else byte_count
    if size is None:
        raise TypeError("put() needs a byte count")
    return current_builder().put(endpoint_value, destination, source, bytes=size, after=after,
                                 predicate=predicate)


def put_inline(endpoint_value: Value, destination: Value, values, **kwargs) -> Token:
    return current_builder().put_inline(endpoint_value, destination, values, **kwargs)


def signal(endpoint_value: Value, flag: Value, value=None, *, epoch=None, after: Optional[Token] = None,
           group: Optional[Value] = None, expected=None) -> Token:
    payload = epoch if epoch is not None else value
    if payload is None:
        raise TypeError("signal() needs the value to publish")
    return current_builder().signal(endpoint_value, flag, epoch=payload, after=after, group=group,
                                    expected=expected)


def wait(transfer: Token, predicate=None, iteration=None, reuse=None) -> None:
    current_builder().wait(transfer, predicate=predicate, iteration=iteration, reuse=reuse)


def planned_wait(transfer: Token, iteration, reuse: int, final=None) -> None:
    """Completion whose frequency the planner chooses: at most every ``reuse`` iterations."""
    current_builder().wait(transfer, iteration=iteration, reuse=reuse, final=final)


def begin_group(endpoint_value: Value) -> Value:
    return current_builder().begin_group(endpoint_value)


def wait_group(group: Value) -> None:
    current_builder().wait_group(group)


def system_fence() -> None:
    current_builder().system_fence()


def invoke_phase(program_id: int, *arguments) -> None:
    """Splice point of an externally planned transport phase (see ``ProgramBuilder.invoke_phase``)."""
    current_builder().invoke_phase(program_id, *arguments)


def drain(endpoint_value: Value) -> None:
    current_builder().drain(endpoint_value)


def wait_signal(signal_pointer, expected) -> None:
    current_builder().wait_signal(signal_pointer, expected)
