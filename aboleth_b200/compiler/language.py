"""Tier-2 program builder: the semantic operations a kernel author states.

A program says *what* must travel and be published - ``put``, ``put_inline``,
``signal``, ``wait``, ``wait_signal``, ``drain``, groups - and never *how*: no
fences, no doorbells, no completion polling.  The specializer derives those.
The operation set and its contracts are the reference's Tier-2 builtins
(python/aboleth/language.py:117-566; docs/PROGRAMMING_MODEL.md:95-128); here a
program is built host-side as text IR (no Triton) and compiled to CUDA C++.

    b = ProgramBuilder("alltoall", args=[("send", "ptr"), ("recv_table", "table"), ...])
    peer = b.let("peer", "pid + (pid >= RANK)")
    e = b.endpoint("endpoints", peer)
    t = b.put(e, b.remote("recv_table", peer, offset="RANK*4096"),
              b.local(f"send + {peer}*4096"), bytes=4096)
    s = b.signal(e, b.remote("flag_table", peer, offset="RANK*8"), epoch=1, after=t)
    b.wait_signal(f"my_flags + {peer}*8", 1)
    b.wait(s)

Tokens, groups and endpoints are values of the program being built; they cannot
be passed to another builder.
"""
from __future__ import annotations

import contextlib
from dataclasses import dataclass
from typing import Iterable, Optional, Sequence, Union

Expr = Union[str, int]


def _e(value: Expr) -> str:
    """Render an expression operand: wrapped in parentheses when it has spaces."""
    text = str(value)
    if any(c.isspace() for c in text) or "=" in text and not text.startswith("("):
        return f"({text})"
    return text


@dataclass(frozen=True)
class Value:
    name: str
    kind: str
    owner: int

    def __str__(self) -> str:
        return self.name


class Token(Value):
    pass


class ProgramBuilder:
    def __init__(self, name: str, *, args: Sequence[tuple[str, str]] = (), threads: int = 32,
                 grid: Optional[int] = None):
        self.name = name
        self.args = list(args)
        self.threads = threads
        self.grid = grid
        self._lines: list[str] = []
        self._indent = 0
        self._counter = 0

    # -- plumbing ---------------------------------------------------------------------
    def _fresh(self, prefix: str) -> str:
        self._counter += 1
        return f"%{prefix}{self._counter}"

    def _emit(self, text: str) -> None:
        self._lines.append("  " * self._indent + text)

    def _own(self, value: Value) -> str:
        if not isinstance(value, Value) or value.owner != id(self):
            raise TypeError("tokens, groups, endpoints and regions cannot cross programs")
        return value.name

    def _define(self, prefix: str, kind: str, text: str, cls=Value) -> Value:
        name = self._fresh(prefix)
        self._emit(f"{name} = {text}")
        return cls(name, kind, id(self))

    @staticmethod
    def _attrs(**attrs) -> str:
        parts = []
        for key, value in attrs.items():
            if value is None or value is False:
                continue
            parts.append(key if value is True else f"{key}={_e(value)}")
        return (" " + " ".join(parts)) if parts else ""

    # -- bindings ---------------------------------------------------------------------
    def let(self, name: str, expr: Expr) -> str:
        """Name a scalar expression (visible to the issuer analysis)."""
        self._emit(f"let {name} {_e(expr)}")
        return name

    def endpoint(self, table: str, index: Expr) -> Value:
        return self._define("e", "endpoint", f"endpoint {table} {_e(index)}")

    def local(self, address: Expr, *, key: Expr = 0, at: Expr = None,
              valid: Optional[tuple[Expr, Expr, Expr]] = None) -> Value:
        """A local region.  ``valid=(count, capacity, item_bytes)`` declares a valid
        prefix followed by dead padding; ``at`` is the byte offset of this view."""
        v = None if valid is None else ",".join(str(x).replace(" ", "") for x in valid)
        return self._define("l", "local", f"local {_e(address)}" + self._attrs(key=key, at=at, valid=v))

    def remote(self, table: str, peer: Expr, *, offset: Expr = None) -> Value:
        """A peer's region from an (address, key) table (PeerRegionTable.regions)."""
        return self._define("r", "remote", f"remote {table} {_e(peer)}" + self._attrs(offset=offset))

    def remote_at(self, address: Expr, *, key: Expr = 0) -> Value:
        return self._define("r", "remote", f"remote_at {_e(address)}" + self._attrs(key=key))

    # -- semantic operations -------------------------------------------------------------
    def put(self, endpoint: Value, dst: Value, src: Value, *, bytes: Expr,
            after: Optional[Token] = None, predicate: Expr = None) -> Token:
        return self._define("t", "token",
                            f"put {self._own(endpoint)} {self._own(dst)} {self._own(src)}" +
                            self._attrs(bytes=bytes, after=after and self._own(after), pred=predicate),
                            Token)

    def put_inline(self, endpoint: Value, dst: Value, values: Iterable[tuple[Expr, int]], *,
                   after: Optional[Token] = None, predicate: Expr = None) -> Token:
        """``values`` = (expression, bits) pairs; bits in {8, 16, 24, 32, 64}, <= 972 bytes."""
        items = ",".join(f"{_e(v)}:{bits}" for v, bits in values)
        return self._define("t", "token",
                            f"put_inline {self._own(endpoint)} {self._own(dst)} values={items}" +
                            self._attrs(after=after and self._own(after), pred=predicate), Token)

    def signal(self, endpoint: Value, flag: Value, *, epoch: Expr, after: Optional[Token] = None,
               group: Optional[Value] = None, expected: Expr = None) -> Token:
        return self._define("s", "token",
                            f"signal {self._own(endpoint)} {self._own(flag)}" +
                            self._attrs(epoch=epoch, after=after and self._own(after),
                                        group=group and self._own(group), expected=expected), Token)

    def wait(self, token: Token, *, predicate: Expr = None, iteration: Expr = None,
             reuse: Optional[int] = None, final: Expr = None) -> None:
        """Sender-side completion.  With ``iteration``/``reuse`` the planner chooses how
        often to actually wait (``planned_wait``)."""
        if iteration is not None or reuse is not None:
            if iteration is None or reuse is None:
                raise ValueError("a planned wait needs both iteration= and reuse=")
            self._emit(f"planned_wait {self._own(token)}" +
                       self._attrs(iteration=iteration, reuse=reuse, final=final))
        else:
            self._emit(f"wait {self._own(token)}" + self._attrs(pred=predicate))

    planned_wait = wait

    def begin_group(self, endpoint: Value) -> Value:
        return self._define("g", "group", f"begin_group {self._own(endpoint)}")

    def wait_group(self, group: Value) -> None:
        self._emit(f"wait_group {self._own(group)}")

    def wait_signal(self, flag_address: Expr, epoch: Expr) -> None:
        self._emit(f"wait_signal {_e(flag_address)} {_e(epoch)}")

    def drain(self, endpoint: Value) -> None:
        self._emit(f"drain {self._own(endpoint)}")

    def system_fence(self) -> None:
        self._emit("system_fence")

    def invoke_phase(self, program_id: int, *arguments: Union[Expr, Value]) -> None:
        """Run the externally planned transport phase ``program_id`` here.  The fragment comes from
        the transport program given to ``compile_program(..., plan=...)``; values of this builder
        (an endpoint, say) and expressions may be passed for its parameters."""
        rendered = [str(self._own(a)) if isinstance(a, Value) else _e(a) for a in arguments]
        self._emit(" ".join(["invoke_phase", str(int(program_id)), *rendered]))

    # -- frontend code the analyses need to see --------------------------------------------
    def store(self, base: Expr, *, offset: int, width: int, value: Expr) -> None:
        """A scalar store at a constant offset (candidate for inline forwarding)."""
        self._emit(f"store {_e(base)}" + self._attrs(offset=offset, width=width, value=value))

    def tensor_store(self, name: str) -> None:
        """Mark a CTA-wide write of local memory (the code itself goes in ``stmt``)."""
        self._emit(f"tensor_store {name}")

    def stmt(self, code: str, *, unknown_write: bool = False) -> None:
        self._emit(f'stmt "{code}"' if not unknown_write else f'stmt "{code}"')
        if unknown_write:
            self._emit("tensor_store opaque")

    def barrier(self) -> None:
        self._emit("barrier")

    @contextlib.contextmanager
    def for_range(self, var: str, lo: Expr, hi: Expr):
        self._emit(f"for {var} {_e(lo)} {_e(hi)} {{")
        self._indent += 1
        try:
            yield var
        finally:
            self._indent -= 1
            self._emit("}")

    @contextlib.contextmanager
    def if_(self, condition: Expr):
        self._emit(f"if {_e(condition)} {{")
        self._indent += 1
        try:
            yield
        finally:
            self._indent -= 1
            self._emit("}")

    # -- result -----------------------------------------------------------------------------
    def text(self, *, backend: str = "p2p", rank: int = 0, world_size: int = 1) -> str:
        head = f"program {self.name} backend={backend} rank={rank} world={world_size} threads={self.threads}"
        if self.grid is not None:
            head += f" grid={self.grid}"
        lines = [head] + [f"arg {n} {t}" for n, t in self.args] + self._lines
        return "\n".join(lines) + "\n"
