"""Binding a planned communication attachment to the slots of a client kernel.

A *transport program* is the communication of one attachment (one or more logical
transfers that share a publication) written against named scalar slots: the endpoint, and
for every region pair a remote pointer/key, a local pointer/key, a byte count and a
predicate; for the publication a remote and a local flag address with their keys and the
iteration counters.  The client kernel supplies values for the slots at its insertion
point.  ``TransportProgramBinding.to_builder()`` turns a binding into a Tier-2 program
(predicated puts chained into one strong signal, then a planned wait), which the pass
pipeline specialises per transport like any other program.

Data model after the reference (python/aboleth/transport_binding.py:16-265; the program
records of python/aboleth/pattern.py); slot types are i1 / i32 / i64.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Sequence

from .compiler.language import ProgramBuilder

ARTIFACT_KINDS = ("inline_fragment", "bindable_epilogue", "standalone_kernel")
_CUDA_TYPES = {"i1": "i32", "i32": "i32", "i64": "u64"}


SLOT_KINDS = {"i1": "a predicate", "i32": "a 32-bit integer", "i64": "a 64-bit address or handle"}


def _expect(slot: "BoundScalar", kind: str, role: str) -> None:
    if slot.kind != kind:
        raise ValueError(f"{role} {slot.name!r} is declared {slot.kind}; it has to be {kind} "
                         f"({SLOT_KINDS[kind]})")


@dataclass(frozen=True)
class BoundScalar:
    """One named scalar a client kernel supplies at the insertion point.  ``kind`` is the slot's
    width class: ``i1`` predicate, ``i32`` count / key / counter, ``i64`` address or handle."""

    name: str
    kind: str

    def __post_init__(self):
        if not self.name or not (self.name[0].isalpha() or self.name[0] == "_"):
            raise ValueError(f"slot name {self.name!r} is not an identifier")
        if self.kind not in SLOT_KINDS:
            raise ValueError(f"slot {self.name!r}: kind {self.kind!r} is not one of {sorted(SLOT_KINDS)}")


@dataclass(frozen=True)
class RegionSide:
    """One end of a transfer: where the bytes are and the key that authorises the access."""

    pointer: BoundScalar
    key: BoundScalar

    def __post_init__(self):
        _expect(self.pointer, "i64", "region pointer")
        _expect(self.key, "i32", "region key")


@dataclass(frozen=True)
class RegionBinding:
    """A predicated transfer of at most ``max_bytes`` from ``local`` to ``remote`` that carries
    out the logical ``operations`` named."""

    remote: RegionSide
    local: RegionSide
    byte_count: BoundScalar
    predicate: BoundScalar
    max_bytes: int
    operations: tuple[str, ...] = ()

    def __post_init__(self):
        _expect(self.byte_count, "i32", "byte count")
        _expect(self.predicate, "i1", "transfer predicate")
        if self.max_bytes < 1:
            raise ValueError(f"a region moves at least one byte, max_bytes is {self.max_bytes}")

    def slots(self) -> tuple[BoundScalar, ...]:
        return tuple(slot for _, slot in self.roles())

    def roles(self) -> tuple[tuple[str, BoundScalar], ...]:
        """(role, slot) in the order a program takes them."""
        return (("remote pointer", self.remote.pointer), ("local pointer", self.local.pointer),
                ("byte count", self.byte_count), ("local key", self.local.key),
                ("remote key", self.remote.key), ("predicate", self.predicate))


@dataclass(frozen=True)
class PublicationBinding:
    """The flag that publishes an attachment (epoch = iteration + 1) and the loop counters the
    completion planner works with."""

    remote: RegionSide
    local: RegionSide
    iteration: BoundScalar
    iterations: BoundScalar

    def __post_init__(self):
        _expect(self.iteration, "i32", "iteration counter")
        _expect(self.iterations, "i32", "iteration bound")

    def slots(self) -> tuple[BoundScalar, ...]:
        return tuple(slot for _, slot in self.roles())

    def roles(self) -> tuple[tuple[str, BoundScalar], ...]:
        return (("remote pointer", self.remote.pointer), ("local pointer", self.local.pointer),
                ("local key", self.local.key), ("remote key", self.remote.key),
                ("iteration", self.iteration), ("iterations", self.iterations))


# The records below are what a bound program looks like from the client kernel's side: plain
# names, in the order the program takes them.

@dataclass(frozen=True)
class KernelTransportArgument:
    name: str
    kind: str


@dataclass(frozen=True)
class KernelTransportTransfer:
    operations: tuple[str, ...]
    destination: str
    source: str
    byte_count: str
    source_key: str
    destination_key: str
    predicate: str
    max_bytes: int


@dataclass(frozen=True)
class KernelTransportSignal:
    destination: str
    source: str
    source_key: str
    destination_key: str
    iteration: str
    iterations: str


@dataclass(frozen=True)
class KernelTransportReduction:
    """A reduction the client kernel applies while it consumes the received rows."""

    operation: str
    sources: tuple[str, ...]
    destination: str
    combiner: str = "add"

    def __post_init__(self):
        if not self.operation or not self.sources or not self.destination:
            raise ValueError("a transport reduction names an operation, sources and a destination")


@dataclass(frozen=True)
class KernelTransportTransform:
    """A transform the packing kernel applies while it produces the source (e.g. fp8 quantisation)."""

    operation: str
    name: str
    role: str = "values"


@dataclass(frozen=True)
class KernelTransportProgram:
    name: str
    operations: tuple[str, ...]
    kernel: str
    insertion_point: str
    arguments: tuple[KernelTransportArgument, ...]
    transfers: tuple[KernelTransportTransfer, ...]
    signal: Optional[KernelTransportSignal]
    artifact: str = "inline_fragment"
    reductions: tuple[KernelTransportReduction, ...] = ()
    transforms: tuple[KernelTransportTransform, ...] = ()
    program_id: Optional[int] = None


@dataclass(frozen=True)
class TransportProgramBinding:
    name: str
    operations: tuple[str, ...]
    kernel: str
    insertion_point: str
    endpoint: BoundScalar
    regions: tuple[RegionBinding, ...]
    publication: PublicationBinding
    artifact: str = "inline_fragment"
    reductions: tuple[KernelTransportReduction, ...] = ()
    transforms: tuple[KernelTransportTransform, ...] = ()

    def __post_init__(self):
        if not self.name or not self.kernel or not self.insertion_point:
            raise ValueError("transport binding requires name, kernel, and insertion point")
        if self.artifact not in ARTIFACT_KINDS:
            raise ValueError(f"unknown artifact kind {self.artifact!r}; expected one of "
                             + ", ".join(ARTIFACT_KINDS))
        _expect(self.endpoint, "i64", "endpoint handle")
        if not self.operations or not self.regions:
            raise ValueError("transport binding requires operations and regions")
        realized = tuple(op for region in self.regions for op in region.operations)
        if len(realized) != len(set(realized)) or set(realized) != set(self.operations):
            raise ValueError("transport binding must realize each logical operation once")

    def slots(self) -> tuple[BoundScalar, ...]:
        """The bound scalars in invocation order.  One name is one role: the same name under
        two roles is refused (the second role would be issued through the first one's storage)."""
        candidates = [("endpoint", self.endpoint)]
        for index, region in enumerate(self.regions):
            candidates += [(f"region {index} {role}", slot) for role, slot in region.roles()]
        candidates += [(f"publication {role}", slot) for role, slot in self.publication.roles()]
        result, roles = [], {}
        for role, slot in candidates:
            previous = roles.get(slot.name)
            if previous is None:
                roles[slot.name] = (role, slot.kind)
                result.append(slot)
            elif previous != (role, slot.kind):
                raise ValueError(f"transport binding {self.name!r} binds slot {slot.name!r} to two roles: "
                                 f"the {previous[0]} ({previous[1]}) and the {role} ({slot.kind})")
        return tuple(result)

    def to_program(self, program_id: Optional[int] = None) -> KernelTransportProgram:
        return KernelTransportProgram(
            name=self.name, operations=self.operations, kernel=self.kernel,
            insertion_point=self.insertion_point,
            arguments=tuple(KernelTransportArgument(s.name, s.kind) for s in self.slots()),
            transfers=tuple(KernelTransportTransfer(
                operations=r.operations, destination=r.remote.pointer.name, source=r.local.pointer.name,
                byte_count=r.byte_count.name, source_key=r.local.key.name,
                destination_key=r.remote.key.name, predicate=r.predicate.name, max_bytes=r.max_bytes)
                for r in self.regions),
            signal=KernelTransportSignal(
                destination=self.publication.remote.pointer.name, source=self.publication.local.pointer.name,
                source_key=self.publication.local.key.name, destination_key=self.publication.remote.key.name,
                iteration=self.publication.iteration.name, iterations=self.publication.iterations.name),
            artifact=self.artifact, reductions=self.reductions, transforms=self.transforms,
            program_id=program_id)

    def to_builder(self, *, reuse: int = 1, threads: int = 32) -> ProgramBuilder:
        """The attachment as a Tier-2 program whose arguments are the slots, in slot order.

        Every region becomes one predicated put; the puts are chained, the last one carries
        the strong signal (epoch = iteration + 1), and a planned wait with ``reuse`` lets the
        completion pass pick the interval."""
        args = [(s.name, _CUDA_TYPES[s.kind]) for s in self.slots()]
        b = ProgramBuilder(_symbol(self.name), args=args, threads=threads)
        # The endpoint slot carries the handle itself: a one-entry table at the argument's address.
        endpoint = b.endpoint(f"(&{self.endpoint.name})", 0)
        token = None
        for region in self.regions:
            dst = b.remote_at(region.remote.pointer.name, key=region.remote.key.name)
            src = b.local(region.local.pointer.name, key=region.local.key.name)
            token = b.put(endpoint, dst, src, bytes=region.byte_count.name, after=token,
                          predicate=region.predicate.name)
        flag = b.remote_at(self.publication.remote.pointer.name, key=self.publication.remote.key.name)
        ready = b.signal(endpoint, flag, epoch=f"{self.publication.iteration.name} + 1", after=token)
        b.wait(ready, iteration=self.publication.iteration.name, reuse=reuse,
               final=f"{self.publication.iteration.name} + 1 == {self.publication.iterations.name}")
        return b


    def to_fragment(self, program_id: int, *, interval: Optional[int] = None,
                    capacities: Sequence[int] = (), reuse: Optional[int] = None) -> str:
        """The attachment as a ``fragment`` of an external transport program, for
        ``compile_program(kernel, plan=...)``: its parameters are the slots (all 64-bit
        placeholders, in slot order), its body is :meth:`to_builder`'s.  With ``interval`` a
        ``phase`` record carries the resolved completion interval and the peers' queue capacities,
        and the fragment's wait takes them at the splice; with ``reuse`` the wait keeps a reuse
        distance of its own instead."""
        builder = self.to_builder(reuse=reuse or 1)
        body = [line for line in builder.text(backend="p2p", rank=0, world_size=1).splitlines()
                if line and not line.startswith(("program ", "arg "))]
        if reuse is None:
            body = [line.replace(" reuse=1", "") if line.lstrip().startswith("planned_wait") else line
                    for line in body]
        params = ",".join(f"{slot.name}:i64" for slot in self.slots())
        symbol = _symbol(self.name)
        text = ""
        if interval is not None:
            if interval < 1:
                raise ValueError("a resolved completion interval is at least 1")
            text += f"phase {symbol} program_id={program_id} interval={interval}"
            if capacities:
                text += " capacities=" + ",".join(str(int(c)) for c in capacities)
            text += "\n"
        elif reuse is None:
            raise ValueError("a fragment needs a planned interval or a reuse distance")
        return text + f"fragment {symbol} program_id={program_id} params={params} {{\n" + \
            "".join(f"  {line}\n" for line in body) + "}\n"

    def invoke_text(self, program_id: int, **slots: str) -> str:
        """The ``invoke_phase`` line a kernel states at its insertion point: every slot once, in
        slot order (values of the kernel's own program, argument names or expressions)."""
        names = [slot.name for slot in self.slots()]
        missing, extra = [n for n in names if n not in slots], [n for n in slots if n not in names]
        if missing or extra:
            raise ValueError(f"transport program {program_id}: missing slots {missing}, unknown slots {extra}")
        rendered = []
        for name in names:
            text = str(slots[name])
            rendered.append(f"({text})" if any(c.isspace() for c in text) and not text.startswith("(") else text)
        return " ".join(["invoke_phase", str(int(program_id)), *rendered])


def transport_program_text(name: str, fragments: Sequence[str]) -> str:
    """An external transport program: the module ``compile_program(..., plan=...)`` reads."""
    return f"program {_symbol(name)} kind=transport_program\n" + "".join(fragments)


def _symbol(name: str) -> str:
    stem = "".join(c if c.isalnum() else "_" for c in name)
    return ("t_" + stem) if not stem[:1].isalpha() else stem


@dataclass(frozen=True)
class InvokeManifest:
    program_id: int
    arguments: tuple[KernelTransportArgument, ...]
    transfers: tuple[KernelTransportTransfer, ...]
    signal: Optional[KernelTransportSignal]

    @property
    def slot_names(self) -> tuple[str, ...]:
        return tuple(a.name for a in self.arguments)


def invoke_manifest(program: KernelTransportProgram) -> InvokeManifest:
    if program.program_id is None:
        raise ValueError("transport program is not bound")
    return InvokeManifest(program.program_id, program.arguments, program.transfers, program.signal)


def invoke_transport_program(manifest: InvokeManifest, symbol: str, **slots: str) -> str:
    """The call a CUDA client writes at its insertion point: every slot of the manifest must be
    given exactly once (as a C++ expression); returns ``symbol(expr, ...);`` in slot order."""
    missing = [n for n in manifest.slot_names if n not in slots]
    extra = [n for n in slots if n not in manifest.slot_names]
    if missing or extra:
        raise ValueError(f"transport program {manifest.program_id}: missing slots {missing}, unknown slots {extra}")
    casts = {"i64": "static_cast<std::uint64_t>", "i32": "static_cast<int>", "i1": "static_cast<int>"}
    values = ", ".join(f"{casts[a.kind]}({slots[a.name]})" for a in manifest.arguments)
    return f"{symbol}({values});"
