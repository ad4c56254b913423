"""Physicalisation: attach the transfers of a compiled pattern to client kernels.

``physicalize_pattern`` takes a :class:`CompiledPattern` and, per attachment, a
:class:`PhaseBinding` (which client kernel produces or consumes the data, where the
communication is inserted, how many peer segments and which publication).  For each it
derives the slots a client kernel must supply - one region pair per surviving transfer of
the attachment, named after the logical regions - and returns
:class:`TransportProgramBinding` objects with stable program ids.  ``RuntimeBindings`` maps
logical regions onto the runtime buffers that back them.

Role of the reference's python/aboleth/physicalization.py:28-833 (artifact forms 28-37,
attachment 60-105, result 108-127, runtime bindings 131-206, entry point 817-833).
"""
from __future__ import annotations

from dataclasses import dataclass
from enum import Enum
from typing import Callable, Optional, Sequence

from .pattern import CompiledPattern
from .planning import RegionEffect
from .transport_binding import (BoundScalar, InvokeManifest, KernelTransportProgram,
                                KernelTransportReduction, KernelTransportTransform, PublicationBinding,
                                RegionBinding, RegionSide, TransportProgramBinding, invoke_manifest)


class Artifact(Enum):
    """The three forms an attachment's communication may be materialised as."""

    INLINE_FRAGMENT = "inline_fragment"        # device code included into the client kernel
    BINDABLE_EPILOGUE = "bindable_epilogue"    # a device function the client calls last
    STANDALONE_KERNEL = "standalone_kernel"    # its own launch between client kernels


_PHYSICALIZED_KINDS = ("transfer", "reduction", "copy", "transform")
_KNOWN_TRANSFORM_STEMS = ("quantize.e4m3.g128",)


@dataclass(frozen=True)
class PhaseBinding:
    """Where one generated communication phase meets client code."""

    producer: Optional[str]
    consumer: Optional[str]
    name: str
    kernel: str
    insertion_point: str
    peer_segments: int
    publication: str
    items_per_transfer: int = 0
    artifact: Artifact = Artifact.INLINE_FRAGMENT
    operations: tuple[str, ...] = ()   # logical operations realised here (default: the one named `name`)

    def __post_init__(self):
        for field in ("name", "kernel", "insertion_point", "publication"):
            if not getattr(self, field):
                raise ValueError(f"communication attachment {field} cannot be empty")
        if self.producer is None and self.consumer is None:
            raise ValueError("communication attachment requires a producer or consumer boundary")
        if self.peer_segments <= 0:
            raise ValueError("communication attachment peer_segments must be positive")
        if self.items_per_transfer < 0:
            raise ValueError("items_per_transfer cannot be negative")
        if not isinstance(self.artifact, Artifact):
            raise ValueError(f"communication attachment artifact must be an Artifact, got {self.artifact!r}; "
                             "expected one of " + ", ".join(f"Artifact.{k.name}" for k in Artifact))


@dataclass(frozen=True)
class PhysicalizedPattern:
    compiled: CompiledPattern
    bindings: tuple[TransportProgramBinding, ...]
    programs: tuple[KernelTransportProgram, ...]

    def binding(self, name: str) -> TransportProgramBinding:
        for b in self.bindings:
            if b.name == name:
                return b
        raise KeyError(f"no transport binding named {name!r}")

    def program(self, name: str) -> KernelTransportProgram:
        for p in self.programs:
            if p.name == name:
                return p
        raise KeyError(f"no transport program named {name!r}")

    def manifest(self, name: str) -> InvokeManifest:
        return invoke_manifest(self.program(name))


@dataclass(frozen=True)
class RuntimeBufferBinding:
    buffer: str
    regions: tuple[str, ...]

    def __post_init__(self):
        if not self.buffer or not self.regions:
            raise ValueError("runtime buffer binding requires a buffer and regions")
        if len(self.regions) != len(set(self.regions)):
            raise ValueError("runtime buffer binding regions must be unique")


@dataclass(frozen=True)
class RuntimeBindings:
    buffers: tuple[RuntimeBufferBinding, ...]

    def __post_init__(self):
        regions = tuple(r for b in self.buffers for r in b.regions)
        if len(regions) != len(set(regions)):
            raise ValueError("logical regions may bind to only one runtime buffer")

    def effects(self, compiled: CompiledPattern, resolve: Callable[[str], RegionEffect]) -> dict[str, RegionEffect]:
        """``{logical region: what `resolve` says about its runtime buffer}`` for every region the
        simplified pattern still allocates.  Missing and unknown regions are errors; regions the
        simplifier removed may be listed and are ignored."""
        by_region = {r: b.buffer for b in self.buffers for r in b.regions}
        removed = set(compiled.dataflow.unallocated_regions)
        required = {r.name for r in compiled.regions} - removed
        missing = required - set(by_region)
        if missing:
            raise KeyError("no runtime buffer binding for logical regions: " + ", ".join(sorted(missing)))
        unknown = set(by_region) - required - removed
        if unknown:
            raise KeyError("runtime bindings reference unknown logical regions: " + ", ".join(sorted(unknown)))
        used = {by_region[r] for r in required}
        resolved = {b.buffer: resolve(b.buffer) for b in self.buffers if b.buffer in used}
        return {r: resolved[by_region[r]] for r in sorted(required)}


def _slot(value: str) -> str:
    """A region or operation name as an identifier stem."""
    stem = "".join(c if c.isalnum() else "_" for c in value).strip("_")
    if not stem:
        raise ValueError(f"{value!r} does not make a slot name")
    return stem if stem[0].isalpha() else "r_" + stem


def _side(stem: str) -> RegionSide:
    return RegionSide(BoundScalar(stem + "_ptr", "i64"), BoundScalar(stem + "_key", "i32"))


def _physicalize_attachment(compiled: CompiledPattern, attachment: PhaseBinding,
                            program_id: int) -> tuple[TransportProgramBinding, KernelTransportProgram]:
    stage_names = {s.name for s in compiled.stages}
    for boundary in (attachment.producer, attachment.consumer):
        if boundary is not None and boundary not in stage_names:
            raise KeyError(f"attachment {attachment.name!r} names unknown opaque stage {boundary!r}")
    wanted = attachment.operations or (attachment.name,)
    by_name = {op["name"]: op for op in compiled.dataflow.operations}
    by_region = {r.name: r for r in compiled.regions}
    regions, reductions, transforms, realised = [], [], [], []
    for name in wanted:
        op = by_name.get(name)
        if op is None:
            removed = {r["name"]: r.get("why", "") for r in compiled.dataflow.removed}
            if name in removed:
                raise ValueError(f"operation {name!r} was removed by the simplifier ({removed[name]}); "
                                 "it cannot be attached")
            raise KeyError(f"attachment {attachment.name!r} names unknown operation {name!r}")
        if op["kind"] not in _PHYSICALIZED_KINDS:
            raise ValueError(f"operation {name!r} of kind {op['kind']!r} cannot be physicalised")
        if op["kind"] == "transform":
            if not any(name.startswith(stem) or op.get("src", "").startswith(stem) or stem in name
                       for stem in _KNOWN_TRANSFORM_STEMS):
                raise ValueError(f"transform {name!r} is not one physicalisation can obligate a kernel with")
            transforms.append(KernelTransportTransform(name, op["dst"], name.rsplit(".", 1)[-1]))
            continue
        if op["kind"] == "reduction":
            reductions.append(KernelTransportReduction(name, tuple(op["src"].split(",")), op["dst"]))
            continue
        src, dst = by_region.get(op["src"]), by_region.get(op["dst"])
        if src is None or dst is None:
            raise KeyError(f"operation {name!r} touches an undeclared region")
        rows = src.rows if not attachment.items_per_transfer else min(src.rows, attachment.items_per_transfer)
        stem = _slot(name)
        regions.append(RegionBinding(
            remote=_side(_slot(op["dst"])), local=_side(_slot(op["src"])),
            byte_count=BoundScalar(stem + "_bytes", "i32"), predicate=BoundScalar(stem + "_live", "i1"),
            max_bytes=max(rows * src.row_bytes // attachment.peer_segments, 1), operations=(name,)))
        realised.append(name)
    if not regions:
        raise ValueError(f"attachment {attachment.name!r} realises no transfer")
    stem = _slot(attachment.name)
    publication = PublicationBinding(
        remote=_side(stem + "_ready"), local=_side(stem + "_ready_src"),
        iteration=BoundScalar(stem + "_iteration", "i32"), iterations=BoundScalar(stem + "_iterations", "i32"))
    binding = TransportProgramBinding(
        name=attachment.name, operations=tuple(realised), kernel=attachment.kernel,
        insertion_point=attachment.insertion_point, endpoint=BoundScalar(stem + "_endpoint", "i64"),
        regions=tuple(regions), publication=publication, artifact=attachment.artifact.value,
        reductions=tuple(reductions), transforms=tuple(transforms))
    return binding, binding.to_program(program_id)


def physicalize_pattern(compiled: CompiledPattern, attachments: Sequence[PhaseBinding]) -> PhysicalizedPattern:
    """One transport program per attachment; program ids follow the attachment order."""
    names = [a.name for a in attachments]
    if len(names) != len(set(names)):
        raise ValueError("communication attachments must have unique names")
    claimed: dict[str, str] = {}
    bindings, programs = [], []
    for program_id, attachment in enumerate(attachments):
        binding, program = _physicalize_attachment(compiled, attachment, program_id)
        for op in binding.operations:
            if op in claimed:
                raise ValueError(f"operation {op!r} is attached twice ({claimed[op]!r} and {attachment.name!r})")
            claimed[op] = attachment.name
        bindings.append(binding)
        programs.append(program)
    return PhysicalizedPattern(compiled, tuple(bindings), tuple(programs))
