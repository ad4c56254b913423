"""Externally attached planned transport fragments.

A client that owns its kernels can attach four small device functions instead of a whole
transport program: a predicated ``put`` whose publication happens elsewhere, the
``publish`` of everything posted so far, a system ``fence`` and the ``drain`` that
reclaims the endpoint.  Each is a Tier-2 program compiled to device code for the current
transport (on peer memory the publish and the drain lower to fences only; on queue
transports to the doorbell and the completion poll).

After the reference's python/aboleth/planned_phase.py:18-200 (same four programs, slot
names and insertion points).
"""
from __future__ import annotations

from .compiler.artifact import FragmentArtifact
from .compiler.driver import compile_program
from .compiler.language import ProgramBuilder
from .physicalization import Artifact

PLANNED_FRAGMENT_MAX_REGISTERS = 64

PUT_SLOTS = (("endpoint", "i64"), ("destination", "i64"), ("source", "i64"), ("bytes", "i32"),
             ("source_key", "i32"), ("destination_key", "i32"), ("predicate", "i1"))
_CUDA = {"i64": "u64", "i32": "i32", "i1": "i32"}


def _builder(name: str, slots) -> ProgramBuilder:
    return ProgramBuilder(name.replace(".", "_"), args=[(n, _CUDA[t]) for n, t in slots], threads=32)


def planned_put_program(*, name: str = "phase.put", max_bytes: int, cta_exclusive: bool = False) -> ProgramBuilder:
    """One predicated put through ``endpoint``; nothing is published here (the client publishes with
    the publish fragment).  ``cta_exclusive``: the calling CTA is the endpoint's only issuer."""
    if max_bytes <= 0:
        raise ValueError("planned put max_bytes must be positive")
    b = _builder(name, PUT_SLOTS)
    ep = b.endpoint("(&endpoint)", 0)
    token = b.put(ep, b.remote_at("destination", key="destination_key"), b.local("source", key="source_key"),
                  bytes="bytes", predicate="predicate")
    b.wait(token)
    b.insertion_point, b.max_bytes, b.reservation_scope = "payload_put", max_bytes, "cta" if cta_exclusive else "gpu"
    return b


def planned_publish_program(*, name: str = "phase.publish") -> ProgramBuilder:
    """Make everything posted on ``endpoint`` so far visible to the peer (a system fence on peer
    memory, the doorbell on a queue)."""
    b = _builder(name, (("endpoint", "i64"), ("only_if_advanced", "i1")))
    with b.if_("only_if_advanced"):
        b.system_fence()
    b.insertion_point = "phase_publish"
    return b


def planned_fence_program(*, name: str = "phase.fence") -> ProgramBuilder:
    b = _builder(name, (("predicate", "i1"),))
    with b.if_("predicate"):
        b.system_fence()
    b.insertion_point = "phase_fence"
    return b


def planned_drain_program(*, name: str = "phase.drain") -> ProgramBuilder:
    """Wait until the endpoint has retired everything it was given (vacuous on peer memory)."""
    b = _builder(name, (("endpoint", "i64"),))
    b.drain(b.endpoint("(&endpoint)", 0))
    b.insertion_point = "phase_reclaim"
    return b


def _compile(builder: ProgramBuilder, artifact: Artifact, options=None) -> FragmentArtifact:
    compiled = compile_program(builder, options)
    if compiled.cuda is None:
        raise ValueError("the pipeline was stopped before the lowering; nothing to attach")
    symbol = compiled.name + "_fragment"
    source = compiled.cuda.replace(f'extern "C" __global__ void {compiled.name}(',
                                   f"__device__ __forceinline__ void {symbol}(", 1)
    parameters = tuple((n, {"u64": "unsigned long long", "i32": "int"}[t]) for n, t in builder.args)
    return FragmentArtifact(builder.name, symbol, artifact.value, source, parameters, compiled.facts,
                            compiled.key)


def compile_planned_put_artifact(*, max_bytes: int, cta_exclusive: bool = False,
                                 artifact: Artifact = Artifact.BINDABLE_EPILOGUE, options=None) -> FragmentArtifact:
    return _compile(planned_put_program(max_bytes=max_bytes, cta_exclusive=cta_exclusive), artifact, options)


def compile_planned_publish_artifact(*, artifact: Artifact = Artifact.BINDABLE_EPILOGUE,
                                     options=None) -> FragmentArtifact:
    return _compile(planned_publish_program(), artifact, options)


def compile_planned_fence_artifact(*, artifact: Artifact = Artifact.BINDABLE_EPILOGUE,
                                   options=None) -> FragmentArtifact:
    return _compile(planned_fence_program(), artifact, options)


def compile_planned_drain_artifact(*, artifact: Artifact = Artifact.BINDABLE_EPILOGUE,
                                   options=None) -> FragmentArtifact:
    return _compile(planned_drain_program(), artifact, options)
