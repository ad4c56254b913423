"""Driver of the Tier-2 specializer: text IR in, scheduled IR + CUDA C++ + facts out.

The pass pipeline itself is native (``csrc/spec``, ``libab200_spec.so``); this
module calls it, keys the result for caching, and turns emitted source into a
loadable artefact with nvcc (offline, ``-arch=sm_100a``).
"""
from __future__ import annotations

import ctypes
import hashlib
import json
import os
from dataclasses import dataclass, field
from pathlib import Path
from typing import Optional, Union

from .. import _native
from .language import ProgramBuilder
from .options import CompileOptions, current_options


class CompileError(ValueError):
    """The program violates a rule of the dialect or cannot be lowered."""


def _lib() -> ctypes.CDLL:
    lib = _native.load("spec")
    if not getattr(lib, "_ab_typed", False):
        for name in ("ab200_spec_compile", "ab200_spec_plan", "ab200_spec_materialize"):
            fn = getattr(lib, name)
            fn.restype = ctypes.c_void_p
            fn.argtypes = [ctypes.c_char_p, ctypes.c_char_p]
        lib.ab200_spec_affine.restype = ctypes.c_void_p
        lib.ab200_spec_affine.argtypes = [ctypes.c_char_p]
        lib.ab200_spec_free.argtypes = [ctypes.c_void_p]
        lib._ab_typed = True
    return lib


def _call(fn, *args) -> dict:
    lib = _lib()
    raw = fn(*[a.encode() if isinstance(a, str) else a for a in args])
    try:
        text = ctypes.string_at(raw).decode()
    finally:
        lib.ab200_spec_free(raw)
    result = json.loads(text)
    if not result.get("ok"):
        raise CompileError(result.get("error", "specializer failed"))
    return result


def library_digest() -> str:
    """Hash of the specializer library: part of every artefact key."""
    path = _native.library_path("spec")
    if not path.exists():
        _native.build("spec")
    return hashlib.sha256(path.read_bytes()).hexdigest()[:16]


def pipeline_key(program_text: str, options: CompileOptions) -> str:
    """Cache identity of one compilation.  Every input that can change the emitted
    code takes part: the specializer build, the transport, copy mode, completion
    interval, plan hash, inline bytes, every switch, queue capacity, registration
    strictness, queue placement, endpoint profile, target architecture."""
    h = hashlib.sha256()
    for part in (library_digest(), options.backend, options.p2p_copy, options.completion_interval,
                 options.plan_hash, options.inline_bytes, ",".join(sorted(options.passes)),
                 options.queue_capacity, int(options.strict_registrations),
                 int(options.gpu_resident_queues), options.endpoint_profile, options.arch,
                 options.coop_min, options.coop_elements, options.rank, options.world_size,
                 options.stop_after, program_text):
        h.update(str(part).encode())
        h.update(b"\0")
    return h.hexdigest()


@dataclass
class CompiledProgram:
    name: str
    ir: str                      # scheduled IR after the last pass that ran
    cuda: Optional[str]          # emitted CUDA C++ (None when stop_after cut the pipeline)
    facts: dict                  # batches, fences, flag writes, ... (see lower.cpp)
    passes: dict                 # rewrites made per pass
    key: str
    options: CompileOptions
    source: str = field(repr=False, default="")


def materialize_phases(program_text: str, plan_text: str) -> str:
    """``materialize-transport-phase``: replace every ``invoke_phase <id> <args...>`` of the program
    by the body of the fragment with that program id in the external transport program ``plan_text``.

    The plan is a program of its own (``program <name> kind=transport_program``) whose body holds
    ``phase <name> program_id=<id> interval=<k> capacities=<c0,c1,...>`` records and
    ``fragment <name> program_id=<id> params=<p:type,...> { ... }`` definitions.  Planned waits of
    the spliced body that carry no reuse distance receive the smallest completion interval and the
    smallest peer queue capacity of the phases bound to that id
    (reference: compiler/lib/Transforms/MaterializeTransportPhase.cpp:28-217).
    """
    return _call(_lib().ab200_spec_materialize, program_text, plan_text)["ir"]


def compile_program(program: Union[str, ProgramBuilder], options: Optional[CompileOptions] = None,
                    *, plan: Optional[str] = None, **overrides) -> CompiledProgram:
    """Run the pass pipeline and the lowering for the current (or given) options.  ``plan`` is the
    external transport program for a kernel that contains ``invoke_phase`` operations."""
    from dataclasses import replace

    opts = options or current_options()
    if overrides:
        opts = replace(opts, **overrides)
    text = program if isinstance(program, str) else program.text(
        backend=opts.backend, rank=opts.rank, world_size=opts.world_size)
    if plan is not None:
        text = materialize_phases(text, plan)
    result = _call(_lib().ab200_spec_compile, text, opts.to_native())
    name = text.split()[1] if text.startswith("program") else "program"
    compiled = CompiledProgram(name=name, ir=result["ir"], cuda=result.get("cuda"),
                               facts=result.get("facts", {}), passes=result.get("passes", {}),
                               key=pipeline_key(text, opts), options=opts, source=text)
    _dump(compiled)
    return compiled


def _dump(compiled: CompiledProgram) -> None:
    """``ABOLETH_DUMP_SCHEDULED_IR=<dir>`` writes, per compilation, the input program, the IR after the
    last pass that ran, the emitted CUDA C++ and the facts (the reference dumps its post-schedule IR the
    same way, python/aboleth/compiler.py:399-404)."""
    root = os.environ.get("ABOLETH_DUMP_SCHEDULED_IR")
    if not root:
        return
    out = Path(root) / f"{compiled.name}-{compiled.options.backend}-{compiled.key[:12]}"
    out.mkdir(parents=True, exist_ok=True)
    (out / "program.txt").write_text(compiled.source)
    (out / "scheduled.ir").write_text(compiled.ir)
    if compiled.cuda is not None:
        (out / "kernel.cu").write_text(compiled.cuda)
    (out / "facts.json").write_text(json.dumps({"facts": compiled.facts, "passes": compiled.passes}, indent=1))


def run_planner(kind: str, request: str) -> dict:
    """Run one native planning pass (see csrc/spec/planning.cpp)."""
    return _call(_lib().ab200_spec_plan, kind, request)


def affine_in_program_id(expr: str) -> dict:
    return _call.__wrapped__(expr) if hasattr(_call, "__wrapped__") else json.loads(_affine(expr))


def _affine(expr: str) -> str:
    lib = _lib()
    raw = lib.ab200_spec_affine(expr.encode())
    try:
        return ctypes.string_at(raw).decode()
    finally:
        lib.ab200_spec_free(raw)


def include_dir() -> Path:
    return Path(_native.__file__).resolve().parent / "include"


def install_compiler() -> None:
    """Make the specializer ready: build (if stale) and load the native pass library.

    The reference hooks its passes into another compiler's stage list
    (python/aboleth/compiler.py:470-471); here the pipeline is this package's own native
    library, so installing means having it built and loaded.  Idempotent."""
    _lib()
