"""Tier 2: a program builder and a specializer that plans completion, ordering and
batching and emits CUDA C++ for sm_100a."""
from .artifact import Artifact, LoadedKernel, build_artifact, cache_dir
from .driver import (CompileError, CompiledProgram, compile_program, include_dir, library_digest,
                     materialize_phases,
                     pipeline_key, run_planner)
from .language import ProgramBuilder, Token, Value
from .options import (DEFAULT_INLINE_BYTES, OPTIMIZATIONS, PIPELINE_ORDER, CompileOptions,
                      compilation, current_options, enabled_optimizations)
