"""Offline artefacts of emitted Tier-2 kernels: nvcc -> cubin, keyed and cached.

Mirrors the reference's artefact pipeline in spirit
(python/aboleth/artifact.py:108-278: fragment pipeline -> PTX -> ``ptxas -c``,
binding signature hash, resource fields), with nvcc compiling emitted CUDA C++
for ``sm_100a`` instead of Triton/LLVM.  The cache is digest-keyed and guarded
by a file lock so that ranks started together build once.
"""
from __future__ import annotations

import ctypes
import fcntl
import hashlib
import json
import os
import re
import shutil
import subprocess
from dataclasses import dataclass
from pathlib import Path
from typing import Optional, Sequence

from .driver import CompiledProgram, include_dir


def cache_dir() -> Path:
    root = os.environ.get("ABOLETH_CACHE_DIR") or os.path.join(
        os.environ.get("XDG_CACHE_HOME", os.path.expanduser("~/.cache")), "aboleth_b200", "artifacts")
    path = Path(root)
    path.mkdir(parents=True, exist_ok=True)
    return path


@dataclass(frozen=True)
class Artifact:
    name: str
    key: str
    cubin: Path
    source: Path
    registers: Optional[int]
    spill_bytes: Optional[int]
    shared_bytes: Optional[int]
    cubin_bytes: int
    signature: str               # sha256 of the kernel's argument list (binding signature)

    def manifest(self) -> dict:
        return {"name": self.name, "key": self.key, "n_regs": self.registers,
                "n_spills": self.spill_bytes, "shared": self.shared_bytes,
                "cubin_bytes": self.cubin_bytes, "signature": self.signature}


def _nvcc() -> str:
    path = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(path).exists():
        raise RuntimeError("nvcc was not found; emitted kernels cannot be compiled")
    return path


def build_artifact(compiled: CompiledProgram, *, force: bool = False) -> Artifact:
    """Compile the emitted source to a cubin for the compilation's architecture."""
    if compiled.cuda is None:
        raise ValueError("the pipeline was stopped before the lowering; nothing to build")
    out = cache_dir() / compiled.key[:2] / compiled.key
    out.mkdir(parents=True, exist_ok=True)
    cubin, source, meta = out / "kernel.cubin", out / "kernel.cu", out / "manifest.json"
    with open(out / ".lock", "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        if force or not (cubin.exists() and meta.exists()):
            source.write_text(compiled.cuda)
            arch = compiled.options.arch
            cmd = [_nvcc(), "-gencode", f"arch=compute_{arch[3:]},code={arch}", "-O3", "-std=c++17",
                   "-lineinfo", f"-I{include_dir()}", "-Xptxas", "-v", "-cubin", "-o", str(cubin),
                   str(source)]
            proc = subprocess.run(cmd, capture_output=True, text=True)
            if proc.returncode != 0:
                raise RuntimeError("nvcc failed on emitted kernel:\n" + proc.stderr)
            log = proc.stdout + proc.stderr
            regs = re.search(r"Used (\d+) registers", log)
            spill = re.search(r"(\d+) bytes spill stores", log)
            smem = re.search(r"(\d+) bytes smem", log)
            header = re.search(r"__global__ void \w+\(([^)]*)\)", compiled.cuda)
            meta.write_text(json.dumps({
                "registers": int(regs.group(1)) if regs else None,
                "spill_bytes": int(spill.group(1)) if spill else None,
                "shared_bytes": int(smem.group(1)) if smem else 0,
                "signature": hashlib.sha256((header.group(1) if header else "").encode()).hexdigest(),
            }))
        info = json.loads(meta.read_text())
    return Artifact(compiled.name, compiled.key, cubin, source, info["registers"],
                    info["spill_bytes"], info["shared_bytes"], cubin.stat().st_size,
                    info["signature"])


class LoadedKernel:
    """A cubin loaded through the CUDA driver; ``launch`` enqueues it on a stream."""

    def __init__(self, artifact: Artifact):
        self._cuda = ctypes.CDLL("libcuda.so.1")
        self._module = ctypes.c_void_p()
        self._function = ctypes.c_void_p()
        data = artifact.cubin.read_bytes()
        self._check(self._cuda.cuModuleLoadData(ctypes.byref(self._module), data), "cuModuleLoadData")
        self._check(self._cuda.cuModuleGetFunction(ctypes.byref(self._function), self._module,
                                                   artifact.name.encode()), "cuModuleGetFunction")
        self.artifact = artifact

    def _check(self, rc: int, what: str) -> None:
        if rc != 0:
            raise RuntimeError(f"{what} failed with CUresult {rc}")

    def launch(self, grid: int, threads: int, args: Sequence[int], stream: int = 0,
               shared_bytes: int = 0) -> None:
        """``args`` are 64-bit values (addresses or integers), one per kernel parameter."""
        values = [ctypes.c_uint64(int(a) & (2 ** 64 - 1)) for a in args]
        pointers = (ctypes.c_void_p * len(values))(*[ctypes.cast(ctypes.pointer(v), ctypes.c_void_p)
                                                     for v in values])
        self._check(self._cuda.cuLaunchKernel(self._function, grid, 1, 1, threads, 1, 1, shared_bytes,
                                              ctypes.c_void_p(stream), pointers, None), "cuLaunchKernel")


# ---- artifact forms of a bound transport program -------------------------------------------------

@dataclass(frozen=True)
class FragmentArtifact:
    """Device code of one transport program, ready to be included into a client kernel.

    ``source`` declares ``__device__ void <symbol>(<slots...>, unsigned long long *ab_status)``;
    ``call`` renders the invocation for given slot expressions.  ``facts`` are the pipeline's
    facts for this transport (batches, fences, flag writes)."""

    name: str
    symbol: str
    artifact: str
    source: str
    parameters: tuple[tuple[str, str], ...]
    facts: dict
    key: str

    def call(self, status: str = "nullptr", **slots: str) -> str:
        missing = [n for n, _ in self.parameters if n not in slots]
        if missing:
            raise ValueError(f"fragment {self.name!r}: missing slots {missing}")
        return f"{self.symbol}({', '.join(slots[n] for n, _ in self.parameters)}, {status});"


@dataclass(frozen=True)
class StandaloneKernel:
    """A transport program compiled to its own cubin."""

    name: str
    artifact: Artifact
    parameters: tuple[tuple[str, str], ...]
    facts: dict

    def load(self) -> LoadedKernel:
        return LoadedKernel(self.artifact)


def _parameters(cuda: str, name: str) -> tuple[tuple[str, str], ...]:
    header = re.search(r"__global__ void " + re.escape(name) + r"\(([^)]*)\)", cuda)
    if header is None:
        raise RuntimeError(f"emitted source has no kernel named {name}")
    out = []
    for item in header.group(1).split(","):
        item = item.strip()
        if not item or item.endswith("ab_status"):
            continue
        ctype, _, ident = item.rpartition(" ")
        out.append((ident.lstrip("*"), ctype + ("*" if ident.startswith("*") else "")))
    return tuple(out)


def compile_fragment_artifact(binding, *, reuse: int = 1, threads: int = 32,
                              options=None) -> FragmentArtifact:
    """Specialise a :class:`TransportProgramBinding` for the current compilation and return it as
    device code: the emitted kernel body with a ``__device__`` signature instead of an entry point."""
    from .driver import compile_program

    compiled = compile_program(binding.to_builder(reuse=reuse, threads=threads), options)
    if compiled.cuda is None:
        raise ValueError("the pipeline was stopped before the lowering; nothing to bind")
    symbol = compiled.name + "_fragment"
    source = compiled.cuda.replace(f'extern "C" __global__ void {compiled.name}(',
                                   f"__device__ __forceinline__ void {symbol}(", 1)
    if source == compiled.cuda:
        raise RuntimeError("emitted source has no entry point to rebind")
    return FragmentArtifact(binding.name, symbol, binding.artifact, source,
                            _parameters(compiled.cuda, compiled.name), compiled.facts, compiled.key)


def realize_bindable_epilogue(binding, **kwargs) -> FragmentArtifact:
    """The fragment of a binding declared ``bindable_epilogue``: the client calls it as the last
    statement of its kernel, after a CTA barrier if several threads produced the source."""
    if binding.artifact != "bindable_epilogue":
        raise ValueError(f"binding {binding.name!r} is declared {binding.artifact!r}, not bindable_epilogue")
    if binding.reductions:
        raise ValueError("a bindable epilogue cannot carry reductions: they belong to the consumer kernel")
    return compile_fragment_artifact(binding, **kwargs)


def realize_standalone_kernel(binding, *, reuse: int = 1, threads: int = 32, options=None,
                              force: bool = False) -> StandaloneKernel:
    """Compile a binding declared ``standalone_kernel`` to a cubin of its own (nvcc, sm_100a)."""
    from .driver import compile_program

    if binding.artifact != "standalone_kernel":
        raise ValueError(f"binding {binding.name!r} is declared {binding.artifact!r}, not standalone_kernel")
    if binding.reductions:
        raise ValueError("a standalone transport kernel cannot carry reductions")
    compiled = compile_program(binding.to_builder(reuse=reuse, threads=threads), options)
    artifact = build_artifact(compiled, force=force)
    return StandaloneKernel(binding.name, artifact, _parameters(compiled.cuda, compiled.name), compiled.facts)
