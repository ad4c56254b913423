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
