"""Builds and loads the native libraries that sit beside this file.

Three shared objects are produced in ``aboleth_b200/_lib``:

``libab200_kernels.so``
    every hand-written sm_100a kernel (``csrc/kernels/*.cu``), compiled by nvcc
    with ``-gencode arch=compute_100a,code=sm_100a``;
``libab200_runtime.so``
    the host runtime (``csrc/host``): key table, CUDA IPC, host-proxy thread;
``libab200_spec.so``
    the Tier-2 specializer core (``csrc/spec``): plain C++17, no CUDA.

The objects are loaded with :mod:`ctypes`; every entry point is ``extern "C"``.
A library whose sources changed is rebuilt; one that cannot be built or loaded
raises instead of falling back to anything else.
"""
from __future__ import annotations

import ctypes
import hashlib
import os
import shutil
import subprocess
import sys
import threading
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

_ROOT = Path(__file__).resolve().parent
_LIB = _ROOT / "_lib"
_INCLUDE = _ROOT / "include"
_CSRC = _ROOT / "csrc"
_ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
_LOCK = threading.Lock()
_LOADED: dict[str, ctypes.CDLL] = {}


def _nvcc() -> str:
    path = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(path).exists():
        raise RuntimeError("nvcc was not found; the sm_100a kernels cannot be built")
    return path


def _digest(paths: list[Path], flags: list[str]) -> str:
    h = hashlib.sha256()
    for flag in flags:
        # Paths under the package are hashed relative to it: a copy of the tree at
        # another location must not look like a source change.
        h.update(flag.replace(str(_ROOT), "<pkg>").encode())
    headers = sorted(_INCLUDE.rglob("*.h")) + sorted(_INCLUDE.rglob("*.cuh")) + sorted(
        _CSRC.rglob("*.cuh")) + sorted(_CSRC.rglob("*.h")) + sorted(_CSRC.rglob("*.hpp"))
    for path in list(paths) + headers:
        h.update(path.name.encode())
        h.update(path.read_bytes())
    return h.hexdigest()


def _run(cmd: list[str]) -> str:
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError("native build failed:\n  " + " ".join(cmd) + "\n" + proc.stdout + proc.stderr)
    return proc.stdout + proc.stderr


def _targets() -> dict[str, dict]:
    kernels = sorted((_CSRC / "kernels").glob("*.cu"))
    host = sorted((_CSRC / "host").glob("*.cu")) + sorted((_CSRC / "host").glob("*.cpp"))
    spec = sorted((_CSRC / "spec").glob("*.cpp"))
    common = ["-O3", "-std=c++17", f"-I{_INCLUDE}", "-Xcompiler", "-fPIC"]
    # Extra preprocessor definitions for the kernels, e.g. ABOLETH_KERNEL_DEFINES=AB_GEMM_TRACE.
    defines = [f"-D{d}" for d in os.environ.get("ABOLETH_KERNEL_DEFINES", "").split(",") if d]
    return {
        "kernels": {
            "sources": kernels,
            "compile": [_nvcc(), *_ARCH, "-lineinfo", *common, *defines, f"-I{_CSRC / 'kernels'}",
                        "-Xptxas", "-v", "-c"],
            "link": [_nvcc(), *_ARCH, "-shared", "-Xcompiler", "-fPIC"],
        },
        "runtime": {
            "sources": host,
            "compile": [_nvcc(), *_ARCH, *common, "-c"],
            "link": [_nvcc(), *_ARCH, "-shared", "-Xcompiler", "-fPIC", "-lpthread", "-ldl"],
        },
        "spec": {
            "sources": spec,
            "compile": ["g++", "-O2", "-std=c++17", "-fPIC", "-Wall", f"-I{_INCLUDE}",
                        f"-I{_CSRC / 'spec'}", "-c"],
            "link": ["g++", "-shared", "-fPIC"],
        },
    }


def library_path(name: str) -> Path:
    return _LIB / f"libab200_{name}.so"


def build(name: str, *, force: bool = False, verbose: bool = False) -> Path:
    """Build one library if its sources changed.  Returns the ``.so`` path."""
    target = _targets()[name]
    sources: list[Path] = target["sources"]
    out = library_path(name)
    if not sources:
        raise RuntimeError(f"no sources for native library {name!r}")
    _LIB.mkdir(exist_ok=True)
    stamp = _LIB / f"{name}.sha256"
    digest = _digest(sources, target["compile"] + target["link"])
    if not force and out.exists() and stamp.exists() and stamp.read_text() == digest:
        return out
    import fcntl
    with open(_LIB / f"{name}.lock", "w") as lock:
        # Ranks started together build once: the others wait here and then see the stamp.
        fcntl.flock(lock, fcntl.LOCK_EX)
        if not force and out.exists() and stamp.exists() and stamp.read_text() == digest:
            return out
        return _build_locked(name, target, sources, out, stamp, digest, verbose)


def _build_locked(name, target, sources, out, stamp, digest, verbose) -> Path:
    objdir = _LIB / f"obj_{name}"
    objdir.mkdir(exist_ok=True)
    logs: list[str] = []

    def compile_one(src: Path) -> Path:
        obj = objdir / (src.stem + ".o")
        logs.append(_run(target["compile"] + [str(src), "-o", str(obj)]))
        return obj

    with ThreadPoolExecutor(max_workers=min(8, len(sources))) as pool:
        objects = list(pool.map(compile_one, sources))
    tmp = out.with_suffix(".so.tmp")
    _run(target["link"] + [str(o) for o in objects] + ["-o", str(tmp)])
    os.replace(tmp, out)
    stamp.write_text(digest)
    (_LIB / f"{name}.buildlog.txt").write_text("\n".join(logs))
    if verbose:
        print("\n".join(logs), file=sys.stderr)
    return out


def build_all(*, force: bool = False, verbose: bool = False) -> dict[str, Path]:
    return {name: build(name, force=force, verbose=verbose)
            for name, target in _targets().items() if target["sources"]}


def load(name: str) -> ctypes.CDLL:
    """Load (building first if needed) one native library."""
    with _LOCK:
        lib = _LOADED.get(name)
        if lib is not None:
            return lib
        path = library_path(name)
        if os.environ.get("ABOLETH_B200_NO_BUILD") != "1" or not path.exists():
            path = build(name)
        lib = ctypes.CDLL(str(path))
        _LOADED[name] = lib
        return lib


if __name__ == "__main__":
    for lib_name, lib_path in build_all(force="--force" in sys.argv, verbose="-v" in sys.argv).items():
        print(lib_name, lib_path)
