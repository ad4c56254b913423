"""Tier-1 device library as a relocatable package: include directory, manifest, digest.

The reference generates its Tier-1 header and a static archive through the compiler
(python/aboleth/device_library.py:153-223,226-431,501-555).  Here the header is hand-written
(``include/aboleth/device.cuh``), so "generating" the library means publishing a copy under
a digest-keyed cache directory together with ``manifest.json`` (ABI 2, operations, kinds
served, specialisation), guarded by a file lock so that ranks started together publish once.
With ``archive=True`` the package also holds ``lib/libaboleth_tier1.a``: relocatable device
code with one ``aboleth_tier1_<op>_<transport>`` symbol per operation and transport (nvcc
``-rdc=true -dc`` and ``ar qcs``), for clients that link instead of including.

    python -m aboleth_b200.device_library --transports p2p,proxy [--specialize p2p] [--out DIR]
"""
from __future__ import annotations

import argparse
import fcntl
import hashlib
import json
import os
import shutil
import sys
from dataclasses import dataclass
from pathlib import Path
from typing import Optional, Sequence

import subprocess

from . import abi
from .compiler.driver import include_dir

OPERATIONS = ("open", "put", "put_warp", "put_block", "put_inline", "put_inline_small", "signal", "signal_block",
              "put_signal", "put_many", "put_many_signal", "put_many_flush", "quiet", "wait_signal",
              "wait_signal_status")
SERVED = ("p2p", "proxy")


@dataclass(frozen=True)
class DeviceLibrary:
    include_dir: Path
    header: Path
    manifest: Path
    digest: str
    archive: Optional[Path] = None      # header-only: there is no archive to link
    bitcode: Optional[Path] = None

    def nvcc_flags(self, arch: str = "sm_100a") -> list[str]:
        return ["-gencode", f"arch=compute_{arch[3:]},code={arch}", f"-I{self.include_dir}", "-std=c++17"]


def library_identity(transports: Sequence[str], specialize: Optional[str], options: dict) -> str:
    h = hashlib.sha256()
    for path in sorted(include_dir().rglob("*")):
        if path.is_file():
            h.update(path.name.encode())
            h.update(path.read_bytes())
    h.update(json.dumps({"transports": sorted(transports), "specialize": specialize,
                         "options": options}, sort_keys=True).encode())
    return h.hexdigest()


def _root() -> Path:
    base = os.environ.get("ABOLETH_CACHE_DIR") or os.path.join(
        os.environ.get("XDG_CACHE_HOME", os.path.expanduser("~/.cache")), "aboleth_b200")
    return Path(base) / "device-library"


# Linkable form: one `extern "C" __device__` symbol per operation and transport, all-scalar
# arguments, the Status as a 64-bit return value (the reference's exported Tier-1 symbols,
# python/aboleth/tier1.py:70-77, emit/tier1_header.py:35-92).  A symbol checks that the
# endpoint it is given is of its transport and reports Malformed otherwise.
SYMBOL_OPS = {
    "put": ("unsigned long long dst, unsigned dst_key, unsigned long long src, unsigned src_key, unsigned bytes",
            "aboleth::put(ctx, ref, aboleth::RemoteRegion{dst, dst_key}, aboleth::LocalRegion{src, src_key}, bytes);"),
    "put_inline": ("unsigned long long dst, unsigned dst_key, unsigned long long value",
                   "aboleth::put_inline(ctx, ref, aboleth::RemoteRegion{dst, dst_key}, value);"),
    "signal": ("unsigned long long flag, unsigned flag_key, unsigned long long value",
               "aboleth::signal(ctx, ref, aboleth::RemoteRegion{flag, flag_key}, value);"),
    "put_signal": ("unsigned long long dst, unsigned dst_key, unsigned long long src, unsigned src_key, "
                   "unsigned bytes, unsigned long long flag, unsigned flag_key, unsigned long long value",
                   "aboleth::put_signal(ctx, ref, aboleth::RemoteRegion{dst, dst_key}, "
                   "aboleth::LocalRegion{src, src_key}, bytes, aboleth::RemoteRegion{flag, flag_key}, value);"),
    "put_many": ("unsigned long long descs, unsigned count",
                 "aboleth::put_many(ctx, ref, reinterpret_cast<const aboleth::PutDesc *>(descs), count);"),
    "put_many_signal": ("unsigned long long descs, unsigned count, unsigned long long flag, unsigned flag_key, "
                        "unsigned long long value",
                        "aboleth::put_many_signal(ctx, ref, reinterpret_cast<const aboleth::PutDesc *>(descs), "
                        "count, aboleth::RemoteRegion{flag, flag_key}, value);"),
    "put_many_flush": ("unsigned long long descs, unsigned count",
                       "aboleth::put_many_flush(ctx, ref, reinterpret_cast<const aboleth::PutDesc *>(descs), count);"),
    "quiet": ("", "aboleth::quiet(ctx, ref);"),
}


def symbol_names(transports: Sequence[str]) -> list[str]:
    names = [f"aboleth_tier1_{op}_{t}" for t in transports for op in SYMBOL_OPS]
    return names + ["aboleth_tier1_wait_signal"]


def _symbols_source(transports: Sequence[str]) -> str:
    lines = ['// Linkable Tier-1 symbols (device code, relocatable).  Link with -rdc=true.',
             '#include "aboleth/device.cuh"', ""]
    for t in transports:
        kind = abi.KIND_BITS[t if t in SERVED else "proxy"]
        for op, (params, body) in SYMBOL_OPS.items():
            args = "unsigned long long endpoints, unsigned peer" + (", " + params if params else "")
            lines += [f'extern "C" __device__ unsigned long long aboleth_tier1_{op}_{t}({args}) {{',
                      "    unsigned long long status = 0;",
                      "    const aboleth::DeviceContext ctx{reinterpret_cast<const std::uint64_t *>(endpoints), "
                      "nullptr, &status};",
                      "    const aboleth::PeerRef ref = aboleth::open(ctx, static_cast<int>(peer));",
                      f"    if (ref.kind != {kind}u)",
                      "        return static_cast<unsigned long long>(aboleth::Status::Malformed);",
                      f"    {body}", "    return status;", "}", ""]
    lines += ['extern "C" __device__ unsigned long long aboleth_tier1_wait_signal(unsigned long long flag, '
              'unsigned long long value, unsigned long long timeout_ns) {',
              "    return static_cast<unsigned long long>(aboleth::wait_signal_status("
              "reinterpret_cast<const std::uint64_t *>(flag), value, timeout_ns));", "}", ""]
    return "\n".join(lines)


def _build_archive(out: Path, inc: Path, transports: Sequence[str], arch: str = "sm_100a") -> Path:
    """nvcc -rdc=true -dc the symbol file, then `ar qcs`: a static archive of relocatable device code."""
    lib = out / "lib"
    lib.mkdir(exist_ok=True)
    source = lib / "tier1_symbols.cu"
    source.write_text(_symbols_source(transports))
    obj, archive = lib / "tier1_symbols.o", lib / "libaboleth_tier1.a"
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    steps = [[nvcc, "-gencode", f"arch=compute_{arch[3:]},code={arch}", "-std=c++17", "-O3", "-rdc=true", "-dc",
              f"-I{inc}", str(source), "-o", str(obj)],
             ["ar", "qcs", str(archive), str(obj)]]
    if archive.exists():
        archive.unlink()
    for cmd in steps:
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode != 0:
            raise RuntimeError("building the Tier-1 archive failed:\n" + " ".join(cmd) + "\n" + proc.stderr)
    return archive


def generate_device_library(out: Path, *, transports: Sequence[str] = ("p2p",),
                            specialize: Optional[str] = None, archive: bool = False,
                            **options) -> DeviceLibrary:
    """Write the include tree and the manifest (and, with ``archive=True``, the static archive of
    linkable symbols) into ``out``."""
    unknown = [t for t in transports if t not in abi.KIND_BITS]
    if unknown:
        raise ValueError(f"unknown transports {unknown}")
    if specialize is not None and specialize not in SERVED:
        raise ValueError(f"a specialised library pins one of {SERVED}")
    digest = library_identity(transports, specialize, {**options, "archive": archive})
    inc = out / "include"
    if inc.exists():
        shutil.rmtree(inc)
    shutil.copytree(include_dir(), inc)
    header = inc / "aboleth" / "device.cuh"
    # The published header carries its options: it is marked as generated, and a specialised one
    # pins its transport (the per-call kind test disappears; the other kind does not compile).
    baked = "#define ABOLETH_TIER1_GENERATED 1\n"
    if specialize is not None:
        baked += ("// Specialised build: only '%s' endpoints are served.\n#define ABOLETH_TIER1_SPECIALIZED %d\n"
                  % (specialize, abi.KIND_BITS[specialize]))
    header.write_text(header.read_text().replace("#define ABOLETH_TIER1_ABI 2",
                                                 baked + "#define ABOLETH_TIER1_ABI 2", 1))
    if specialize is not None:
        transports = [t for t in transports if (t if t in SERVED else "proxy") == specialize]
        if not transports:
            raise ValueError(f"none of the requested transports is served by a library specialised for {specialize}")
    lanes = int(options.get("endpoints_per_peer", 1))
    if lanes != 1:
        header.write_text(header.read_text().replace(
            "#ifndef ABOLETH_TIER1_ENDPOINTS_PER_PEER",
            f"#define ABOLETH_TIER1_ENDPOINTS_PER_PEER {lanes}\n#ifndef ABOLETH_TIER1_ENDPOINTS_PER_PEER", 1))
    built = _build_archive(out, inc, list(transports)) if archive else None
    manifest = out / "manifest.json"
    manifest.write_text(json.dumps({
        "archive": str(built.relative_to(out)) if built else None,
        "symbols": symbol_names(list(transports)) if built else [],
        "abi": abi.TIER1_ABI, "digest": digest, "arch": "sm_100a", "operations": list(OPERATIONS),
        "requested_transports": sorted(transports),
        "served_directly": [t for t in transports if t in SERVED],
        "served_by_host_proxy": [t for t in transports if t not in SERVED],
        "kind_bits": abi.KIND_BITS, "specialized": specialize, "bounded_waits": True,
        "endpoints_per_peer": options.get("endpoints_per_peer", 1), "header_only": built is None}, indent=1))
    return DeviceLibrary(inc, header, manifest, digest, archive=built)


def cached_device_library(*, transports: Sequence[str] = ("p2p",), specialize: Optional[str] = None,
                          archive: bool = False, **options) -> DeviceLibrary:
    digest = library_identity(transports, specialize, {**options, "archive": archive})
    out = _root() / digest[:16]
    out.mkdir(parents=True, exist_ok=True)
    with open(out / ".lock", "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        manifest = out / "manifest.json"
        if manifest.exists() and json.loads(manifest.read_text()).get("digest") == digest:
            inc = out / "include"
            built = json.loads(manifest.read_text()).get("archive")
            return DeviceLibrary(inc, inc / "aboleth" / "device.cuh", manifest, digest,
                                 archive=out / built if built else None)
        return generate_device_library(out, transports=transports, specialize=specialize, archive=archive,
                                       **options)


def device_library(**kwargs) -> DeviceLibrary:
    return cached_device_library(**kwargs)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="aboleth_b200.device_library")
    ap.add_argument("--transports", default="p2p")
    ap.add_argument("--specialize", default=None)
    ap.add_argument("--archive", action="store_true", help="also build the static archive of linkable symbols")
    ap.add_argument("--out", type=Path, default=None)
    args = ap.parse_args(argv)
    transports = [t for t in args.transports.split(",") if t]
    lib = (generate_device_library(args.out, transports=transports, specialize=args.specialize,
                                   archive=args.archive)
           if args.out else cached_device_library(transports=transports, specialize=args.specialize,
                                                  archive=args.archive))
    print(json.dumps({"include_dir": str(lib.include_dir), "header": str(lib.header),
                      "manifest": str(lib.manifest), "digest": lib.digest,
                      "archive": str(lib.archive) if lib.archive else None}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
