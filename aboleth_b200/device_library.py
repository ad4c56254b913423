"""Tier-1 device library as a relocatable package: include directory, manifest, digest.

The reference generates its Tier-1 header and a static archive through the compiler
(python/aboleth/device_library.py:153-223,226-431,501-555).  Here the header is hand-written
(``include/aboleth/device.cuh``), so "generating" the library means publishing a copy under
a digest-keyed cache directory together with ``manifest.json`` (ABI 2, operations, kinds
served, specialisation), guarded by a file lock so that ranks started together publish once.

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

from . import abi
from .compiler.driver import include_dir

OPERATIONS = ("open", "put", "put_warp", "put_block", "put_inline", "signal", "signal_block",
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


def generate_device_library(out: Path, *, transports: Sequence[str] = ("p2p",),
                            specialize: Optional[str] = None, **options) -> DeviceLibrary:
    """Write the include tree and the manifest into ``out``."""
    unknown = [t for t in transports if t not in abi.KIND_BITS]
    if unknown:
        raise ValueError(f"unknown transports {unknown}")
    if specialize is not None and specialize not in SERVED:
        raise ValueError(f"a specialised library pins one of {SERVED}")
    digest = library_identity(transports, specialize, options)
    inc = out / "include"
    if inc.exists():
        shutil.rmtree(inc)
    shutil.copytree(include_dir(), inc)
    header = inc / "aboleth" / "device.cuh"
    if specialize is not None:
        # A specialised library makes other kinds a compile-time error instead of a status.
        guard = ("\n// Specialised build: only '%s' endpoints are served.\n#define ABOLETH_TIER1_SPECIALIZED %d\n"
                 % (specialize, abi.KIND_BITS[specialize]))
        header.write_text(header.read_text().replace("#define ABOLETH_TIER1_ABI 2",
                                                     "#define ABOLETH_TIER1_ABI 2" + guard))
    manifest = out / "manifest.json"
    manifest.write_text(json.dumps({
        "abi": abi.TIER1_ABI, "digest": digest, "arch": "sm_100a", "operations": list(OPERATIONS),
        "requested_transports": sorted(transports),
        "served_directly": [t for t in transports if t in SERVED],
        "served_by_host_proxy": [t for t in transports if t not in SERVED],
        "kind_bits": abi.KIND_BITS, "specialized": specialize, "bounded_waits": True,
        "endpoints_per_peer": options.get("endpoints_per_peer", 1), "header_only": True}, indent=1))
    return DeviceLibrary(inc, header, manifest, digest)


def cached_device_library(*, transports: Sequence[str] = ("p2p",), specialize: Optional[str] = None,
                          **options) -> DeviceLibrary:
    digest = library_identity(transports, specialize, options)
    out = _root() / digest[:16]
    out.mkdir(parents=True, exist_ok=True)
    with open(out / ".lock", "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        manifest = out / "manifest.json"
        if manifest.exists() and json.loads(manifest.read_text()).get("digest") == digest:
            inc = out / "include"
            return DeviceLibrary(inc, inc / "aboleth" / "device.cuh", manifest, digest)
        return generate_device_library(out, transports=transports, specialize=specialize, **options)


def device_library(**kwargs) -> DeviceLibrary:
    return cached_device_library(**kwargs)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="aboleth_b200.device_library")
    ap.add_argument("--transports", default="p2p")
    ap.add_argument("--specialize", default=None)
    ap.add_argument("--out", type=Path, default=None)
    args = ap.parse_args(argv)
    transports = [t for t in args.transports.split(",") if t]
    lib = (generate_device_library(args.out, transports=transports, specialize=args.specialize)
           if args.out else cached_device_library(transports=transports, specialize=args.specialize))
    print(json.dumps({"include_dir": str(lib.include_dir), "header": str(lib.header),
                      "manifest": str(lib.manifest), "digest": lib.digest}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
