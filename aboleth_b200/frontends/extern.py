"""The exported Tier-1 symbols as data: names, scalar argument types, prototypes, link flags.

Every symbol is ``aboleth_tier1_<operation>_<transport>`` (plus the transport-free
``aboleth_tier1_wait_signal``), takes scalars only - addresses as 64-bit integers, keys, sizes and
peers as 32-bit - and returns the 64-bit status (0 = ok) of the call.  The first two arguments of
every operation are the endpoint-handle table of :meth:`World.exchange_regions` and the peer.
"""
from __future__ import annotations

from dataclasses import dataclass
from pathlib import Path
from typing import Sequence

from .. import abi
from ..device_library import SYMBOL_OPS, DeviceLibrary

_C_TO_SHORT = {"unsigned long long": "u64", "unsigned": "u32"}


@dataclass(frozen=True)
class ExternSymbol:
    """One linkable device function."""
    name: str
    operation: str
    transport: str                      # "" for wait_signal
    arg_names: tuple[str, ...]
    arg_types: tuple[str, ...]          # "u64" | "u32"
    return_type: str = "u64"

    @property
    def prototype(self) -> str:
        back = {v: k for k, v in _C_TO_SHORT.items()}
        args = ", ".join(f"{back[t]} {n}" for t, n in zip(self.arg_types, self.arg_names))
        return f'extern "C" __device__ unsigned long long {self.name}({args});'


def _parse(params: str) -> tuple[tuple[str, ...], tuple[str, ...]]:
    names, types = [], []
    for item in (p.strip() for p in params.split(",") if p.strip()):
        ctype, _, name = item.rpartition(" ")
        names.append(name)
        types.append(_C_TO_SHORT[ctype.strip()])
    return tuple(names), tuple(types)


def extern_symbols(transports: Sequence[str] = ("p2p",)) -> list[ExternSymbol]:
    """The table for ``transports``, in the order the archive defines the symbols."""
    unknown = [t for t in transports if t not in abi.KIND_BITS]
    if unknown:
        raise ValueError(f"unknown transports {unknown}")
    out = []
    for transport in transports:
        for operation, (params, _body) in SYMBOL_OPS.items():
            names, types = _parse("unsigned long long endpoints, unsigned peer" + (", " + params if params else ""))
            out.append(ExternSymbol(f"aboleth_tier1_{operation}_{transport}", operation, transport, names, types))
    out.append(ExternSymbol("aboleth_tier1_wait_signal", "wait_signal", "", ("flag", "value", "timeout_ns"),
                            ("u64", "u64", "u64")))
    return out


def prototypes_header(transports: Sequence[str] = ("p2p",)) -> str:
    """A header of prototypes only: no templates, no inline code, nothing but ``extern "C"``."""
    lines = ["// Prototypes of the linkable Tier-1 symbols (link with -rdc=true against libaboleth_tier1.a).",
             "// Every function returns the call's status: 0 ok, 1 timeout, 2 completion failure, 3 malformed.",
             "#pragma once", ""]
    lines += [symbol.prototype for symbol in extern_symbols(transports)]
    return "\n".join(lines) + "\n"


def write_prototypes(library: DeviceLibrary, transports: Sequence[str]) -> Path:
    """Write ``aboleth_tier1_symbols.h`` beside the library's headers and return its path."""
    path = Path(library.include_dir) / "aboleth" / "aboleth_tier1_symbols.h"
    path.write_text(prototypes_header(transports))
    return path


def link_flags(library: DeviceLibrary) -> list[str]:
    """What a relocatable-device-code link needs to find the symbols."""
    if library.archive is None:
        raise ValueError("this device library was generated header-only: ask for archive=True")
    return ["-rdc=true", f"-I{library.include_dir}", f"-L{Path(library.archive).parent}", "-laboleth_tier1"]
