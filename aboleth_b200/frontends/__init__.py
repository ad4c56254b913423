"""Bindings of the Tier-1 device library for other kernel languages.

The reference binds its exported Tier-1 symbols into Triton (``extern_libs``) and the CuTe DSL
(``cute.extern``), python/aboleth/frontends/triton/tier1.py and frontends/cute.py.  Neither language
is a code path of this build, so what is offered is the language-neutral half of those modules: the
typed table of exported symbols, a header of plain C prototypes, and the link line - everything a
kernel language that can call an ``extern "C" __device__`` function needs.
"""
from .extern import ExternSymbol, extern_symbols, link_flags, prototypes_header, write_prototypes

__all__ = ["ExternSymbol", "extern_symbols", "link_flags", "prototypes_header", "write_prototypes"]
