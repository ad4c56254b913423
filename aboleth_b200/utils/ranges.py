"""NVTX ranges around host phases (dispatch, experts, combine, fused TP calls).

Off by default: ``ABOLETH_NVTX=1`` turns them on, so that a timeline capture shows which
launches belong to which phase.  The ranges cost a few hundred nanoseconds each and do not
synchronise anything.
"""
from __future__ import annotations

import contextlib
import os
from typing import Iterator


def ranges_enabled() -> bool:
    return os.environ.get("ABOLETH_NVTX", "0") not in ("", "0")


@contextlib.contextmanager
def host_range(name: str) -> Iterator[None]:
    if not ranges_enabled():
        yield
        return
    import torch

    torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        torch.cuda.nvtx.range_pop()
