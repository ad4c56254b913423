"""ctypes view of ``libab200_kernels.so`` (every hand-written sm_100a kernel).

There is no PyTorch fallback behind these wrappers: if the library cannot be
built or loaded, or a launch fails, the call raises.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from .. import _native

_c = ctypes
_VP, _I, _U64, _F = _c.c_void_p, _c.c_int, _c.c_uint64, _c.c_float

_SIGNATURES = {
    "ab_alltoall": [_VP, _VP, _VP, _VP, _VP, _U64, _U64, _U64] + [_I] * 10 + [_VP],
    "ab_fill_payload": [_VP, _U64, _U64, _c.c_uint, _c.c_uint, _VP],
    "ab_check_payload": [_VP, _U64, _U64, _c.c_uint, _c.c_uint, _VP, _VP],
    "ab_pingpong": [_VP, _U64, _U64, _VP, _VP, _VP, _U64, _U64, _I, _I, _I, _I, _I, _VP],
    "ab_tier1_exercise": [_VP, _VP] + [_U64] * 8 + [_c.c_uint32, _I, _I, _VP],
    "ab_ep_dispatch": [_VP, _F, _VP, _I, _VP],
    "ab_ep_combine": [_VP, _F, _VP, _I, _VP],
    "ab_quant_fp8": [_VP, _VP, _VP, _I, _I, _I, _F, _I, _VP],
    "ab_router_topk": [_VP, _VP, _VP, _I, _I, _I, _I, _VP],
    "ab_expert_offsets": [_VP, _VP, _VP, _I, _I, _I, _VP],
    "ab_permute": [_VP] * 9 + [_I] * 7 + [_VP],
    "ab_unpermute": [_VP] * 7 + [_I] * 5 + [_VP],
    "ab_standin_expert": [_VP, _VP, _I] + [_VP] * 6 + [_I] * 7 + [_VP],
}

_launches = 0


def lib() -> ctypes.CDLL:
    handle = _native.load("kernels")
    if not getattr(handle, "_ab_typed", False):
        for name, argtypes in _SIGNATURES.items():
            fn = getattr(handle, name, None)
            if fn is not None:
                fn.argtypes = argtypes
                fn.restype = _I
        handle._ab_typed = True
    return handle


def declare(name: str, argtypes: list) -> None:
    """Register the signature of a kernel entry point defined elsewhere."""
    _SIGNATURES[name] = argtypes
    handle = _native._LOADED.get("kernels")
    if handle is not None and hasattr(handle, name):
        fn = getattr(handle, name)
        fn.argtypes = argtypes
        fn.restype = _I


def stream_ptr(stream: Optional[torch.cuda.Stream] = None) -> int:
    return (stream or torch.cuda.current_stream()).cuda_stream


def ptr(tensor: Optional[torch.Tensor]) -> int:
    return 0 if tensor is None else tensor.data_ptr()


def call(name: str, *args) -> None:
    """Launch ``name``; raise if the launcher reports an error."""
    global _launches
    rc = getattr(lib(), name)(*args)
    if rc != 0:
        raise RuntimeError(f"{name} failed with code {rc} (bad arguments or CUDA launch error)")
    _launches += 1


def launch_count() -> int:
    """How many kernels of this library were launched by this process."""
    return _launches
