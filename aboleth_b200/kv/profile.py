"""Target profiles of KV-cache page migration: SM copy vs copy engine, workers, readiness grouping.

Reference: python/aboleth/kv/profile.py:112-131 and docs/KV_CACHE.md:79-85 (``h200-nvlink``:
64 MiB copy-engine threshold, 16 workers, 256 elements, 4 consumers per readiness event;
``generic-generated-p2p``: never the copy engine, per-consumer readiness).  ``b200-nvlink`` is
this build's default: SM copies with 16-byte vectors saturate an NVLink 5 direction well
below the copy-engine threshold.
"""
from __future__ import annotations

from dataclasses import dataclass, replace
from typing import Optional


@dataclass(frozen=True)
class KVTargetProfile:
    name: str
    copy_engine_threshold: Optional[int]   # bytes per run at which cudaMemcpyAsync takes over; None = never
    copy_workers: int
    block_elements: int
    consumers_per_readiness: int
    threads: int = 256


GENERIC_KV_TARGET_PROFILE = KVTargetProfile("generic-generated-p2p", None, 16, 256, 1)
H200_NVLINK_KV_TARGET_PROFILE = KVTargetProfile("h200-nvlink", 64 << 20, 16, 256, 4)
B200_NVLINK_KV_TARGET_PROFILE = KVTargetProfile("b200-nvlink", 256 << 20, 32, 512, 4, threads=512)

_PROFILES = {p.name: p for p in (GENERIC_KV_TARGET_PROFILE, H200_NVLINK_KV_TARGET_PROFILE,
                                 B200_NVLINK_KV_TARGET_PROFILE)}


@dataclass(frozen=True)
class KVRuntimeOverrides:
    copy_workers: Optional[int] = None
    copy_engine_threshold: Optional[int] = None
    consumers_per_readiness: Optional[int] = None

    @classmethod
    def from_mapping(cls, values) -> "KVRuntimeOverrides":
        """From an engine's free-form connector options (``aboleth_kv_<field>`` or ``<field>``); absent
        keys stay unset, present ones must be positive integers."""
        chosen = {}
        for name in ("copy_workers", "copy_engine_threshold", "consumers_per_readiness"):
            raw = values.get(f"aboleth_kv_{name}", values.get(name))
            if raw is None:
                continue
            number = int(raw)
            if number < 1:
                raise ValueError(f"KV runtime override {name}={raw!r} must be a positive integer")
            chosen[name] = number
        return cls(**chosen)


def select_kv_target_profile(device_name: str = "", *, overrides: Optional[KVRuntimeOverrides] = None,
                             name: Optional[str] = None) -> KVTargetProfile:
    if name is not None:
        profile = _PROFILES[name]
    elif "B200" in device_name:
        profile = B200_NVLINK_KV_TARGET_PROFILE
    elif "H200" in device_name:
        profile = H200_NVLINK_KV_TARGET_PROFILE
    else:
        profile = GENERIC_KV_TARGET_PROFILE
    if overrides is not None:
        changes = {k: v for k, v in vars(overrides).items() if v is not None}
        profile = replace(profile, **changes)
    return profile
