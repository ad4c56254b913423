"""Switches and per-compilation settings of the Tier-2 specializer.

The switch names, their defaults and the ``ABOLETH_PASSES`` grammar
(``default``, ``all``, ``none`` or a comma list of ``+name`` / ``-name``) are the
reference's (python/aboleth/compiler.py:79-134; docs/COMPILER_SEMANTICS.md:39-55),
so an ablation script written for it drives this specializer unchanged.
``compilation(...)`` sets the remaining knobs for the calls made inside the
``with`` block through context variables (python/aboleth/compiler.py:474-582).
"""
from __future__ import annotations

import contextlib
import contextvars
import os
from dataclasses import dataclass, field, replace
from typing import Iterator, Optional

DEFAULT_INLINE_BYTES = 28

OPTIMIZATIONS = {
    "shape-specialization": True,
    "endpoint-fanout": True,
    "coalesce-receives": True,
    "valid-extents": True,
    "plan-storage": True,
    "dead-communication": True,
    "completion-planning": True,
    "forward-inline-payloads": True,
    "plan-publication": True,
    "coalesce-submissions": True,
    "order-publications": True,
    "elide-epochs": True,
    "defer-announcement": False,
    "analyze-issuers": True,
    "share-producer-fence": True,
    "ionic-fenced-publication": True,
    "gpu-doorbell": True,
    "invariant-descriptors": True,
    "vector-wqe-stores": False,
    "self-reclaim": True,
}

# Pipeline order, used by ablation sweeps (waterfall adds passes in this order).
PIPELINE_ORDER = (
    "valid-extents", "completion-planning", "forward-inline-payloads", "plan-publication",
    "coalesce-submissions", "order-publications", "elide-epochs", "defer-announcement",
    "analyze-issuers",
)


def enabled_optimizations(spec: Optional[str] = None) -> frozenset[str]:
    """Resolve ``ABOLETH_PASSES`` (or ``spec``) over the defaults."""
    text = os.environ.get("ABOLETH_PASSES", "") if spec is None else spec
    enabled = {name for name, on in OPTIMIZATIONS.items() if on}
    for token in text.split(","):
        token = token.strip()
        if not token or token == "default":
            continue
        if token == "all":
            enabled = set(OPTIMIZATIONS)
            continue
        if token == "none":
            enabled = set()
            continue
        name = token[1:]
        if token[0] not in "+-" or name not in OPTIMIZATIONS:
            raise ValueError(f"ABOLETH_PASSES: {token!r} is not +name or -name for a name in "
                             f"{sorted(OPTIMIZATIONS)}")
        (enabled.add if token[0] == "+" else enabled.discard)(name)
    return frozenset(enabled)


@dataclass(frozen=True)
class CompileOptions:
    """Everything that changes emitted code; hashed into the artefact key."""

    backend: str = "p2p"
    rank: int = 0
    world_size: int = 1
    queue_capacity: int = 0
    completion_interval: int = 0
    strict_registrations: bool = False
    gpu_resident_queues: bool = False
    inline_bytes: int = DEFAULT_INLINE_BYTES
    p2p_copy: str = "cooperative"          # or "scalar" (ABOLETH_P2P_SCALAR)
    coop_min: int = 256                    # ABOLETH_P2P_COOP_MIN
    coop_elements: int = 2048              # ABOLETH_P2P_COOP_ELEMENTS, 32..4096
    endpoint_profile: str = ""
    plan_hash: str = ""
    arch: str = "sm_100a"
    passes: frozenset = field(default_factory=enabled_optimizations)
    stop_after: str = ""

    def to_native(self) -> str:
        parts = [f"backend={self.backend}", f"enable={','.join(sorted(self.passes))}",
                 f"inline_bytes={self.inline_bytes}", f"queue_capacity={self.queue_capacity}",
                 f"completion_interval={self.completion_interval}",
                 f"strict_registrations={int(self.strict_registrations)}",
                 f"coop_min={self.coop_min}", f"coop_elements={self.coop_elements}",
                 f"p2p_scalar={int(self.p2p_copy == 'scalar')}"]
        if self.stop_after:
            parts.append(f"stop_after={self.stop_after}")
        return " ".join(parts)


def _from_environment() -> CompileOptions:
    env = os.environ
    opts = CompileOptions(passes=enabled_optimizations())
    if env.get("ABOLETH_P2P_SCALAR") == "1":
        opts = replace(opts, p2p_copy="scalar")
    if env.get("ABOLETH_P2P_COOP_MIN"):
        opts = replace(opts, coop_min=int(env["ABOLETH_P2P_COOP_MIN"]))
    if env.get("ABOLETH_P2P_COOP_ELEMENTS"):
        opts = replace(opts, coop_elements=int(env["ABOLETH_P2P_COOP_ELEMENTS"]))
    if env.get("ABOLETH_RDMA_INLINE_BYTES"):
        opts = replace(opts, inline_bytes=int(env["ABOLETH_RDMA_INLINE_BYTES"]))
    return opts


_CURRENT: contextvars.ContextVar[Optional[CompileOptions]] = contextvars.ContextVar(
    "aboleth_b200_compile_options", default=None)


def current_options() -> CompileOptions:
    """Options of the innermost ``compilation`` block; environment defaults outside one."""
    return _CURRENT.get() or _from_environment()


@contextlib.contextmanager
def compilation(backend: str = "p2p", **settings) -> Iterator[CompileOptions]:
    """Fix the specializer options for everything compiled inside the block.

    Precedence: explicit keyword > environment variable > default.
    """
    if backend not in ("p2p", "proxy", "rdma", "efa", "ionic"):
        raise ValueError(f"unknown transport {backend!r}")
    passes = settings.pop("passes", None)
    opts = replace(_from_environment(), backend=backend, **settings)
    if passes is not None:
        opts = replace(opts, passes=enabled_optimizations(passes) if isinstance(passes, str)
                       else frozenset(passes))
    token = _CURRENT.set(opts)
    try:
        yield opts
    finally:
        _CURRENT.reset(token)
