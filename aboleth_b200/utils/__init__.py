"""Small host-side helpers: profiler ranges, provenance records and the requirement gate
(``python -m aboleth_b200.utils.gated``)."""
from .provenance import provenance
from .ranges import host_range, ranges_enabled

__all__ = ["host_range", "provenance", "ranges_enabled"]
