"""Small host-side helpers: profiler ranges and provenance records."""
from .provenance import provenance
from .ranges import host_range, ranges_enabled

__all__ = ["host_range", "provenance", "ranges_enabled"]
