"""Small host-side helpers: profiler ranges, provenance records, the requirement gate
(``python -m aboleth_b200.utils.gated``), the SLURM rank launcher (``python -m
aboleth_b200.utils.launch``) and host-side liveness of the ranks (:mod:`.liveness`)."""
from .liveness import Heartbeat, PeerLost
from .provenance import provenance
from .ranges import host_range, ranges_enabled

__all__ = ["Heartbeat", "PeerLost", "host_range", "provenance", "ranges_enabled"]
