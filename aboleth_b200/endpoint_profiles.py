"""Measured endpoint profiles: how many bytes one endpoint (lane) should carry, how many
lanes help, and how many sender warps per lane, per (backend, platform, queue memory, link).

Seed entries, the fit rule and the store layout follow the reference
(python/aboleth/endpoint_profiles.py:57-87,198,229-349,380,455-...): a fit picks the fewest
lanes within 95 % of the widest at the largest size where fan-out still pays 15 %; bytes per
endpoint is the smallest size where that width pays 15 % over one lane, divided by the width;
a held-out size must keep the planned lanes at 90 % of one lane.

    python -m aboleth_b200.endpoint_profiles list|show NAME|pin NAME|retire NAME
"""
from __future__ import annotations

import argparse
import json
import os
import sys
from dataclasses import asdict, dataclass
from pathlib import Path
from typing import Mapping, Optional, Sequence

GAIN, NEAR, HOLDOUT = 1.15, 0.95, 0.90
PROBE_PROTOCOL = 2


@dataclass(frozen=True)
class EndpointProfile:
    identity: str
    backend: str
    platform: str
    queue_memory: str
    peer_link: str
    bytes_per_endpoint: int
    max_lanes: int
    sender_warps: int = 1
    source: str = "seed"

    def to_request(self) -> str:
        return (f"backend={self.backend} platform={self.platform} queueMemory={self.queue_memory} "
                f"peerLink={self.peer_link} bytesPerEndpoint={self.bytes_per_endpoint} "
                f"maxLanes={self.max_lanes} senderWarps={self.sender_warps} identity={self.identity}")


SEED_PROFILES = {
    # 8 x B200 over NVLink 5 (18 links): 256 KiB per endpoint, up to 16 lanes, 8 sender warps.
    "B200_NV18": EndpointProfile("seed:B200_NV18", "p2p", "B200", "none", "NV18", 262144, 16, 8),
    # B200 + NDR400 with host queues: 256 KiB per endpoint, 4 lanes.
    "B200_NDR400": EndpointProfile("seed:B200_NDR400", "rdma", "B200", "host", "", 262144, 4, 1),
    # The NIC-less ring of this build: one lane, the host thread is the bottleneck.
    "B200_HOSTRING": EndpointProfile("seed:B200_HOSTRING", "proxy", "B200", "host", "", 1 << 20, 1, 1),
}


@dataclass(frozen=True)
class ProbeSample:
    """Median microseconds per iteration of put + strong signal + sender wait."""

    bytes: int
    lanes: int
    warps: int
    microseconds: float


def fit_profile(samples: Sequence[ProbeSample], *, backend: str, platform: str, queue_memory: str,
                peer_link: str, identity: str) -> Optional[EndpointProfile]:
    """Fit lanes / bytes-per-endpoint / warps from probe samples; None if fan-out never pays."""
    by_size: dict[int, dict[int, float]] = {}
    for s in samples:
        best = by_size.setdefault(s.bytes, {})
        best[s.lanes] = min(best.get(s.lanes, float("inf")), s.microseconds)
    sizes = sorted(by_size)
    if len(sizes) < 2:
        return None
    holdout, fit_sizes = sizes[-1], sizes[:-1]
    chosen_lanes, chosen_size = 1, None
    for size in reversed(fit_sizes):
        lanes_t = by_size[size]
        if 1 not in lanes_t:
            continue
        widest = max(lanes_t)
        if lanes_t[1] / lanes_t[widest] < GAIN:
            continue  # fan-out does not pay 15 % here
        target = lanes_t[widest] / NEAR
        chosen_lanes = min(l for l, t in lanes_t.items() if t <= target)
        chosen_size = size
        break
    if chosen_size is None or chosen_lanes == 1:
        return None
    pays_at = next((size for size in fit_sizes
                    if 1 in by_size[size] and chosen_lanes in by_size[size]
                    and by_size[size][1] / by_size[size][chosen_lanes] >= GAIN), chosen_size)
    held = by_size[holdout]
    if 1 in held and chosen_lanes in held and held[chosen_lanes] > held[1] / HOLDOUT:
        return None  # the held-out size does not confirm the plan
    warp_times: dict[int, float] = {}
    for s in samples:
        if s.lanes == 1 and s.bytes == min(sizes, key=lambda b: abs(b - 65536)):
            warp_times[s.warps] = min(warp_times.get(s.warps, float("inf")), s.microseconds)
    warps = min(warp_times, key=warp_times.get) if warp_times else 1
    return EndpointProfile(identity, backend, platform, queue_memory, peer_link,
                           max(pays_at // chosen_lanes, 4096), chosen_lanes, warps, source="probe")


class ProfileStore:
    """``$XDG_CACHE_HOME/aboleth/endpoint-profiles`` (or ``ABOLETH_PROFILE_DIR``): one JSON per key."""

    def __init__(self, root: Optional[Path] = None):
        base = os.environ.get("ABOLETH_PROFILE_DIR") or os.path.join(
            os.environ.get("XDG_CACHE_HOME", os.path.expanduser("~/.cache")), "aboleth", "endpoint-profiles")
        self.root = Path(root or base)

    def _path(self, key: str) -> Path:
        return self.root / (key.replace("/", "_").replace(":", "_") + ".json")

    @staticmethod
    def key(backend: str, platform: str, queue_memory: str, peer_link: str) -> str:
        return f"{backend}-{platform}-{queue_memory}-{peer_link or 'any'}"

    def load(self, key: str) -> Optional[EndpointProfile]:
        path = self._path(key)
        try:
            record = json.loads(path.read_text())
            if record.get("probe_protocol") != PROBE_PROTOCOL or record.get("retired"):
                return None  # stale or retired entries are never trusted
            return EndpointProfile(**record["profile"])
        except (OSError, ValueError, KeyError, TypeError):
            return None

    def save(self, key: str, profile: EndpointProfile, *, pinned: bool = False) -> None:
        self.root.mkdir(parents=True, exist_ok=True)
        self._path(key).write_text(json.dumps(
            {"probe_protocol": PROBE_PROTOCOL, "pinned": pinned, "profile": asdict(profile)}, indent=1))

    def retire(self, key: str) -> bool:
        path = self._path(key)
        if not path.exists():
            return False
        record = json.loads(path.read_text())
        record["retired"] = True
        path.write_text(json.dumps(record, indent=1))
        return True

    def list(self) -> list[str]:
        return sorted(p.stem for p in self.root.glob("*.json")) if self.root.exists() else []


def resolve_profiles(peer_transports: Mapping[int, object], links: Mapping[int, str],
                     platform: str = "B200", store: Optional[ProfileStore] = None) -> dict[str, EndpointProfile]:
    """One profile per backend in use: a cached probe result if present, else the seed."""
    store = store or ProfileStore()
    out: dict[str, EndpointProfile] = {}
    for peer, transport in peer_transports.items():
        backend = getattr(transport, "value", str(transport))
        backend = backend if backend in ("p2p", "rdma") else "proxy"
        if backend in out:
            continue
        queue = "none" if backend == "p2p" else "host"
        link = links.get(peer, "") if backend == "p2p" else ""
        cached = store.load(store.key(backend, platform, queue, link))
        seed = {"p2p": "B200_NV18", "rdma": "B200_NDR400", "proxy": "B200_HOSTRING"}[backend]
        out[backend] = cached or SEED_PROFILES[seed]
    return out


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="aboleth_b200.endpoint_profiles")
    ap.add_argument("command", choices=["list", "show", "pin", "retire", "seeds"])
    ap.add_argument("name", nargs="?")
    args = ap.parse_args(argv)
    store = ProfileStore()
    if args.command == "seeds":
        print(json.dumps({k: asdict(v) for k, v in SEED_PROFILES.items()}, indent=1))
    elif args.command == "list":
        print("\n".join(store.list()))
    elif args.command == "show":
        profile = store.load(args.name) or SEED_PROFILES.get(args.name)
        print(json.dumps(asdict(profile), indent=1) if profile else "unknown profile")
    elif args.command == "pin":
        if args.name not in SEED_PROFILES:
            print("only seed profiles can be pinned by name", file=sys.stderr)
            return 1
        p = SEED_PROFILES[args.name]
        store.save(store.key(p.backend, p.platform, p.queue_memory, p.peer_link), p, pinned=True)
    elif args.command == "retire":
        return 0 if store.retire(args.name) else 1
    return 0


if __name__ == "__main__":
    sys.exit(main())
