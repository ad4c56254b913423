"""Host-side liveness of the ranks of a world, checked between steps.

A kernel that waits for a peer gives up after its bounded wait and reports a timeout,
but seconds late and without saying which peer.  The cheaper place to learn that a
rank is gone is the host, before the next launch: every rank bumps a counter in the
bootstrap's key-value store from a small thread, and ``check()`` - called between
steps, with nothing of this rank in flight - raises :class:`PeerLost` naming the ranks
whose counter stopped.  ``leave()`` announces an orderly departure, which peers see at
once.  Nothing here touches a GPU.

The reference has no heartbeat and no rank replacement (its waits are unbounded); this
is an addition of this build.  Works over any store with ``set(key, bytes)`` and
``get(key) -> bytes`` of already-written keys plus ``check([key]) -> bool``, such as
``torch.distributed.TCPStore`` (the store of :class:`TcpStoreBootstrap`).
"""
from __future__ import annotations

import threading
import time
from typing import Optional, Sequence


class PeerLost(RuntimeError):
    """One or more ranks stopped beating (``lost``) or announced that they left (``left``)."""

    def __init__(self, lost: Sequence[int], left: Sequence[int]):
        self.lost, self.left = tuple(lost), tuple(left)
        parts = []
        if self.lost:
            parts.append(f"no heartbeat from rank(s) {list(self.lost)}")
        if self.left:
            parts.append(f"rank(s) {list(self.left)} left")
        super().__init__("; ".join(parts))


class Heartbeat:
    """``Heartbeat(store, rank, world_size).start()``; then ``check()`` between steps."""

    def __init__(self, store, rank: int, world_size: int, *, interval: float = 0.2, timeout: float = 2.0,
                 prefix: str = "aboleth/liveness", clock=time.monotonic):
        if not 0 <= rank < world_size:
            raise ValueError("rank out of range")
        if timeout <= interval:
            raise ValueError("the timeout must exceed the beat interval")
        self.store, self.rank, self.world_size = store, rank, world_size
        self.interval, self.timeout, self.prefix, self._clock = interval, timeout, prefix, clock
        self._beats = 0
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None
        # What was last seen of each peer, and when it last changed.
        self._seen: dict[int, tuple[int, float]] = {}

    def _key(self, rank: int, what: str = "beat") -> str:
        return f"{self.prefix}/{what}/{rank}"

    def beat(self) -> None:
        """One beat (the thread calls this; a caller without the thread may call it per step)."""
        self._beats += 1
        self.store.set(self._key(self.rank), str(self._beats).encode())

    def start(self) -> "Heartbeat":
        self.beat()
        now = self._clock()
        self._seen = {peer: (0, now) for peer in range(self.world_size) if peer != self.rank}

        def run():
            while not self._stop.wait(self.interval):
                try:
                    self.beat()
                except Exception:  # noqa: BLE001 - the store went away with rank 0: peers will notice
                    return

        self._thread = threading.Thread(target=run, name="aboleth-heartbeat", daemon=True)
        self._thread.start()
        return self

    def _read(self, key: str) -> Optional[bytes]:
        try:
            if not self.store.check([key]):
                return None
            return bytes(self.store.get(key))
        except Exception:  # noqa: BLE001 - an unreachable store reads as silence
            return None

    def peers(self) -> dict[int, str]:
        """``alive`` / ``lost`` / ``left`` for every other rank, as of now."""
        now = self._clock()
        out = {}
        for peer in range(self.world_size):
            if peer == self.rank:
                continue
            if self._read(self._key(peer, "left")) is not None:
                out[peer] = "left"
                continue
            raw = self._read(self._key(peer))
            count = int(raw.decode()) if raw else 0
            last, since = self._seen.get(peer, (0, now))
            if count != last:
                self._seen[peer] = (count, now)
                since = now
            elif peer not in self._seen:
                self._seen[peer] = (count, now)
            out[peer] = "alive" if now - since <= self.timeout else "lost"
        return out

    def check(self) -> None:
        """Raise :class:`PeerLost` if any peer is lost or has left.  Call it between steps."""
        states = self.peers()
        lost = [p for p, s in states.items() if s == "lost"]
        left = [p for p, s in states.items() if s == "left"]
        if lost or left:
            raise PeerLost(lost, left)

    def leave(self) -> None:
        """Announce an orderly departure (between steps, nothing in flight) and stop beating."""
        try:
            self.store.set(self._key(self.rank, "left"), b"1")
        finally:
            self.stop()

    def stop(self) -> None:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2 * self.interval + 1.0)
            self._thread = None
