"""Control-plane collectives used only while a world is being brought up.

Everything a rank tells its peers during bring-up (topology, endpoint
connection records, exported regions) travels through one primitive,
``all_gather(tag, payload) -> {rank: bytes}``.  Three carriers implement it:

* :class:`TcpStoreBootstrap` - a ``torch.distributed.TCPStore`` hosted by rank 0,
  keys ``aboleth/{sequence}/{tag}/{rank}``;
* :class:`PipeBootstrap` with :class:`PipeBootstrapCoordinator` - multiprocessing
  pipes to a coordinator, for launchers that spawn their own ranks;
* :class:`TorchDistributedBootstrap` - an existing process group's
  ``all_gather_object``.

Payloads are framed as *bundles*: ``<III`` (version, rank, record count) and
``<I``-length-prefixed records.  The framing, the store key scheme and the
error behaviour (version skew, truncation, trailing bytes, a peer that never
arrives) are those of the reference (python/aboleth/bootstrap.py:19-70,
:84-139, :142-247, :250-359) so the two implementations can share a store.
"""
from __future__ import annotations

import os
import struct
import time
from datetime import timedelta
from multiprocessing.connection import wait as _wait_connections
from typing import Iterable, Mapping, Protocol, runtime_checkable

_HEADER = struct.Struct("<III")
_LENGTH = struct.Struct("<I")


def encode_bundle(version: int, rank: int, records: Iterable[bytes]) -> bytes:
    """Frame ``records`` from ``rank`` as one bundle of the given version."""
    body = bytearray()
    n = 0
    for record in records:
        record = bytes(record)
        body += _LENGTH.pack(len(record))
        body += record
        n += 1
    return _HEADER.pack(int(version), int(rank), n) + bytes(body)


def decode_bundle(payload: bytes, *, version: int, kind: str) -> tuple[int, tuple[bytes, ...]]:
    """Return ``(rank, records)`` or raise ``ValueError`` saying what is wrong."""
    data = memoryview(bytes(payload))
    if len(data) < _HEADER.size:
        raise ValueError(f"truncated Aboleth {kind} bundle")
    got_version, rank, count = _HEADER.unpack_from(data)
    if got_version != version:
        raise ValueError(
            f"unsupported Aboleth {kind}-bundle version {got_version}: this rank speaks "
            f"version {version}, so every rank must run the same Aboleth build")
    cursor = _HEADER.size
    records: list[bytes] = []
    for _ in range(count):
        if cursor + _LENGTH.size > len(data):
            raise ValueError(f"truncated Aboleth {kind} record")
        (length,) = _LENGTH.unpack_from(data, cursor)
        cursor += _LENGTH.size
        if cursor + length > len(data):
            raise ValueError(f"truncated Aboleth {kind} record")
        records.append(bytes(data[cursor:cursor + length]))
        cursor += length
    if cursor != len(data):
        raise ValueError(f"trailing bytes in Aboleth {kind} bundle")
    return int(rank), tuple(records)


@runtime_checkable
class Bootstrap(Protocol):
    rank: int
    world_size: int

    def all_gather(self, tag: str, payload: bytes) -> dict[int, bytes]: ...


def _check_rank(rank: int, world_size: int, what: str) -> None:
    if world_size < 1:
        raise ValueError(f"{what} needs at least one rank")
    if not 0 <= rank < world_size:
        raise ValueError(f"{what} rank is outside the world")


class TorchDistributedBootstrap:
    """Bring-up collectives over a process group the client already owns.

    Only metadata crosses the group.  Every record carries the caller's
    sequence number, tag and rank so that ranks which entered different
    collectives fail loudly instead of exchanging unrelated bytes.
    """

    def __init__(self, group):
        self._group = group
        self.rank = int(group.rank())
        self.world_size = int(group.size())
        _check_rank(self.rank, self.world_size, "torch.distributed bootstrap")
        self._sequence = 0

    def all_gather(self, tag: str, payload: bytes) -> dict[int, bytes]:
        import torch.distributed as dist

        sequence, self._sequence = self._sequence, self._sequence + 1
        mine = (sequence, str(tag), self.rank, bytes(payload))
        slots: list = [None] * self.world_size
        dist.all_gather_object(slots, mine, group=self._group)
        out: dict[int, bytes] = {}
        for rank, record in enumerate(slots):
            if not (isinstance(record, tuple) and len(record) == 4):
                raise RuntimeError(
                    f"rank {rank} returned an invalid Aboleth bootstrap record for {tag}")
            their_sequence, their_tag, their_rank, their_payload = record
            if int(their_sequence) != sequence or their_tag != tag or int(their_rank) != rank:
                raise RuntimeError(
                    f"rank {rank} entered a different Aboleth bootstrap collective than {tag}")
            out[rank] = bytes(their_payload)
        return out

    def barrier(self, tag: str = "barrier") -> None:
        self.all_gather(tag, b"")


class PipeBootstrap:
    """A rank's end of a pipe to a :class:`PipeBootstrapCoordinator`."""

    def __init__(self, rank: int, world_size: int, connection):
        self.rank = int(rank)
        self.world_size = int(world_size)
        self._connection = connection

    def all_gather(self, tag: str, payload: bytes) -> dict[int, bytes]:
        self._connection.send({"kind": "aboleth_all_gather", "tag": tag, "rank": self.rank,
                               "payload": bytes(payload)})
        reply = self._connection.recv()
        kind = reply.get("kind")
        if kind == "aboleth_bootstrap_error":
            raise RuntimeError(reply["error"])
        if kind != "aboleth_all_gather_result" or reply.get("tag") != tag:
            raise RuntimeError(f"invalid Aboleth bootstrap response for {tag}")
        gathered = {int(r): bytes(v) for r, v in reply["payloads"].items()}
        if set(gathered) != set(range(self.world_size)):
            raise RuntimeError(f"incomplete Aboleth bootstrap result for {tag}")
        return gathered

    def barrier(self, tag: str = "barrier") -> None:
        self.all_gather(tag, b"")


class PipeBootstrapCoordinator:
    """Collects one message per rank and answers every rank with all of them.

    A failure (a rank that reports ``ok=False``, a malformed message, a rank
    that does not arrive within ``timeout`` seconds) is broadcast to every
    rank as an error before it is raised here, so no rank is left waiting.
    """

    def __init__(self, connections: Mapping[int, object], world_size: int):
        self._connections = dict(connections)
        self.world_size = int(world_size)
        if set(self._connections) != set(range(self.world_size)):
            raise ValueError("bootstrap connections must cover every rank")

    def all_gather(self, tag: str, *, timeout: float = 300) -> dict[int, bytes]:
        deadline = time.monotonic() + timeout
        waiting = {conn: rank for rank, conn in self._connections.items()}
        payloads: dict[int, bytes] = {}
        try:
            while waiting:
                left = deadline - time.monotonic()
                if left <= 0:
                    raise TimeoutError(
                        f"ranks {sorted(waiting.values())} did not reach bootstrap {tag}")
                for conn in _wait_connections(tuple(waiting), timeout=left):
                    rank = waiting.pop(conn)
                    message = conn.recv()
                    if message.get("ok") is False:
                        raise RuntimeError(message["error"])
                    if (message.get("kind") != "aboleth_all_gather" or message.get("tag") != tag
                            or int(message.get("rank", -1)) != rank):
                        raise RuntimeError(
                            f"rank {rank} sent an invalid bootstrap message for {tag}")
                    payloads[rank] = bytes(message["payload"])
        except Exception as error:
            self._broadcast({"kind": "aboleth_bootstrap_error", "tag": tag, "error": str(error)},
                            tolerate=True)
            raise
        self._broadcast({"kind": "aboleth_all_gather_result", "tag": tag, "payloads": payloads})
        return payloads

    def serve(self, collectives: int, *, timeout: float = 300) -> None:
        """Serve ``collectives`` successive all-gathers, whatever their tags."""
        for _ in range(collectives):
            self._serve_any(timeout)

    def _serve_any(self, timeout: float) -> None:
        deadline = time.monotonic() + timeout
        waiting = {conn: rank for rank, conn in self._connections.items()}
        payloads: dict[int, bytes] = {}
        tag = None
        try:
            while waiting:
                left = deadline - time.monotonic()
                if left <= 0:
                    raise TimeoutError(
                        f"ranks {sorted(waiting.values())} did not reach bootstrap {tag}")
                for conn in _wait_connections(tuple(waiting), timeout=left):
                    rank = waiting.pop(conn)
                    message = conn.recv()
                    if message.get("ok") is False:
                        raise RuntimeError(message["error"])
                    if tag is None:
                        tag = message.get("tag")
                    if (message.get("kind") != "aboleth_all_gather" or message.get("tag") != tag
                            or int(message.get("rank", -1)) != rank):
                        raise RuntimeError(
                            f"rank {rank} sent an invalid bootstrap message for {tag}")
                    payloads[rank] = bytes(message["payload"])
        except Exception as error:
            self._broadcast({"kind": "aboleth_bootstrap_error", "tag": tag, "error": str(error)},
                            tolerate=True)
            raise
        self._broadcast({"kind": "aboleth_all_gather_result", "tag": tag, "payloads": payloads})

    def _broadcast(self, message: dict, *, tolerate: bool = False) -> None:
        for conn in self._connections.values():
            try:
                conn.send(message)
            except (EOFError, OSError):
                if not tolerate:
                    raise


class TcpStoreBootstrap:
    """Bring-up collectives over a ``TCPStore``; rank 0 hosts the store.

    No process group is created.  Keys are numbered by a per-instance counter,
    so all ranks must issue the same collectives in the same order, and rank 0
    must outlive the others' last collective.
    """

    def __init__(self, rank: int, world_size: int, *, host: str, port: int, timeout: float = 300.0):
        from torch.distributed import TCPStore

        self.rank = int(rank)
        self.world_size = int(world_size)
        _check_rank(self.rank, self.world_size, "Aboleth bootstrap")
        self.host = str(host)
        self.port = int(port)
        self.timeout = float(timeout)
        self._sequence = 0
        self._store = TCPStore(self.host, self.port, self.world_size, self.rank == 0,
                               timeout=timedelta(seconds=self.timeout))

    @classmethod
    def from_env(cls, *, timeout: float = 300.0) -> "TcpStoreBootstrap":
        values = {}
        for name in ("MASTER_ADDR", "MASTER_PORT", "RANK", "WORLD_SIZE"):
            value = os.environ.get(name)
            if not value:
                raise RuntimeError(
                    f"{name} is unset: the Aboleth TCP bootstrap reads MASTER_ADDR, "
                    "MASTER_PORT, RANK, and WORLD_SIZE")
            values[name] = value
        return cls(int(values["RANK"]), int(values["WORLD_SIZE"]), host=values["MASTER_ADDR"],
                   port=int(values["MASTER_PORT"]), timeout=timeout)

    def _key(self, sequence: int, tag: str, rank: int) -> str:
        return f"aboleth/{sequence}/{tag}/{rank}"

    @property
    def store(self):
        """The key-value store behind the collectives (``set`` / ``get`` / ``add``), for small
        out-of-band messages between the same ranks; ``None`` once closed."""
        return self._store

    def all_gather(self, tag: str, payload: bytes) -> dict[int, bytes]:
        if self._store is None:
            raise RuntimeError("Aboleth TCP bootstrap is closed")
        sequence, self._sequence = self._sequence, self._sequence + 1
        self._store.set(self._key(sequence, tag, self.rank), bytes(payload))
        gathered: dict[int, bytes] = {}
        for peer in range(self.world_size):
            try:
                gathered[peer] = bytes(self._store.get(self._key(sequence, tag, peer)))
            except Exception as error:  # the store raises on its own timeout
                raise TimeoutError(
                    f"rank {self.rank} did not receive rank {peer} at bootstrap {tag}") from error
        return gathered

    def barrier(self, tag: str = "barrier") -> None:
        """All ranks arrive; rank 0 (the store's host) returns last.

        After the gather every other rank acknowledges that it has read all keys, and rank 0
        waits for those acknowledgements: when ``barrier`` returns on rank 0 no peer still
        needs the store, so rank 0 may drop it.
        """
        sequence = self._sequence
        self.all_gather(tag, b"")
        if self.rank != 0:
            self._store.set(self._key(sequence, tag + ".read", self.rank), b"\x01")
            return
        for peer in range(1, self.world_size):
            try:
                self._store.get(self._key(sequence, tag + ".read", peer))
            except Exception as error:
                raise TimeoutError(
                    f"rank 0 did not see rank {peer} leave bootstrap {tag}") from error

    def close(self) -> None:
        self._store = None


class LocalBootstrap:
    """A world of one: every collective returns the caller's own payload."""

    rank = 0
    world_size = 1

    def all_gather(self, tag: str, payload: bytes) -> dict[int, bytes]:
        return {0: bytes(payload)}

    def barrier(self, tag: str = "barrier") -> None:
        return None
