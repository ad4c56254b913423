"""World: one rank's view of every peer - endpoints, regions, address tables.

Bring-up is four steps, each a metadata all-gather over the bootstrap:

1. topology (``aboleth.world.topology.v2``): CUDA ordinal + ``host:boot_id``;
2. connections (``aboleth.world.connections.v3[:slot]``): per peer the wire
   transport code and either the peer-memory device ordinal or the 128-byte
   connection record of a queue endpoint;
3. regions (``aboleth.world.regions.{tag}.v3``): per (target peer, name) an
   :class:`AllocationHandle`;
4. the resulting :class:`PeerRegionTable` holds device tables a kernel indexes
   by rank: endpoint handles (kind bits or-ed in) and (address, key) pairs.

Tags, record layouts, validation rules (bundle covers every peer, transport
choice is symmetric, P2P device matches topology), the rollback of endpoints
after a failed connect and the ``auto`` policy (peer memory for same-node
payloads up to 16 KiB) follow the reference (python/aboleth/world.py:38-69,
181-246,272-400,439-604,750-916,1043-1177).
"""
from __future__ import annotations

import pathlib
import socket
import struct
from dataclasses import dataclass
from typing import Iterable, Mapping, Optional
from uuid import UUID

import torch

from .abi import WIRE_CODES
from .bootstrap import Bootstrap, LocalBootstrap, decode_bundle, encode_bundle
from .runtime import (AllocationHandle, AllocationProvider, LocalEndpoint, RegisteredBuffer,
                      RemoteBuffer, Runtime, Transport, connection_info_from_bytes,
                      connection_transport)

_TOPOLOGY_VERSION = 2
_CONNECTION_VERSION = 3
_REGION_VERSION = 3
_TOPOLOGY_HEAD = struct.Struct("<I")
_CONNECTION_HEAD = struct.Struct("<II")
_REGION_HEAD = struct.Struct("<IH")
_P2P_BODY = struct.Struct("<i")
_WIRE_BACK = {code: Transport(name) for name, code in WIRE_CODES.items()}


def _node_identity() -> str:
    """``hostname:boot_id``: two containers with one hostname stay distinct.

    ``ABOLETH_NODE_IDENTITY`` replaces it, so that ranks of one host can stand in for
    several nodes (the reference tests its multi-node bring-up the same way, with two
    "nodes" on one machine: test/CMakeLists.txt ``hardware.world-multinode-local``).
    """
    import os
    forced = os.environ.get("ABOLETH_NODE_IDENTITY", "")
    if forced:
        return forced
    host = socket.gethostname()
    try:
        boot = UUID(pathlib.Path("/proc/sys/kernel/random/boot_id").read_text().strip())
    except (OSError, ValueError):
        return host
    return f"{host}:{boot}"


@dataclass(frozen=True)
class TopologyInfo:
    rank: int
    device: int
    hostname: str

    def to_bytes(self) -> bytes:
        record = _TOPOLOGY_HEAD.pack(self.device) + self.hostname.encode("utf-8")
        return encode_bundle(_TOPOLOGY_VERSION, self.rank, [record])

    @classmethod
    def from_bytes(cls, data: bytes) -> "TopologyInfo":
        rank, records = decode_bundle(data, version=_TOPOLOGY_VERSION, kind="topology")
        if len(records) != 1:
            raise ValueError("an Aboleth topology bundle carries one record")
        (record,) = records
        if len(record) < _TOPOLOGY_HEAD.size:
            raise ValueError("truncated Aboleth topology record")
        hostname = record[_TOPOLOGY_HEAD.size:].decode("utf-8")
        if not hostname:
            raise ValueError("topology hostname cannot be empty")
        return cls(rank, int(_TOPOLOGY_HEAD.unpack_from(record)[0]), hostname)


@dataclass(frozen=True)
class ConnectionRecord:
    transport: Transport
    device: int
    info: object | None = None


@dataclass(frozen=True)
class AutoTransportPolicy:
    """Peer memory for same-node payloads up to a threshold, else the remote transport."""

    p2p_max_payload_bytes: int = 16 * 1024

    def __post_init__(self):
        if self.p2p_max_payload_bytes < 0:
            raise ValueError("P2P payload threshold cannot be negative")

    def select(self, *, can_p2p: bool, payload_bytes: Optional[int],
               remote_transport: Transport) -> Transport:
        if remote_transport not in (Transport.RDMA, Transport.PROXY, Transport.IONIC):
            raise ValueError("remote transport must be rdma or proxy")
        if payload_bytes is not None and payload_bytes < 0:
            raise ValueError("payload bytes cannot be negative")
        if can_p2p and (payload_bytes is None or payload_bytes <= self.p2p_max_payload_bytes):
            return Transport.P2P
        return remote_transport


@dataclass(frozen=True)
class LocalRegion:
    name: str
    address: int
    length: int
    lkey: int
    device: int
    generation: int
    _owner: RegisteredBuffer

    def export(self, peer: int, provider: AllocationProvider) -> AllocationHandle:
        offset = self.address - self._owner.address
        return self._owner.export_allocation(
            peer, offset=offset, length=self.length,
            mapped=provider != AllocationProvider.IB_VERBS)


def _encode_connections(rank: int, endpoints: Mapping[int, LocalEndpoint]) -> bytes:
    records = []
    for peer in sorted(endpoints):
        endpoint = endpoints[peer]
        head = _CONNECTION_HEAD.pack(peer, WIRE_CODES[endpoint.transport.value])
        if endpoint.transport == Transport.P2P:
            records.append(head + _P2P_BODY.pack(endpoint.device))
        else:
            records.append(head + endpoint.connection_info.to_bytes())
    return encode_bundle(_CONNECTION_VERSION, rank, records)


def _decode_connections(data: bytes) -> tuple[int, dict[int, ConnectionRecord]]:
    rank, records = decode_bundle(data, version=_CONNECTION_VERSION, kind="connection")
    out: dict[int, ConnectionRecord] = {}
    for record in records:
        if len(record) < _CONNECTION_HEAD.size:
            raise ValueError("truncated Aboleth connection record")
        peer, code = _CONNECTION_HEAD.unpack_from(record)
        body = record[_CONNECTION_HEAD.size:]
        if peer in out:
            raise ValueError("duplicate peer in Aboleth connection bundle")
        transport = _WIRE_BACK.get(code)
        if transport is None:
            raise ValueError(f"unknown connection transport {code}")
        if transport == Transport.P2P:
            if len(body) != _P2P_BODY.size:
                raise ValueError("invalid P2P connection-info size")
            out[peer] = ConnectionRecord(transport, _P2P_BODY.unpack(body)[0])
        else:
            info = connection_info_from_bytes(body)
            if connection_transport(info) != transport:
                raise ValueError("connection transport payload mismatch")
            out[peer] = ConnectionRecord(transport, -1, info)
    return rank, out


def _encode_regions(rank: int, regions: Mapping[str, LocalRegion],
                    endpoints: Mapping[int, LocalEndpoint], mapped_provider) -> bytes:
    records = []
    for target in sorted(endpoints):
        provider = (mapped_provider if endpoints[target].transport == Transport.P2P
                    else AllocationProvider.IB_VERBS)
        # Queue transports served by the ring on one node still need a mapping:
        # the proxy thread dereferences the peer's address.
        if provider == AllocationProvider.IB_VERBS:
            provider = mapped_provider
        for name in sorted(regions):
            encoded = name.encode("utf-8")
            if len(encoded) > 0xFFFF:
                raise ValueError("Aboleth region name is too large")
            records.append(_REGION_HEAD.pack(target, len(encoded)) + encoded +
                           regions[name].export(rank, provider).to_bytes())
    return encode_bundle(_REGION_VERSION, rank, records)


def _decode_regions(data: bytes, *, target_rank: int) -> tuple[int, dict[str, AllocationHandle]]:
    rank, records = decode_bundle(data, version=_REGION_VERSION, kind="region")
    out: dict[str, AllocationHandle] = {}
    for record in records:
        if len(record) < _REGION_HEAD.size:
            raise ValueError("truncated Aboleth region record")
        target, name_length = _REGION_HEAD.unpack_from(record)
        end = _REGION_HEAD.size + name_length
        if end > len(record):
            raise ValueError("truncated Aboleth region metadata")
        if target != target_rank:
            continue
        name = record[_REGION_HEAD.size:end].decode("utf-8")
        if not name:
            raise ValueError("invalid region name in Aboleth bundle")
        if name in out:
            raise ValueError("duplicate targeted region in Aboleth bundle")
        out[name] = AllocationHandle.from_bytes(record[end:])
    return rank, out


def _signed(values: Iterable[int]) -> list[int]:
    return [v - (1 << 64) if v >= (1 << 63) else v for v in values]


class PeerRegionTable:
    """Device tables over one exchange: who is where, under which key."""

    def __init__(self, world: "World", local_regions: Mapping[str, LocalRegion],
                 remote_regions: Mapping[int, Mapping[str, RemoteBuffer]],
                 strictly_ordered: bool = True):
        self.strictly_ordered = strictly_ordered
        self._world = world
        self._local = dict(local_regions)
        self._remote = {int(p): dict(r) for p, r in remote_regions.items()}
        self._tables: dict[tuple[str, str], torch.Tensor] = {}
        self._closed = False
        handles: list[int] = []
        for peer in range(world.world_size):
            for slot in range(world.endpoints_per_peer):
                handles.append(0 if peer == world.rank else world.endpoint(peer, slot=slot).handle)
        # Peer-major [world x endpoints_per_peer]; a kernel picks
        # peer * endpoints_per_peer + blockIdx.x % endpoints_per_peer.
        self._endpoint_handles = torch.tensor(_signed(handles), dtype=torch.int64,
                                              device=world.torch_device)

    @property
    def endpoint_handles(self) -> torch.Tensor:
        self._ensure_open()
        return self._endpoint_handles

    @property
    def rank(self) -> int:
        return self._world.rank

    @property
    def world_size(self) -> int:
        return self._world.world_size

    @property
    def closed(self) -> bool:
        return self._closed

    @property
    def names(self) -> tuple[str, ...]:
        return tuple(sorted(self._local))

    def local(self, name: str) -> LocalRegion:
        self._ensure_open()
        try:
            return self._local[name]
        except KeyError as error:
            raise KeyError(f"unknown local region {name!r}") from error

    def remote(self, peer: int, name: str) -> RemoteBuffer:
        self._ensure_open()
        if peer == self._world.rank:
            raise ValueError("the local rank has no remote region; use local()")
        try:
            return self._remote[peer][name]
        except KeyError as error:
            raise KeyError(f"rank {peer} did not export region {name!r}") from error

    def _table(self, kind: str, name: str, values) -> torch.Tensor:
        key = (kind, name)
        if key not in self._tables:
            self._tables[key] = torch.tensor(_signed(values()), dtype=torch.int64,
                                             device=self._world.torch_device)
        return self._tables[key]

    def addresses(self, name: str) -> torch.Tensor:
        """int64 ``[world]``: each rank's ``name`` region as seen from this rank."""
        self._ensure_open()
        me = self._world.rank
        return self._table("addresses", name, lambda: [
            self.local(name).address if p == me else self.remote(p, name).address
            for p in range(self.world_size)])

    def rkeys(self, name: str) -> torch.Tensor:
        self._ensure_open()
        me = self._world.rank
        return self._table("rkeys", name, lambda: [
            0 if p == me else self.remote(p, name).rkey for p in range(self.world_size)])

    def regions(self, name: str) -> torch.Tensor:
        """int64 ``[world, 2]`` flattened: (address, key) pairs, rank-major."""
        self._ensure_open()
        me = self._world.rank

        def build():
            out = []
            for p in range(self.world_size):
                if p == me:
                    out += [self.local(name).address, self.local(name).lkey]
                else:
                    out += [self.remote(p, name).address, self.remote(p, name).rkey]
            return out

        return self._table("regions", name, build)

    def generations(self, name: str) -> torch.Tensor:
        self._ensure_open()
        me = self._world.rank
        return self._table("generations", name, lambda: [
            self.local(name).generation if p == me else self.remote(p, name).generation
            for p in range(self.world_size)])

    def _ensure_open(self) -> None:
        if self._closed:
            raise RuntimeError("peer region table is closed")

    def close(self) -> None:
        if self._closed:
            return
        self._closed = True
        for regions in self._remote.values():
            for buffer in regions.values():
                buffer.close()
        self._tables.clear()


class World:
    """One rank among ``world_size``; ``world_size == 1`` is allowed here."""

    TOPOLOGY_TAG = "aboleth.world.topology.v2"
    CONNECTION_TAG = "aboleth.world.connections.v3"

    @staticmethod
    def region_tag(tag: str) -> str:
        return f"aboleth.world.regions.{tag}.v3"

    def __init__(self, rank: int, world_size: int, *, device=None,
                 bootstrap: Optional[Bootstrap] = None, runtime: Optional[Runtime] = None):
        self.rank = int(rank)
        self.world_size = int(world_size)
        if self.world_size < 1:
            raise ValueError("an Aboleth world needs at least one rank")
        if not 0 <= self.rank < self.world_size:
            raise ValueError("rank is outside the world")
        if bootstrap is None:
            if self.world_size != 1:
                raise ValueError("a bootstrap is required for more than one rank")
            bootstrap = LocalBootstrap()
        if bootstrap.rank != self.rank or bootstrap.world_size != self.world_size:
            raise ValueError("bootstrap rank/world size does not match the world")
        self.bootstrap = bootstrap
        self.runtime = runtime if runtime is not None else Runtime(device)
        self.device = self.runtime.device_index
        self.torch_device = self.runtime.torch_device
        self._endpoints: dict[int, tuple[LocalEndpoint, ...]] = {}
        self._endpoints_per_peer = 1
        self._topology: dict[int, TopologyInfo] = {}
        self._transport: Optional[Transport] = None
        self._peer_transports: dict[int, Transport] = {}
        self._tables: list[PeerRegionTable] = []
        self._connected = False
        self._closed = False

    # -- facts ----------------------------------------------------------------
    @property
    def hca(self) -> str:
        return self.runtime.hca

    @property
    def lid(self) -> int:
        return self.runtime.lid

    @property
    def transport(self) -> Optional[Transport]:
        return self._transport

    @property
    def peer_transports(self) -> Mapping[int, Transport]:
        return dict(self._peer_transports)

    @property
    def transport_geography(self) -> tuple[tuple[int, str], ...]:
        return tuple((p, t.value) for p, t in sorted(self._peer_transports.items()))

    @property
    def gpu_resident_queues(self) -> bool:
        return False

    @property
    def strict_registrations(self) -> bool:
        return True

    @property
    def endpoints_per_peer(self) -> int:
        return self._endpoints_per_peer

    @property
    def topology(self) -> Mapping[int, TopologyInfo]:
        return dict(self._topology)

    @property
    def endpoints(self) -> Mapping[int, LocalEndpoint]:
        return {peer: slots[0] for peer, slots in self._endpoints.items()}

    def endpoint(self, peer: int, *, slot: int = 0) -> LocalEndpoint:
        self._ensure_open()
        try:
            return self._endpoints[peer][slot]
        except (KeyError, IndexError) as error:
            raise KeyError(f"no endpoint to rank {peer} in slot {slot}") from error

    # -- bring-up ---------------------------------------------------------------
    def _can_p2p(self, info: TopologyInfo, same_node: bool) -> bool:
        if not same_node:
            return False
        if self.runtime._cpu:
            return True
        if info.device >= torch.cuda.device_count():
            return True  # another process's ordinal; IPC decides at import
        if info.device == self.device:
            return True
        return bool(torch.cuda.can_device_access_peer(self.device, info.device))

    def connect_all(self, transport, *, remote_transport=Transport.RDMA,
                    payload_bytes: Optional[int] = None,
                    auto_policy: Optional[AutoTransportPolicy] = None,
                    endpoints_per_peer: int = 1) -> None:
        self._ensure_open()
        if self._connected:
            raise RuntimeError("Aboleth World is already connected")
        endpoints_per_peer = int(endpoints_per_peer)
        if endpoints_per_peer < 1:
            raise ValueError("endpoints_per_peer must be >= 1")
        requested = Transport(transport)
        remote = Transport(remote_transport)
        policy = AutoTransportPolicy() if auto_policy is None else auto_policy
        if not isinstance(policy, AutoTransportPolicy):
            raise TypeError("auto_policy must be an AutoTransportPolicy")
        if remote not in (Transport.RDMA, Transport.PROXY, Transport.IONIC):
            raise ValueError("remote transport must be rdma or proxy")
        if requested == Transport.EFA:
            raise ValueError("unsupported World transport")

        mine = TopologyInfo(self.rank, self.device, _node_identity())
        gathered = self.bootstrap.all_gather(self.TOPOLOGY_TAG, mine.to_bytes())
        topology = {peer: TopologyInfo.from_bytes(blob) for peer, blob in gathered.items()}
        for peer, info in topology.items():
            if info.rank != peer:
                raise RuntimeError(f"invalid topology bundle from rank {peer}")

        chosen: dict[int, Transport] = {}
        for peer, info in topology.items():
            if peer == self.rank:
                continue
            same_node = info.hostname == mine.hostname
            can_p2p = self._can_p2p(info, same_node)
            if requested == Transport.AUTO:
                chosen[peer] = policy.select(can_p2p=can_p2p, payload_bytes=payload_bytes,
                                             remote_transport=remote)
            elif requested == Transport.P2P:
                if not same_node:
                    raise ValueError(f"rank {peer} is not on the local node")
                if not can_p2p:
                    raise ValueError(f"rank {peer} is not P2P accessible")
                chosen[peer] = Transport.P2P
            else:
                chosen[peer] = requested

        per_slot: list[dict[int, LocalEndpoint]] = []
        try:
            for slot in range(endpoints_per_peer):
                endpoints: dict[int, LocalEndpoint] = {}
                per_slot.append(endpoints)
                for peer, selected in chosen.items():
                    endpoints[peer] = self.runtime.create_local_endpoint(selected)
                tag = self.CONNECTION_TAG if slot == 0 else f"{self.CONNECTION_TAG}:{slot}"
                bundles = self.bootstrap.all_gather(tag, _encode_connections(self.rank, endpoints))
                for peer, endpoint in endpoints.items():
                    their_rank, connections = _decode_connections(bundles[peer])
                    expected = set(range(self.world_size)) - {peer}
                    if their_rank != peer or set(connections) != expected:
                        raise RuntimeError(f"invalid endpoint bundle from rank {peer}")
                    record = connections[self.rank]
                    if record.transport != endpoint.transport:
                        raise RuntimeError("peer transport selection is asymmetric")
                    if endpoint.transport == Transport.P2P:
                        if record.device != topology[peer].device:
                            raise RuntimeError(f"P2P device mismatch for rank {peer}")
                        endpoint.connect_p2p(peer, record.device)
                    else:
                        if record.info is None:
                            raise RuntimeError("queue connection omitted endpoint info")
                        endpoint.connect(peer, record.info)
        except Exception as original:
            for endpoints in per_slot:
                for endpoint in endpoints.values():
                    try:
                        endpoint.close()
                    except Exception as cleanup:  # noqa: BLE001
                        original.add_note(f"Aboleth endpoint rollback also failed: {cleanup}")
            raise
        self._endpoints = {peer: tuple(e[peer] for e in per_slot) for peer in chosen}
        self._endpoints_per_peer = endpoints_per_peer
        self._topology = topology
        self._peer_transports = chosen
        kinds = set(chosen.values())
        self._transport = (next(iter(kinds)) if len(kinds) == 1 else
                           (Transport.P2P if not kinds else Transport.AUTO))
        self._connected = True

    # -- memory ------------------------------------------------------------------
    def register(self, tensor: torch.Tensor, *, network: bool = True) -> RegisteredBuffer:
        self._ensure_open()
        return self.runtime.register(tensor, network=network)

    def region(self, name: str, registration: RegisteredBuffer,
               tensor: Optional[torch.Tensor] = None, *, offset: int = 0,
               length: Optional[int] = None) -> LocalRegion:
        self._ensure_open()
        if not name:
            raise ValueError("Aboleth region name cannot be empty")
        if tensor is not None:
            if not tensor.is_contiguous():
                raise ValueError("Aboleth region tensor must be contiguous")
            if tensor.device != registration.tensor.device:
                raise ValueError("region tensor and registration use different devices")
            address = tensor.data_ptr() + offset
            available = tensor.numel() * tensor.element_size() - offset
        else:
            address = registration.address + offset
            available = registration.length - offset
        if length is None:
            length = available
        inside = (offset >= 0 and length >= 0 and address >= registration.address and
                  address + length <= registration.address + registration.length)
        if not inside:
            raise ValueError(f"region {name!r} is outside its registration")
        return LocalRegion(name, address, length, registration.lkey, registration.device,
                           registration.generation, registration)

    def exchange_regions(self, regions: Iterable[LocalRegion], tag: str = "default") -> PeerRegionTable:
        """Tell every peer where the named regions are; learn theirs."""
        self._ensure_open()
        if not self._connected:
            raise RuntimeError("connect_all() must run before exchange_regions()")
        local: dict[str, LocalRegion] = {}
        for region in regions:
            if region.name in local:
                raise ValueError(f"duplicate region name {region.name!r}")
            local[region.name] = region
        endpoints = self.endpoints
        payload = _encode_regions(self.rank, local, endpoints, self.runtime._memory.provider)
        bundles = self.bootstrap.all_gather(self.region_tag(tag), payload)
        remote: dict[int, dict[str, RemoteBuffer]] = {}
        try:
            for peer in endpoints:
                their_rank, handles = _decode_regions(bundles[peer], target_rank=self.rank)
                if their_rank != peer:
                    raise RuntimeError(f"invalid region bundle from rank {peer}")
                if set(handles) != set(local):
                    raise RuntimeError(
                        f"rank {peer} exported regions {sorted(handles)}, expected {sorted(local)}")
                remote[peer] = {}
                for name, handle in handles.items():
                    if handle.peer != peer:
                        raise RuntimeError(f"region {name!r} from rank {peer} names rank {handle.peer}")
                    remote[peer][name] = self.runtime.import_remote_buffer(handle)
        except Exception:
            for buffers in remote.values():
                for buffer in buffers.values():
                    buffer.close()
            raise
        table = PeerRegionTable(self, local, remote)
        self._tables.append(table)
        return table

    # -- Tier 1 / Tier 2 entry points ----------------------------------------------
    def device_library(self, **options):
        """Include directory, header and manifest of the Tier-1 device library."""
        from .device_library import cached_device_library

        transports = sorted({t.value for t in self._peer_transports.values()} or {"p2p"})
        return cached_device_library(transports=transports, **options)

    def compilation(self, **options):
        """Context manager that fixes the Tier-2 specializer options for this world."""
        from .compiler import compilation

        backend = options.pop("backend", None)
        if backend is None:
            backend = (self._transport.value if self._transport not in (None, Transport.AUTO)
                       else "p2p")
        options.setdefault("rank", self.rank)
        options.setdefault("world_size", self.world_size)
        return compilation(backend=backend, **options)

    def endpoint_registration(self, lanes: Optional[int] = None):
        """Agree with every peer on how many endpoint lanes each side offers."""
        lanes = self._endpoints_per_peer if lanes is None else int(lanes)
        blobs = self.bootstrap.all_gather(f"aboleth.world.endpoint-registration.{lanes}",
                                          struct.pack("<II", self.rank, self._endpoints_per_peer))
        offered = {peer: struct.unpack("<II", blob)[1] for peer, blob in blobs.items()}
        return {"lanes": min([lanes, *offered.values()]), "offered": offered}

    def endpoint_profiles(self, lanes: Optional[int] = None):
        """The measured (or seed) endpoint profile of each peer link."""
        from .endpoint_profiles import resolve_profiles

        lanes = self._endpoints_per_peer if lanes is None else int(lanes)
        links = {peer: ("NV18" if t == Transport.P2P else "host") for peer, t in
                 self._peer_transports.items()}
        blob = repr(sorted(links.items())).encode()
        self.bootstrap.all_gather(f"aboleth.world.endpoint-links.{lanes}", blob)
        self._resolved_profiles = resolve_profiles(self._peer_transports, links)
        return self._resolved_profiles

    @property
    def resolved_endpoint_profiles(self):
        return getattr(self, "_resolved_profiles", None)

    # -- teardown ---------------------------------------------------------------------
    def _ensure_open(self) -> None:
        if self._closed:
            raise RuntimeError("Aboleth World is closed")

    def close(self) -> None:
        if self._closed:
            return
        self._closed = True
        for table in self._tables:
            table.close()
        for slots in self._endpoints.values():
            for endpoint in slots:
                endpoint.close()
        self._endpoints.clear()
        self.runtime.close()

    def __enter__(self) -> "World":
        return self

    def __exit__(self, *exc) -> None:
        self.close()
