"""Per-rank runtime: registered buffers, endpoints, exported and imported memory.

The class and wire-record surface follows the reference
(python/aboleth/runtime.py:35-41,83-86,123-328,331-500,532-631,750-1017,
1128-1229,1232-1904): ``Transport``, ``Provider``, ``AllocationProvider``,
``RemoteHandle`` (``<QQIIQ``), ``AllocationHandle`` (``<BBHIiQQQQQQQIHHHQB`` +
blobs, abi 2), ``RegisteredBuffer``, ``LocalBuffer``, ``RemoteBuffer``,
``LocalEndpoint``, ``Endpoint``, ``EndpointTable``, ``Runtime``.

What differs is the machinery underneath.  A B200 NVSwitch box has one data
path that matters - peer memory - so:

* ``register`` records the tensor in the native key table and can export it as
  a CUDA IPC handle; nothing is pinned with a NIC;
* a P2P endpoint is a one-byte device tensor whose address, tagged with kind
  bit 1, is the device handle (as in the reference);
* every queue transport name (rdma, proxy, efa, ionic) is served by the native
  host-proxy ring, whose progress thread moves bytes with CUDA copies;
* a ``cpu`` runtime backs the same API with POSIX shared memory so that the
  whole bring-up (and the proxy ring) can be exercised by CPU-only ranks.
"""
from __future__ import annotations

import ctypes
import struct
import threading
from dataclasses import dataclass
from enum import Enum, IntEnum
from multiprocessing import shared_memory
from typing import Mapping, Optional

import torch

from . import _native
from .abi import (ConnectionInfo, EndpointConfig, KIND_BITS, PROVIDER_CUDA, PROVIDER_EFA,
                  PROVIDER_HIP, PROVIDER_IONIC, PROVIDER_LIBFABRIC, PROVIDER_MLX5, PROVIDER_VERBS,
                  ProxyEndpointDescriptor)


class Transport(str, Enum):
    AUTO = "auto"
    RDMA = "rdma"
    P2P = "p2p"
    PROXY = "proxy"
    EFA = "efa"
    IONIC = "ionic"


class Provider(IntEnum):
    VERBS = PROVIDER_VERBS
    MLX5 = PROVIDER_MLX5
    EFA = PROVIDER_EFA
    LIBFABRIC = PROVIDER_LIBFABRIC
    CUDA = PROVIDER_CUDA
    HIP = PROVIDER_HIP
    IONIC = PROVIDER_IONIC


class AllocationProvider(IntEnum):
    IB_VERBS = 1
    CUDA_IPC = 2
    CUDA_VMM = 3  # virtual-memory allocations with peer and multicast mappings: symmetric.SymmetricArena
    HOST_SHM = 16  # CPU-only ranks of this build; outside the reference's range


# Native connection codes (the third numbering; see abi.py for the other two).
_NATIVE_TRANSPORT = {Transport.RDMA: 1, Transport.PROXY: 2, Transport.EFA: 3, Transport.IONIC: 4}
_NATIVE_TRANSPORT_BACK = {v: k for k, v in _NATIVE_TRANSPORT.items()}


def _lib():
    lib = _native.load("runtime")
    if getattr(lib, "_ab_typed", False):
        return lib
    c = ctypes
    lib.aboleth_runtime_last_error.restype = c.c_char_p
    lib.aboleth_runtime_provider_caps.restype = c.c_uint32
    lib.aboleth_runtime_create_for_device.restype = c.c_void_p
    lib.aboleth_runtime_create_for_device.argtypes = [c.c_int, c.c_char_p]
    lib.aboleth_runtime_destroy.argtypes = [c.c_void_p]
    lib.aboleth_runtime_register_buffer.restype = c.c_void_p
    lib.aboleth_runtime_register_buffer.argtypes = [c.c_void_p, c.c_int, c.c_void_p, c.c_size_t,
                                                    c.c_uint64]
    lib.aboleth_runtime_unregister_buffer.argtypes = [c.c_void_p]
    lib.aboleth_runtime_buffer_lkey.restype = c.c_uint32
    lib.aboleth_runtime_buffer_lkey.argtypes = [c.c_void_p]
    lib.aboleth_runtime_buffer_rkey.restype = c.c_uint32
    lib.aboleth_runtime_buffer_rkey.argtypes = [c.c_void_p]
    lib.aboleth_runtime_create_local_endpoint.restype = c.c_void_p
    lib.aboleth_runtime_create_local_endpoint.argtypes = [c.c_void_p, c.c_uint32, c.c_int,
                                                          c.c_void_p, c.c_size_t, c.c_void_p]
    lib.aboleth_runtime_local_endpoint_connection_info.argtypes = [c.c_void_p, c.c_void_p]
    lib.aboleth_runtime_connect_local_endpoint.argtypes = [c.c_void_p, c.c_void_p]
    lib.aboleth_runtime_local_endpoint_state.argtypes = [c.c_void_p] + [c.POINTER(c.c_uint64)] * 3
    for name in ("capacity", "max_inline", "submit_mode", "gpu_resident_queues"):
        getattr(lib, f"aboleth_runtime_local_endpoint_{name}").argtypes = [
            c.c_void_p, c.POINTER(c.c_uint32)]
    lib.aboleth_runtime_destroy_local_endpoint.argtypes = [c.c_void_p]
    lib.ab200_ipc_export.argtypes = [c.c_void_p, c.c_void_p, c.POINTER(c.c_uint64),
                                     c.POINTER(c.c_uint64)]
    lib.ab200_ipc_open.argtypes = [c.c_void_p, c.POINTER(c.c_void_p)]
    lib.ab200_ipc_close.argtypes = [c.c_void_p]
    lib.ab200_enable_peer_access.argtypes = [c.c_int, c.c_int]
    lib.ab200_proxy_host_submit.restype = c.c_uint64
    lib.ab200_proxy_host_submit.argtypes = [c.c_void_p, c.c_void_p, c.c_int, c.c_double]
    lib.ab200_proxy_host_poll.restype = c.c_uint64
    lib.ab200_proxy_host_poll.argtypes = [c.c_void_p, c.c_uint64, c.c_double]
    lib.ab200_endpoint_descriptor.argtypes = [c.c_void_p, c.c_void_p]
    lib.ab200_endpoint_inject_failure.argtypes = [c.c_void_p, c.c_uint64, c.c_int]
    lib.ab200_endpoint_stats.argtypes = [c.c_void_p, c.POINTER(c.c_uint64)]
    lib.ab200_endpoint_snapshot.restype = c.c_longlong
    lib.ab200_endpoint_snapshot.argtypes = [c.c_void_p, c.c_uint64, c.c_int, c.c_void_p, c.c_size_t]
    lib.ab200_probe_providers.restype = c.c_uint32
    lib.aboleth_runtime_select_device.argtypes = [c.c_int, c.c_char_p, c.c_size_t]
    lib.aboleth_runtime_select_gid_index.argtypes = [c.c_char_p, c.c_int]
    lib.aboleth_runtime_query_port_address.argtypes = [
        c.c_char_p, c.c_int, c.POINTER(c.c_uint16), c.POINTER(c.c_uint8), c.c_void_p,
        c.POINTER(c.c_int), c.POINTER(c.c_uint32)]
    lib._ab_typed = True
    return lib


def last_error() -> str:
    return (_lib().aboleth_runtime_last_error() or b"").decode("utf-8", "replace")


def provider_caps() -> int:
    """Bit mask of providers that are compiled in, loadable and present."""
    return int(_lib().aboleth_runtime_provider_caps())


def probe_providers() -> int:
    """Bit mask of providers whose library resolves through ``dlopen`` and for which
    the machine lists a device, whether or not this build can drive them.

    :func:`provider_caps` is this mask restricted to what the build has a code path
    for (CUDA); the difference tells a caller that an adapter is present but would
    be served through the host-proxy ring.
    """
    return int(_lib().ab200_probe_providers())


def select_device(gpu_index: int = -1) -> str:
    """Name of the mlx5 adapter nearest (deepest shared PCI path) to CUDA ordinal
    ``gpu_index``; ``ABOLETH_HCA`` overrides, a negative ordinal takes the first one.
    Raises :class:`RuntimeError` when the machine lists no such adapter
    (reference: ``aboleth_runtime_select_device``, include/aboleth/runtime_c.h:142-150).
    """
    buffer = ctypes.create_string_buffer(64)
    if _lib().aboleth_runtime_select_device(int(gpu_index), buffer, len(buffer)) != 0:
        raise RuntimeError(last_error())
    return buffer.value.decode()


def select_gid_index(device_name: str = "", port: int = 0) -> int:
    """GID index a verbs client would use on ``device_name``: 0 on InfiniBand, a
    RoCE v2 entry on Ethernet, ``ABOLETH_GID_INDEX`` over both."""
    index = _lib().aboleth_runtime_select_gid_index(device_name.encode(), int(port))
    if index < 0:
        raise RuntimeError(last_error())
    return int(index)


@dataclass(frozen=True)
class PortAddress:
    """Local end of a reliable-connected path (``aboleth_runtime_query_port_address``)."""
    lid: int
    link_layer: int  # 1 InfiniBand (addressed by LID), 2 Ethernet (addressed by GRH)
    gid: bytes
    gid_index: int
    path_mtu: int  # ibv_mtu enumerator: 1 = 256 bytes ... 5 = 4096 bytes

    @property
    def is_global(self) -> bool:
        return self.link_layer != 1

    @property
    def path_mtu_bytes(self) -> int:
        return 128 << self.path_mtu


def query_port_address(device_name: str = "", port: int = 0) -> PortAddress:
    lid, layer = ctypes.c_uint16(), ctypes.c_uint8()
    gid = (ctypes.c_uint8 * 16)()
    index, mtu = ctypes.c_int(), ctypes.c_uint32()
    if _lib().aboleth_runtime_query_port_address(device_name.encode(), int(port), ctypes.byref(lid),
                                                 ctypes.byref(layer), gid, ctypes.byref(index),
                                                 ctypes.byref(mtu)) != 0:
        raise RuntimeError(last_error())
    return PortAddress(lid.value, layer.value, bytes(gid), index.value, mtu.value)


def available_transports() -> tuple[Transport, ...]:
    """Transports this machine can serve right now."""
    out = []
    if provider_caps() & Provider.CUDA:
        out.append(Transport.P2P)
    # The ring needs no provider: in host mode it runs on plain memory.
    out.append(Transport.PROXY)
    return tuple(out)


def connection_info_from_bytes(data: bytes) -> ConnectionInfo:
    """Size-checked view of a peer's 128-byte connection record."""
    return ConnectionInfo.from_bytes(data)


def connection_transport(info: ConnectionInfo) -> Transport:
    try:
        return _NATIVE_TRANSPORT_BACK[int(info.transport)]
    except KeyError as error:
        raise ValueError(f"unknown native endpoint transport {info.transport}") from error


@dataclass(frozen=True)
class RemoteHandle:
    address: int
    length: int
    rkey: int
    peer: int
    generation: int

    _FORMAT = "<QQIIQ"

    def to_bytes(self) -> bytes:
        return struct.pack(self._FORMAT, self.address, self.length, self.rkey, self.peer,
                           self.generation)

    @classmethod
    def from_bytes(cls, data: bytes) -> "RemoteHandle":
        if len(data) != struct.calcsize(cls._FORMAT):
            raise ValueError("invalid Aboleth remote handle size")
        return cls(*struct.unpack(cls._FORMAT, data))


@dataclass(frozen=True)
class AllocationHandle:
    """Everything a peer needs to map (or address) a slice of an allocation."""

    provider: AllocationProvider
    peer: int
    device: int
    generation: int
    address: int
    allocation_length: int
    allocation_size: int
    mapping_offset: int
    offset: int
    length: int
    rkey: int = 0
    ipc_handle: bytes = b""
    ref_counter_handle: bytes = b""
    ref_counter_offset: int = 0
    event_handle: bytes = b""
    event_sync_required: bool = False
    strictly_ordered: bool = False
    abi_version: int = 2

    _HEADER = struct.Struct("<BBHIiQQQQQQQIHHHQB")
    _STRICT = 0x1

    def __post_init__(self) -> None:
        if self.abi_version != 2:
            raise ValueError("unsupported Aboleth allocation-handle version")
        if self.peer < 0 or self.device < 0:
            raise ValueError("allocation handle requires non-negative peer/device")
        sizes = (self.allocation_length, self.allocation_size, self.mapping_offset, self.offset,
                 self.length)
        if min(sizes) < 0 or self.offset + self.length > self.allocation_length:
            raise ValueError("allocation handle region is outside its allocation")
        if self.mapping_offset + self.allocation_length > self.allocation_size:
            raise ValueError("registered buffer exceeds CUDA allocation range")
        mapped = self.provider in (AllocationProvider.CUDA_IPC, AllocationProvider.HOST_SHM)
        if mapped and not self.ipc_handle:
            raise ValueError("CUDA IPC allocation requires a memory handle")
        if self.provider == AllocationProvider.CUDA_IPC and self.rkey != 0:
            raise ValueError("CUDA IPC allocation cannot carry an rkey")
        if self.provider == AllocationProvider.IB_VERBS and (
                self.ipc_handle or self.ref_counter_handle or self.event_handle):
            raise ValueError("verbs allocation cannot carry a CUDA IPC handle")

    def to_bytes(self) -> bytes:
        head = self._HEADER.pack(
            self.abi_version, int(self.provider), self._STRICT if self.strictly_ordered else 0,
            self.peer, self.device, self.generation, self.address, self.allocation_length,
            self.allocation_size, self.mapping_offset, self.offset, self.length, self.rkey,
            len(self.ipc_handle), len(self.ref_counter_handle), len(self.event_handle),
            self.ref_counter_offset, int(self.event_sync_required))
        return head + self.ipc_handle + self.ref_counter_handle + self.event_handle

    @classmethod
    def from_bytes(cls, data: bytes) -> "AllocationHandle":
        if len(data) < cls._HEADER.size:
            raise ValueError("invalid Aboleth allocation-handle size")
        (abi_version, provider, flags, peer, device, generation, address, allocation_length,
         allocation_size, mapping_offset, offset, length, rkey, n_ipc, n_ref, n_event,
         ref_counter_offset, event_sync) = cls._HEADER.unpack_from(data)
        if len(data) != cls._HEADER.size + n_ipc + n_ref + n_event:
            raise ValueError("invalid Aboleth allocation payload size")
        at = cls._HEADER.size
        ipc = bytes(data[at:at + n_ipc])
        ref = bytes(data[at + n_ipc:at + n_ipc + n_ref])
        event = bytes(data[at + n_ipc + n_ref:at + n_ipc + n_ref + n_event])
        provider = AllocationProvider(provider)
        mapped = provider in (AllocationProvider.CUDA_IPC, AllocationProvider.HOST_SHM)
        return cls(provider=provider, peer=peer, device=device, generation=generation,
                   address=address, allocation_length=allocation_length,
                   allocation_size=allocation_size, mapping_offset=mapping_offset, offset=offset,
                   length=length, rkey=rkey, ipc_handle=ipc if mapped else b"",
                   ref_counter_handle=ref if mapped else b"",
                   ref_counter_offset=ref_counter_offset, event_handle=event if mapped else b"",
                   event_sync_required=bool(event_sync),
                   strictly_ordered=bool(flags & cls._STRICT), abi_version=abi_version)


def _check_slice(total: int, offset: int, length: int) -> None:
    if offset < 0 or length < 0 or offset + length > total:
        raise ValueError(f"slice [{offset}, {offset + length}) is outside a {total}-byte buffer")


# ---- memory backends -----------------------------------------------------------------


class _CudaMemory:
    """CUDA IPC through the native runtime."""

    provider = AllocationProvider.CUDA_IPC

    def export(self, address: int) -> tuple[bytes, int, int]:
        handle = ctypes.create_string_buffer(64)
        base, size = ctypes.c_uint64(), ctypes.c_uint64()
        if _lib().ab200_ipc_export(ctypes.c_void_p(address), handle, ctypes.byref(base),
                                   ctypes.byref(size)) != 0:
            raise RuntimeError(f"cannot export CUDA allocation: {last_error()}")
        return handle.raw, base.value, size.value

    def open(self, handle: bytes) -> tuple[int, object]:
        mapped = ctypes.c_void_p()
        if _lib().ab200_ipc_open(handle, ctypes.byref(mapped)) != 0:
            raise RuntimeError(f"cannot import CUDA allocation: {last_error()}")
        return int(mapped.value), None

    def close(self, base: int, keep: object) -> None:
        _lib().ab200_ipc_close(ctypes.c_void_p(base))


class _HostMemory:
    """POSIX shared memory for CPU-only ranks.

    Only tensors created by :meth:`Runtime.allocate` can be exported: the
    handle is the segment's name.
    """

    provider = AllocationProvider.HOST_SHM
    _segments: dict[int, tuple[shared_memory.SharedMemory, int]] = {}
    _lock = threading.Lock()

    @classmethod
    def allocate(cls, nbytes: int) -> torch.Tensor:
        shm = shared_memory.SharedMemory(create=True, size=max(int(nbytes), 1))
        tensor = torch.frombuffer(shm.buf, dtype=torch.uint8, count=int(nbytes))
        with cls._lock:
            cls._segments[tensor.data_ptr()] = (shm, int(nbytes))
        return tensor

    def export(self, address: int) -> tuple[bytes, int, int]:
        with self._lock:
            for base, (shm, size) in self._segments.items():
                if base <= address < base + max(size, 1):
                    return shm.name.encode().ljust(64, b"\0"), base, size
        raise RuntimeError("a cpu runtime can only export tensors made by Runtime.allocate()")

    def open(self, handle: bytes) -> tuple[int, object]:
        shm = shared_memory.SharedMemory(name=handle.rstrip(b"\0").decode())
        view = torch.frombuffer(shm.buf, dtype=torch.uint8, count=shm.size)
        return view.data_ptr(), (shm, view)

    def close(self, base: int, keep: object) -> None:
        if keep is not None:
            shm, view = keep
            del view
            try:
                shm.close()
            except BufferError:
                pass

    @classmethod
    def release(cls, tensor: torch.Tensor) -> None:
        with cls._lock:
            entry = cls._segments.pop(tensor.data_ptr(), None)
        if entry is not None:
            shm, _ = entry
            try:
                shm.close()
            except BufferError:
                pass
            try:
                shm.unlink()
            except FileNotFoundError:
                pass


# ---- buffers -----------------------------------------------------------------------------


class RegisteredBuffer:
    """A tensor entered in the runtime's key table.  Keeps the tensor alive."""

    def __init__(self, runtime: "Runtime", tensor: torch.Tensor, native, generation: int):
        self._runtime = runtime
        self._tensor = tensor
        self._native = native
        self._generation = generation
        self._closed = False

    @property
    def tensor(self) -> torch.Tensor:
        return self._tensor

    @property
    def address(self) -> int:
        return int(self._tensor.data_ptr())

    @property
    def length(self) -> int:
        return int(self._tensor.numel() * self._tensor.element_size())

    @property
    def device(self) -> int:
        return self._runtime.device_index

    @property
    def generation(self) -> int:
        return self._generation

    @property
    def lkey(self) -> int:
        self._ensure_open()
        return int(_lib().aboleth_runtime_buffer_lkey(self._native))

    @property
    def rkey(self) -> int:
        self._ensure_open()
        return int(_lib().aboleth_runtime_buffer_rkey(self._native))

    @property
    def strictly_ordered(self) -> bool:
        return True

    def export(self, peer: int) -> RemoteHandle:
        """The (address, rkey) record a queue-transport peer needs."""
        self._ensure_open()
        return RemoteHandle(self.address, self.length, self.rkey, int(peer), self._generation)

    def export_allocation(self, peer: int, *, offset: int = 0, length: Optional[int] = None,
                          mapped: bool = True) -> AllocationHandle:
        """Describe ``[offset, offset+length)`` so that ``peer`` can map it."""
        self._ensure_open()
        length = self.length - offset if length is None else int(length)
        _check_slice(self.length, offset, length)
        if not mapped:
            return AllocationHandle(
                provider=AllocationProvider.IB_VERBS, peer=int(peer), device=self.device,
                generation=self._generation, address=self.address, allocation_length=self.length,
                allocation_size=self.length, mapping_offset=0, offset=offset, length=length,
                rkey=self.rkey, strictly_ordered=True)
        handle, base, size = self._runtime._memory.export(self.address)
        return AllocationHandle(
            provider=self._runtime._memory.provider, peer=int(peer), device=self.device,
            generation=self._generation, address=self.address, allocation_length=self.length,
            allocation_size=size, mapping_offset=self.address - base, offset=offset, length=length,
            rkey=0 if self._runtime._memory.provider == AllocationProvider.CUDA_IPC else self.rkey,
            ipc_handle=handle, strictly_ordered=True)

    def _ensure_open(self) -> None:
        if self._closed:
            raise RuntimeError("registered buffer is closed")

    def close(self) -> None:
        if self._closed:
            return
        self._closed = True
        _lib().aboleth_runtime_unregister_buffer(self._native)
        self._runtime._buffers.discard(self)


@dataclass(frozen=True)
class LocalBuffer:
    address: int
    length: int
    lkey: int
    owner: RegisteredBuffer

    def slice(self, offset: int, length: int) -> "LocalBuffer":
        _check_slice(self.length, offset, length)
        return LocalBuffer(self.address + offset, length, self.lkey, self.owner)


class ImportedAllocation:
    """One mapping of a peer's allocation, shared by every region cut from it."""

    def __init__(self, runtime: "Runtime", key: tuple, base: int, keep: object, generation: int):
        self._runtime = runtime
        self._key = key
        self.base = base
        self._keep = keep
        self.generation = generation
        self.refs = 0
        self._closed = False

    @property
    def closed(self) -> bool:
        return self._closed

    def ensure_open(self) -> None:
        if self._closed:
            raise RuntimeError("imported allocation is closed")

    def close(self) -> None:
        if not self._closed:
            self._closed = True
            self._runtime._memory.close(self.base, self._keep)


@dataclass(frozen=True)
class RemoteBuffer:
    address: int
    length: int
    rkey: int
    peer: int
    generation: int
    mapping: Optional[ImportedAllocation] = None

    def slice(self, offset: int, length: int) -> "RemoteBuffer":
        _check_slice(self.length, offset, length)
        return RemoteBuffer(self.address + offset, length, self.rkey, self.peer, self.generation,
                            self.mapping)

    def export(self) -> RemoteHandle:
        return RemoteHandle(self.address, self.length, self.rkey, self.peer, self.generation)

    def ensure_open(self) -> None:
        if self.mapping is not None:
            self.mapping.ensure_open()

    def close(self) -> None:
        if self.mapping is not None:
            self.mapping._runtime._release_import(self.mapping)


# ---- endpoints ----------------------------------------------------------------------------


class LocalEndpoint:
    """This rank's end of one connection to one peer."""

    def __init__(self, runtime: "Runtime", transport: Transport, descriptor: torch.Tensor,
                 native=None):
        self._runtime = runtime
        self._transport = transport
        self._descriptor = descriptor
        self._native = native
        self._peer: Optional[int] = None
        self._peer_device: Optional[int] = None
        self._closed = False
        kind = KIND_BITS[transport.value] if transport == Transport.P2P else KIND_BITS["proxy"]
        self._handle = int(descriptor.data_ptr()) | kind

    @property
    def device(self) -> int:
        return self._runtime.device_index

    @property
    def peer(self) -> Optional[int]:
        return self._peer

    @property
    def transport(self) -> Transport:
        return self._transport

    @property
    def handle(self) -> int:
        """The 64-bit device handle: descriptor address with the kind bits set."""
        return self._handle

    @property
    def device_handle(self) -> torch.Tensor:
        return torch.tensor([self._handle - (1 << 64) if self._handle >= (1 << 63) else self._handle],
                            dtype=torch.int64, device=self._descriptor.device)

    @property
    def connection_info(self) -> ConnectionInfo:
        self._ensure_open()
        if self._native is None:
            raise RuntimeError("a P2P endpoint has no native connection info")
        info = ConnectionInfo()
        if _lib().aboleth_runtime_local_endpoint_connection_info(self._native, ctypes.byref(info)):
            raise RuntimeError(last_error())
        return info

    def connect(self, peer: int, info: ConnectionInfo) -> None:
        self._ensure_open()
        if self._native is None:
            raise RuntimeError("connect() is for queue transports; use connect_p2p()")
        if _lib().aboleth_runtime_connect_local_endpoint(self._native, ctypes.byref(info)):
            raise RuntimeError(f"cannot connect to rank {peer}: {last_error()}")
        self._peer = int(peer)

    def connect_p2p(self, peer: int, peer_device: int) -> None:
        self._ensure_open()
        if self._transport != Transport.P2P:
            raise RuntimeError("connect_p2p() is for P2P endpoints")
        self._runtime._enable_peer(peer_device)
        self._peer = int(peer)
        self._peer_device = int(peer_device)

    @property
    def capacity(self) -> int:
        if self._native is None:
            return 2 ** 31 - 1
        out = ctypes.c_uint32()
        _lib().aboleth_runtime_local_endpoint_capacity(self._native, ctypes.byref(out))
        return int(out.value)

    @property
    def max_inline_bytes(self) -> int:
        if self._native is None:
            return 0
        out = ctypes.c_uint32()
        _lib().aboleth_runtime_local_endpoint_max_inline(self._native, ctypes.byref(out))
        return int(out.value)

    @property
    def submit_mode(self) -> str:
        if self._native is None:
            return "direct"
        out = ctypes.c_uint32()
        _lib().aboleth_runtime_local_endpoint_submit_mode(self._native, ctypes.byref(out))
        return {0: "direct", 1: "staged", 2: "proxy"}[int(out.value)]

    @property
    def gpu_resident_queues(self) -> bool:
        return False

    def state(self) -> tuple[int, int, int]:
        """(reserved, retired, status) of the endpoint's ring; zeros for P2P."""
        if self._native is None:
            return (0, 0, 0)
        a, b, c = ctypes.c_uint64(), ctypes.c_uint64(), ctypes.c_uint64()
        if _lib().aboleth_runtime_local_endpoint_state(self._native, ctypes.byref(a),
                                                       ctypes.byref(b), ctypes.byref(c)):
            raise RuntimeError(last_error())
        return int(a.value), int(b.value), int(c.value)

    def descriptor(self) -> ProxyEndpointDescriptor:
        """Host copy of the ring descriptor (queue transports only)."""
        if self._native is None:
            raise RuntimeError("a P2P endpoint has no ring descriptor")
        out = ProxyEndpointDescriptor()
        _lib().ab200_endpoint_descriptor(self._native, ctypes.byref(out))
        return out

    def inject_failure(self, status: int, batches: int = 1) -> None:
        """Host-side fault injection: the next batches retire with ``status``."""
        if self._native is None:
            raise RuntimeError("a P2P endpoint has no ring to fail")
        _lib().ab200_endpoint_inject_failure(self._native, int(status), int(batches))

    def stats(self) -> dict[str, int]:
        if self._native is None:
            return {"batches": 0, "commands": 0, "bytes": 0, "signals": 0}
        words = (ctypes.c_uint64 * 4)()
        _lib().ab200_endpoint_stats(self._native, words)
        return dict(zip(("batches", "commands", "bytes", "signals"), map(int, words)))

    def snapshot_queue(self, first: int = 0, batches: Optional[int] = None) -> list[list[bytes]]:
        """The commands of retired batches ``first .. first + batches`` exactly as their producer
        wrote them into the ring: one list of 32-byte command images per batch.  For differential
        tests (two producers that should put the same bytes on the wire); the ring keeps the last
        64 batches."""
        self._ensure_open()
        if batches is None:
            batches = self.state()[1] - first
        room = batches * (4 + 256 * 32)
        buffer = (ctypes.c_ubyte * max(room, 4))()
        used = _lib().ab200_endpoint_snapshot(self._native, int(first), int(batches), buffer, room)
        if used < 0:
            raise RuntimeError(f"queue snapshot failed: {last_error()}")
        raw, out, at = bytes(buffer[:used]), [], 0
        for _ in range(batches):
            count = int.from_bytes(raw[at:at + 4], "little")
            at += 4
            out.append([raw[at + 32 * k:at + 32 * (k + 1)] for k in range(count)])
            at += 32 * count
        return out

    def local_buffer(self, buffer: RegisteredBuffer, offset: int = 0,
                     length: Optional[int] = None) -> LocalBuffer:
        length = buffer.length - offset if length is None else length
        _check_slice(buffer.length, offset, length)
        return LocalBuffer(buffer.address + offset, length, buffer.lkey, buffer)

    def import_remote(self, handle) -> RemoteBuffer:
        if isinstance(handle, AllocationHandle):
            return self._runtime.import_remote_buffer(handle)
        return RemoteBuffer(handle.address, handle.length, handle.rkey, handle.peer,
                            handle.generation)

    def _ensure_open(self) -> None:
        if self._closed:
            raise RuntimeError("endpoint is closed")

    def close(self) -> None:
        if self._closed:
            return
        self._closed = True
        if self._native is not None:
            _lib().aboleth_runtime_destroy_local_endpoint(self._native)
            self._native = None
        self._runtime._endpoints.discard(self)

    def __enter__(self) -> "LocalEndpoint":
        return self

    def __exit__(self, *exc) -> None:
        self.close()


Endpoint = LocalEndpoint


class EndpointTable:
    """Device table of endpoint handles indexed by peer (self = 0)."""

    def __init__(self, device, endpoints: dict[int, LocalEndpoint], world_size: int):
        self._endpoints = dict(endpoints)
        values = [0] * world_size
        for peer, endpoint in self._endpoints.items():
            values[peer] = endpoint.handle
        signed = [v - (1 << 64) if v >= (1 << 63) else v for v in values]
        self._handles = torch.tensor(signed, dtype=torch.int64, device=device)

    @property
    def device_handles(self) -> torch.Tensor:
        return self._handles

    @property
    def peers(self) -> tuple[int, ...]:
        return tuple(sorted(self._endpoints))

    def endpoint(self, peer: int) -> LocalEndpoint:
        try:
            return self._endpoints[peer]
        except KeyError as error:
            raise KeyError(f"no endpoint to rank {peer}") from error


class EndpointPair:
    """Both ends of one connection inside a single process (one runtime per end)."""

    def __init__(self, transport: Transport, first: "Runtime", second: "Runtime",
                 ids: tuple[int, int]):
        self._transport = Transport(transport)
        a = first.create_local_endpoint(self._transport)
        b = second.create_local_endpoint(self._transport)
        try:
            if self._transport == Transport.P2P:
                a.connect_p2p(ids[1], second.device_index)
                b.connect_p2p(ids[0], first.device_index)
            else:
                info_a, info_b = a.connection_info, b.connection_info
                a.connect(ids[1], info_b)
                b.connect(ids[0], info_a)
        except Exception:
            a.close()
            b.close()
            raise
        self.ids = ids
        self.endpoints = (a, b)
        self._closed = False

    @property
    def transport(self) -> Transport:
        return self._transport

    def close(self) -> None:
        if self._closed:
            return
        for endpoint in reversed(self.endpoints):
            endpoint.close()
        self._closed = True


class EndpointMesh:
    """Every pair of a set of same-process participants connected, with one table per participant.

    ``runtimes`` maps a participant id (a device ordinal, or any small integer for CPU
    runtimes) to its :class:`Runtime`.  Reference: python/aboleth/runtime.py:1020-1165 (pair),
    1168-1231 (mesh); there the runtime is per process and spans devices, here it is per device.
    """

    def __init__(self, runtimes: Mapping[int, "Runtime"], transport: Transport = Transport.P2P):
        self._runtimes = dict(runtimes)
        ids = sorted(self._runtimes)
        if len(ids) < 2:
            raise ValueError("an endpoint mesh needs at least two participants")
        self._pairs: list[EndpointPair] = []
        endpoints: dict[int, dict[int, LocalEndpoint]] = {i: {} for i in ids}
        try:
            for n, first in enumerate(ids):
                for second in ids[n + 1:]:
                    pair = EndpointPair(transport, self._runtimes[first], self._runtimes[second],
                                        (first, second))
                    self._pairs.append(pair)
                    endpoints[first][second], endpoints[second][first] = pair.endpoints
        except Exception:
            for pair in reversed(self._pairs):
                pair.close()
            raise
        size = max(ids) + 1
        self.tables = {i: EndpointTable(self._runtimes[i].torch_device, endpoints[i], size) for i in ids}
        self._closed = False

    def _ensure_open(self) -> None:
        if self._closed:
            raise RuntimeError("Aboleth endpoint mesh is closed")

    def runtime(self, participant: int) -> "Runtime":
        return self._runtimes[participant]

    def endpoint(self, participant: int, peer: int) -> LocalEndpoint:
        self._ensure_open()
        return self.tables[participant].endpoint(peer)

    @property
    def pairs(self) -> tuple[EndpointPair, ...]:
        self._ensure_open()
        return tuple(self._pairs)

    def close(self) -> None:
        if self._closed:
            return
        for pair in reversed(self._pairs):
            pair.close()
        self._closed = True

    def __enter__(self) -> "EndpointMesh":
        self._ensure_open()
        return self

    def __exit__(self, exc_type, exc_value, traceback) -> None:
        try:
            self.close()
        except Exception as cleanup_error:  # keep the original error first
            if exc_value is None:
                raise
            exc_value.add_note(f"Aboleth endpoint-mesh cleanup also failed: {cleanup_error}")


class Runtime:
    """Owns this rank's registrations, endpoints and imported mappings."""

    def __init__(self, device=None):
        if device is None:
            device = torch.cuda.current_device() if torch.cuda.is_available() else "cpu"
        if isinstance(device, torch.device):
            device = device.index if device.type == "cuda" else "cpu"
        self._cpu = device == "cpu"
        self.device_index = 0 if self._cpu else int(device)
        self.torch_device = torch.device("cpu") if self._cpu else torch.device("cuda", self.device_index)
        self._memory = _HostMemory() if self._cpu else _CudaMemory()
        self._native = _lib().aboleth_runtime_create_for_device(
            -1 if self._cpu else self.device_index, None)
        if not self._native:
            raise RuntimeError(f"cannot create runtime: {last_error()}")
        self._buffers: set[RegisteredBuffer] = set()
        self._endpoints: set[LocalEndpoint] = set()
        self._imports: dict[tuple, ImportedAllocation] = {}
        self._generation = 0
        self._peers_enabled: set[int] = set()
        self._owned: list[torch.Tensor] = []
        self._closed = False

    # -- properties kept for API parity; there is no adapter behind them --
    @property
    def device(self) -> Optional[int]:
        return None if self._cpu else self.device_index

    @property
    def hca(self) -> str:
        return ""

    @property
    def rdma_port(self) -> int:
        return 0

    @property
    def gid_index(self) -> int:
        return -1

    @property
    def lid(self) -> int:
        return 0

    @property
    def link_layer(self) -> str:
        return "none"

    def allocate(self, nbytes: int) -> torch.Tensor:
        """A zeroed byte tensor that this runtime can export to peers."""
        if self._cpu:
            tensor = _HostMemory.allocate(nbytes)
            tensor.zero_()
        else:
            tensor = torch.zeros(int(nbytes), dtype=torch.uint8, device=self.torch_device)
        self._owned.append(tensor)
        return tensor

    def register(self, tensor: torch.Tensor, *, network: bool = True) -> RegisteredBuffer:
        """Enter ``tensor`` in the key table.  ``network`` is accepted for API
        parity; there is no adapter to pin memory with."""
        self._ensure_open()
        if not tensor.is_contiguous():
            raise ValueError("only contiguous tensors can be registered")
        if self._cpu != (tensor.device.type == "cpu"):
            raise ValueError(f"tensor lives on {tensor.device}, runtime on {self.torch_device}")
        if not self._cpu and tensor.device.index != self.device_index:
            raise ValueError(f"tensor lives on {tensor.device}, runtime on {self.torch_device}")
        nbytes = tensor.numel() * tensor.element_size()
        if nbytes == 0:
            raise ValueError("cannot register an empty tensor")
        self._generation += 1
        native = _lib().aboleth_runtime_register_buffer(
            self._native, -1 if self._cpu else self.device_index,
            ctypes.c_void_p(tensor.data_ptr()), nbytes, self._generation)
        if not native:
            raise RuntimeError(f"cannot register buffer: {last_error()}")
        buffer = RegisteredBuffer(self, tensor, native, self._generation)
        self._buffers.add(buffer)
        return buffer

    def create_local_endpoint(self, transport: Transport = Transport.P2P, *,
                              config: Optional[EndpointConfig] = None) -> LocalEndpoint:
        self._ensure_open()
        transport = Transport(transport)
        if transport == Transport.P2P:
            descriptor = torch.zeros(8, dtype=torch.uint8, device=self.torch_device)[:1]
            endpoint = LocalEndpoint(self, transport, descriptor)
        else:
            descriptor = torch.zeros(ctypes.sizeof(ProxyEndpointDescriptor), dtype=torch.uint8,
                                     device=self.torch_device)
            native = _lib().aboleth_runtime_create_local_endpoint(
                self._native, _NATIVE_TRANSPORT[transport], -1 if self._cpu else self.device_index,
                ctypes.c_void_p(descriptor.data_ptr()), descriptor.numel(),
                ctypes.byref(config) if config is not None else None)
            if not native:
                raise RuntimeError(f"cannot create {transport.value} endpoint: {last_error()}")
            endpoint = LocalEndpoint(self, transport, descriptor, native)
        self._endpoints.add(endpoint)
        return endpoint

    def export_buffer(self, buffer: RegisteredBuffer, peer: int) -> RemoteHandle:
        return buffer.export(peer)

    def export_allocation(self, buffer: RegisteredBuffer, peer: int, **kwargs) -> AllocationHandle:
        return buffer.export_allocation(peer, **kwargs)

    def import_remote_buffer(self, handle: AllocationHandle, *,
                             same_process_address: Optional[int] = None) -> RemoteBuffer:
        """Make a peer's exported slice addressable from this rank.

        Mappings are cached per (exporting device, handle bytes) and reference
        counted; a handle whose generation is older than one already seen for
        the same allocation is refused, because it describes memory the peer
        has since re-registered.
        """
        self._ensure_open()
        if handle.provider == AllocationProvider.IB_VERBS:
            return RemoteBuffer(handle.address + handle.offset, handle.length, handle.rkey,
                                handle.peer, handle.generation)
        if handle.provider not in (AllocationProvider.CUDA_IPC, AllocationProvider.HOST_SHM):
            raise ValueError(f"allocation provider {handle.provider!r} cannot be imported")
        if same_process_address is not None:
            base = same_process_address - handle.mapping_offset
            return RemoteBuffer(base + handle.mapping_offset + handle.offset, handle.length,
                                handle.rkey, handle.peer, handle.generation)
        key = (self.device_index, handle.device, handle.ipc_handle)
        entry = self._imports.get(key)
        if entry is not None and not entry.closed:
            if handle.generation < entry.generation:
                raise RuntimeError(
                    f"stale allocation handle from rank {handle.peer}: generation "
                    f"{handle.generation} < {entry.generation}")
            entry.generation = max(entry.generation, handle.generation)
        else:
            if not self._cpu:
                self._enable_peer(handle.device)
            base, keep = self._memory.open(handle.ipc_handle)
            entry = ImportedAllocation(self, key, base, keep, handle.generation)
            self._imports[key] = entry
        entry.refs += 1
        return RemoteBuffer(entry.base + handle.mapping_offset + handle.offset, handle.length,
                            handle.rkey, handle.peer, handle.generation, entry)

    def _release_import(self, entry: ImportedAllocation) -> None:
        entry.refs -= 1
        if entry.refs <= 0 and not entry.closed:
            entry.close()
            self._imports.pop(entry._key, None)

    def _enable_peer(self, peer_device: int) -> None:
        if self._cpu or peer_device == self.device_index or peer_device in self._peers_enabled:
            return
        # Other processes' devices are reached through IPC mappings, which
        # enable peer access lazily; this covers same-process peers too.
        if peer_device < torch.cuda.device_count():
            if _lib().ab200_enable_peer_access(self.device_index, peer_device) != 0:
                raise RuntimeError(last_error())
        self._peers_enabled.add(peer_device)

    def _ensure_open(self) -> None:
        if self._closed:
            raise RuntimeError("runtime is closed")

    def close(self) -> None:
        if self._closed:
            return
        for endpoint in list(self._endpoints):
            endpoint.close()
        for entry in list(self._imports.values()):
            entry.close()
        self._imports.clear()
        for buffer in list(self._buffers):
            buffer.close()
        if self._cpu:
            for tensor in self._owned:
                _HostMemory.release(tensor)
        self._owned.clear()
        _lib().aboleth_runtime_destroy(self._native)
        self._closed = True

    def __enter__(self) -> "Runtime":
        return self

    def __exit__(self, *exc) -> None:
        self.close()
