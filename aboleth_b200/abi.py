"""Python mirrors of the C ABI records in ``include/aboleth/abi``.

Three different numberings name a transport and must never be mixed
(reference: docs/TIERS.md:62-64):

* ``KIND_BITS``  - low three bits of a device endpoint handle
  (rdma 0, p2p 1, proxy 2, efa 3, ionic 4; python/aboleth/world.py:431-437);
* ``WIRE_CODES`` - what a connection bundle carries between ranks
  (p2p 1, rdma 2, proxy 3, efa 4, ionic 5; python/aboleth/world.py:45-51);
* native connection codes - ``AbolethConnectionInfo.transport``
  (direct 1, proxy 2, efa 3, ionic 4; python/aboleth/runtime.py:89-94).
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass

KIND_MASK = 7
KIND_BITS = {"rdma": 0, "p2p": 1, "proxy": 2, "efa": 3, "ionic": 4}
WIRE_CODES = {"p2p": 1, "rdma": 2, "proxy": 3, "efa": 4, "ionic": 5}

PROVIDER_VERBS = 1 << 0
PROVIDER_MLX5 = 1 << 1
PROVIDER_EFA = 1 << 2
PROVIDER_LIBFABRIC = 1 << 3
PROVIDER_CUDA = 1 << 4
PROVIDER_HIP = 1 << 5
PROVIDER_IONIC = 1 << 6

CONNECTION_INFO_VERSION = 2
PROXY_ENDPOINT_VERSION = 8
PROXY_SLOT_COUNT = 64
PROXY_MAXIMUM_COMMANDS = 256
PROXY_NOP, PROXY_WRITE, PROXY_WEAK_SIGNAL, PROXY_STRONG_SIGNAL = 0, 1, 2, 3
STATUS_OK, STATUS_TIMEOUT, STATUS_COMPLETION_FAILURE, STATUS_MALFORMED = 0, 1, 2, 3
TRANSPORT_PHASE_PLAN_VERSION = 4
TIER1_ABI = 2


class ConnectionInfo(ctypes.Structure):
    """128-byte ``AbolethConnectionInfo``."""

    _fields_ = [
        ("abi_version", ctypes.c_uint32), ("transport", ctypes.c_uint32),
        ("qpn", ctypes.c_uint32), ("psn", ctypes.c_uint32),
        ("gid_index", ctypes.c_uint32), ("path_mtu", ctypes.c_uint32),
        ("lid", ctypes.c_uint16), ("port_num", ctypes.c_uint8), ("link_layer", ctypes.c_uint8),
        ("gid", ctypes.c_uint8 * 16),
        ("provider", ctypes.c_uint32), ("address_format", ctypes.c_uint32),
        ("address_length", ctypes.c_uint32), ("reserved0", ctypes.c_uint32),
        ("address", ctypes.c_uint8 * 64), ("reserved", ctypes.c_uint8 * 4),
    ]

    def to_bytes(self) -> bytes:
        return bytes(self)

    @classmethod
    def from_bytes(cls, data: bytes) -> "ConnectionInfo":
        if len(data) != ctypes.sizeof(cls):
            raise ValueError(
                f"an Aboleth connection info is {ctypes.sizeof(cls)} bytes, got {len(data)}")
        info = cls.from_buffer_copy(data)
        if info.abi_version != CONNECTION_INFO_VERSION:
            raise ValueError(
                f"unsupported Aboleth connection-info version {info.abi_version}: this rank "
                f"speaks version {CONNECTION_INFO_VERSION}")
        return info


class EndpointConfig(ctypes.Structure):
    """96-byte ``AbolethEndpointConfig``; ``struct_size`` versions it."""

    _fields_ = [
        ("struct_size", ctypes.c_uint32), ("qp_type", ctypes.c_uint32),
        ("qp_depth", ctypes.c_uint32), ("max_inline", ctypes.c_uint32),
        ("qps_per_peer", ctypes.c_uint32), ("sm_map_policy", ctypes.c_uint32),
        ("port", ctypes.c_int32), ("gid_index", ctypes.c_int32),
        ("hca", ctypes.c_char * 64),
    ]

    def __init__(self, **kwargs):
        super().__init__()
        self.struct_size = ctypes.sizeof(EndpointConfig)
        self.gid_index = -1
        for key, value in kwargs.items():
            setattr(self, key, value)


class ProxyCommand(ctypes.Structure):
    _fields_ = [
        ("source_address", ctypes.c_uint64), ("destination_address", ctypes.c_uint64),
        ("bytes", ctypes.c_uint32), ("source_key", ctypes.c_uint32),
        ("destination_key", ctypes.c_uint32), ("opcode", ctypes.c_uint32),
    ]


class ProxyBatchSlot(ctypes.Structure):
    _fields_ = [
        ("ready_sequence", ctypes.c_uint64), ("command_count", ctypes.c_uint32),
        ("reserved", ctypes.c_uint32), ("commands", ProxyCommand * PROXY_MAXIMUM_COMMANDS),
    ]


class ProxyQueueState(ctypes.Structure):
    _fields_ = [
        ("completed_sequence", ctypes.c_uint64), ("status", ctypes.c_uint64),
        ("slots", ProxyBatchSlot * PROXY_SLOT_COUNT),
    ]


class ProxyEndpointDescriptor(ctypes.Structure):
    _fields_ = [
        ("queue_state", ctypes.c_uint64), ("producer_index_address", ctypes.c_uint64),
        ("completion_timeout_cycles", ctypes.c_uint64), ("slot_count", ctypes.c_uint32),
        ("slot_stride", ctypes.c_uint32), ("maximum_commands", ctypes.c_uint32),
        ("abi_version", ctypes.c_uint32),
    ]


class RdmaEndpointDescriptor(ctypes.Structure):
    _fields_ = [(name, ctypes.c_uint64) for name in (
        "send_queue", "send_dbrec", "blueflame", "completion_queue", "completion_dbrec",
        "producer_index_address", "completion_consumer_address", "completion_timeout_cycles")] + [
        (name, ctypes.c_uint32) for name in (
            "send_stride", "send_wqe_count", "qpn", "completion_entry_size",
            "completion_entry_count", "abi_version", "atomic_result_lkey", "reserved1")]


class PutDesc(ctypes.Structure):
    _fields_ = [("dst", ctypes.c_uint64), ("src", ctypes.c_uint64), ("bytes", ctypes.c_uint32),
                ("dst_key", ctypes.c_uint32), ("src_key", ctypes.c_uint32),
                ("pad", ctypes.c_uint32)]


class TransportPhasePlan(ctypes.Structure):
    _fields_ = [(name, ctypes.c_uint32) for name in (
        "abi_version", "byte_size", "active_qps", "data_qps", "data_wqe_bound",
        "data_reclaim_interval", "control_wqe_bound", "control_reclaim_interval", "topology_kind",
        "qp0_role", "publication_mode", "prologue_barrier_kind", "epilogue_barrier_kind", "flags",
        "publication_before_phase", "publication_iteration_delta", "completion_before_phase",
        "completion_iteration_delta", "first_overwrite_phase", "first_overwrite_iteration_delta",
        "reclaim_before_phase", "reclaim_iteration_delta", "payload_bytes", "path_mtu",
        "completion_interval", "buffer_slots", "payload_commit_tokens", "reserved")]


@dataclass(frozen=True)
class TransportCaps:
    name: str
    gpu_initiated: bool
    load_store_addressable: bool
    ordered_delivery: bool
    native_atomics: bool
    fenced_write: bool
    imm_data: bool
    queue_capacity_limited: bool
    selective_completion: bool
    max_inline_bytes: int
    default_completion_interval: int
    completion_model: int  # 0 none, 1 ordered counter, 2 unordered count
    doorbell_model: int    # 0 none, 1 blueflame, 2 host ring, 3 doorbell
    path_mtu: int
    max_data_queues: int


TRANSPORT_CAPS = {
    caps.name: caps for caps in (
        TransportCaps("p2p", True, True, True, True, False, False, False, True, 0, 0, 0, 0, 0, 0),
        TransportCaps("proxy", False, False, True, True, False, False, False, True, 8, 8, 1, 2, 4096, 0),
        TransportCaps("rdma", True, False, True, True, True, False, True, True, 28, 16, 1, 1, 4096, 0),
        TransportCaps("ionic", True, False, True, False, True, False, True, False, 16, 8, 1, 3, 4096, 0),
        TransportCaps("efa", True, False, False, False, False, True, True, False, 0, 16, 2, 3, 4096, 0),
    )
}

PUBLICATION_MODES = {
    "SameQueueStrong": 0, "P2PRelease": 1, "GinSignal": 2, "FenceThenSignal": 3,
    "ImmCounting": 4, "SameQueueFencedWrite": 5,
}


def legal_strong_publication(caps: TransportCaps, prefer_imm: bool = False,
                             strict_registrations: bool = False) -> str:
    """Python twin of ``legal_strong_publication`` in transport_plan.h."""
    if caps.load_store_addressable:
        return "P2PRelease"
    if not caps.ordered_delivery:
        return "ImmCounting" if prefer_imm and caps.imm_data else "FenceThenSignal"
    if strict_registrations and caps.fenced_write:
        return "SameQueueFencedWrite"
    return "SameQueueStrong" if caps.native_atomics else "FenceThenSignal"


def publication_is_checked(caps: TransportCaps) -> bool:
    return caps.native_atomics and not caps.load_store_addressable


assert ctypes.sizeof(ConnectionInfo) == 128
assert ctypes.sizeof(EndpointConfig) == 96
assert ctypes.sizeof(ProxyCommand) == 32
assert ctypes.sizeof(ProxyBatchSlot) == 8208
assert ctypes.sizeof(ProxyQueueState) == 525328
assert ctypes.sizeof(ProxyEndpointDescriptor) == 40
assert ctypes.sizeof(RdmaEndpointDescriptor) == 96
assert ctypes.sizeof(PutDesc) == 32
assert ctypes.sizeof(TransportPhasePlan) == 112
