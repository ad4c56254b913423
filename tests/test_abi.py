"""Layouts that must stay bit-identical to the reference ABI."""
import ctypes
import struct
import subprocess
from pathlib import Path

import pytest

from aboleth_b200 import abi
from aboleth_b200.runtime import AllocationHandle, AllocationProvider, RemoteHandle

INCLUDE = Path(abi.__file__).parent / "include"


def test_struct_sizes_and_offsets():
    assert ctypes.sizeof(abi.ConnectionInfo) == 128
    assert abi.ConnectionInfo.gid.offset == 28 and abi.ConnectionInfo.address.offset == 60
    assert ctypes.sizeof(abi.EndpointConfig) == 96 and abi.EndpointConfig.hca.offset == 32
    assert ctypes.sizeof(abi.ProxyCommand) == 32 and abi.ProxyCommand.opcode.offset == 28
    assert ctypes.sizeof(abi.ProxyBatchSlot) == 8208 and abi.ProxyBatchSlot.commands.offset == 16
    assert ctypes.sizeof(abi.ProxyQueueState) == 525328 and abi.ProxyQueueState.slots.offset == 16
    assert ctypes.sizeof(abi.ProxyEndpointDescriptor) == 40
    assert abi.ProxyEndpointDescriptor.abi_version.offset == 36
    assert ctypes.sizeof(abi.RdmaEndpointDescriptor) == 96
    assert abi.RdmaEndpointDescriptor.abi_version.offset == 84
    assert ctypes.sizeof(abi.TransportPhasePlan) == 112
    assert ctypes.sizeof(abi.PutDesc) == 32


def test_three_transport_numberings_are_distinct():
    assert abi.KIND_BITS == {"rdma": 0, "p2p": 1, "proxy": 2, "efa": 3, "ionic": 4}
    assert abi.WIRE_CODES == {"p2p": 1, "rdma": 2, "proxy": 3, "efa": 4, "ionic": 5}


def test_headers_compile_with_static_asserts(tmp_path):
    src = tmp_path / "t.cpp"
    src.write_text('#include "aboleth/abi/transport_plan.h"\n#include "aboleth/abi/proxy_abi.h"\n'
                   '#include "aboleth/abi/endpoint_abi.h"\nint main(){return 0;}\n')
    subprocess.run(["g++", "-std=c++17", f"-I{INCLUDE}", "-fsyntax-only", str(src)], check=True)


def test_caps_table_matches_header():
    text = (INCLUDE / "aboleth/abi/transport_caps.h").read_text()
    for name, caps in abi.TRANSPORT_CAPS.items():
        row = next(line for line in text.splitlines() if line.strip().startswith('{"%s"' % name))
        cells = [c.strip() for c in row.strip().strip("{},").split(",")]
        assert cells[9] == str(caps.max_inline_bytes) and cells[10] == str(caps.default_completion_interval)
        bools = [c == "true" for c in cells[1:9]]
        assert bools == [caps.gpu_initiated, caps.load_store_addressable, caps.ordered_delivery,
                         caps.native_atomics, caps.fenced_write, caps.imm_data,
                         caps.queue_capacity_limited, caps.selective_completion]


def test_publication_modes():
    c = abi.TRANSPORT_CAPS
    assert abi.legal_strong_publication(c["p2p"], True) == "P2PRelease"
    assert abi.legal_strong_publication(c["rdma"]) == "SameQueueStrong"
    assert abi.legal_strong_publication(c["rdma"], False, True) == "SameQueueFencedWrite"
    assert abi.legal_strong_publication(c["proxy"], False, True) == "SameQueueStrong"
    assert abi.legal_strong_publication(c["ionic"]) == "FenceThenSignal"
    assert abi.legal_strong_publication(c["efa"]) == "FenceThenSignal"
    assert abi.legal_strong_publication(c["efa"], True) == "ImmCounting"
    assert abi.publication_is_checked(c["rdma"]) and not abi.publication_is_checked(c["p2p"])


def test_remote_handle_wire():
    h = RemoteHandle(0x1122334455667788, 4096, 7, 3, 9)
    assert h.to_bytes() == struct.pack("<QQIIQ", 0x1122334455667788, 4096, 7, 3, 9)
    assert RemoteHandle.from_bytes(h.to_bytes()) == h
    with pytest.raises(ValueError):
        RemoteHandle.from_bytes(b"\0" * 5)


def test_allocation_handle_wire_and_validation():
    h = AllocationHandle(provider=AllocationProvider.CUDA_IPC, peer=1, device=2, generation=5,
                         address=0x7000, allocation_length=1024, allocation_size=4096,
                         mapping_offset=512, offset=64, length=128, ipc_handle=b"h" * 64,
                         strictly_ordered=True)
    blob = h.to_bytes()
    head = struct.Struct("<BBHIiQQQQQQQIHHHQB")
    assert len(blob) == head.size + 64
    fields = head.unpack_from(blob)
    assert fields[:6] == (2, 2, 1, 1, 2, 5) and fields[13] == 64
    assert AllocationHandle.from_bytes(blob) == h
    with pytest.raises(ValueError, match="payload size"):
        AllocationHandle.from_bytes(blob + b"x")
    with pytest.raises(ValueError, match="outside its allocation"):
        AllocationHandle(provider=AllocationProvider.CUDA_IPC, peer=0, device=0, generation=0,
                         address=0, allocation_length=10, allocation_size=10, mapping_offset=0,
                         offset=8, length=8, ipc_handle=b"x")
    with pytest.raises(ValueError, match="cannot carry an rkey"):
        AllocationHandle(provider=AllocationProvider.CUDA_IPC, peer=0, device=0, generation=0,
                         address=0, allocation_length=10, allocation_size=10, mapping_offset=0,
                         offset=0, length=8, ipc_handle=b"x", rkey=4)
    with pytest.raises(ValueError, match="version"):
        AllocationHandle(provider=AllocationProvider.IB_VERBS, peer=0, device=0, generation=0,
                         address=0, allocation_length=10, allocation_size=10, mapping_offset=0,
                         offset=0, length=8, abi_version=1)


def test_connection_info_version_skew():
    info = abi.ConnectionInfo()
    info.abi_version = 1
    with pytest.raises(ValueError, match="version 1"):
        abi.ConnectionInfo.from_bytes(bytes(info))
    with pytest.raises(ValueError, match="128 bytes"):
        abi.ConnectionInfo.from_bytes(b"\0" * 64)
