"""World bring-up among CPU ranks: topology, connections, regions, rollback.

CPU ranks use the cpu runtime (POSIX shared memory in place of CUDA IPC); the
peer-memory transport then means "map the peer's segment", so the same tables
and codecs are exercised as on GPUs.
"""
import struct

import pytest

from aboleth_b200 import (AutoTransportPolicy, TcpStoreBootstrap, TopologyInfo, Transport, World)
from aboleth_b200.bootstrap import encode_bundle
from aboleth_b200.world import _decode_connections, _decode_regions
from tests._ranks import run_ranks


def _world_rank(rank, world_size, transport, fan_out):
    boot = TcpStoreBootstrap.from_env(timeout=30)
    with World(rank, world_size, device="cpu", bootstrap=boot) as world:
        world.connect_all(transport, remote_transport="proxy", endpoints_per_peer=fan_out)
        arena = world.runtime.allocate(4096)
        reg = world.register(arena)
        recv = world.region("recv", reg, offset=0, length=2048)
        flags = world.region("flags", reg, offset=2048, length=64)
        table = world.exchange_regions([recv, flags], tag="t")
        # Write my rank into every peer's recv[rank] through the mapping.
        addresses = table.addresses("recv").tolist()
        import ctypes
        for peer in range(world_size):
            ctypes.c_uint8.from_address(addresses[peer] + rank).value = rank + 1
        boot.barrier("written")
        got = arena[:world_size].tolist()
        handles = table.endpoint_handles.tolist()
        regions = table.regions("flags").view(world_size, 2).tolist()
        boot.barrier("read")
        return {"got": got, "handles": handles, "regions": regions,
                "transport": world.transport.value, "geo": world.transport_geography,
                "flag_addr": flags.address, "kinds": [h & 7 for h in handles]}


@pytest.mark.parametrize("transport,kind", [("p2p", 1), ("auto", 1), ("proxy", 2)])
def test_world_exchange_three_cpu_ranks(transport, kind):
    world_size, fan_out = 3, 2
    results = run_ranks(_world_rank, world_size, transport, fan_out)
    assert all(k == "ok" for k, _ in results.values()), results
    for rank in range(world_size):
        out = results[rank][1]
        assert out["got"] == [1, 2, 3]
        assert len(out["handles"]) == world_size * fan_out
        for peer in range(world_size):
            for slot in range(fan_out):
                h = out["handles"][peer * fan_out + slot]
                assert (h == 0) if peer == rank else (h & 7) == kind
        assert out["regions"][rank][0] == out["flag_addr"]
        assert out["transport"] == ("p2p" if kind == 1 else "proxy")


def _two_node_rank(rank, world_size, transport):
    import os
    os.environ["ABOLETH_NODE_IDENTITY"] = f"node{rank // 2}:fake-boot-id"
    boot = TcpStoreBootstrap.from_env(timeout=30)
    with World(rank, world_size, device="cpu", bootstrap=boot) as world:
        try:
            world.connect_all(transport, remote_transport="proxy")
        except ValueError as error:
            boot.barrier("refused")  # rank 0 hosts the store: it stays until every rank has its answer
            return {"error": str(error)}
        arena = world.runtime.allocate(256)
        reg = world.register(arena)
        table = world.exchange_regions([world.region("recv", reg, offset=0, length=256)], tag="n")
        boot.barrier("imported")  # nobody unmaps its segment while a peer is still importing it
        return {"kinds": [h & 7 for h in table.endpoint_handles.tolist()], "geo": world.transport_geography,
                "transport": world.transport.value}


def test_two_fake_nodes_on_one_host_mix_transports():
    """Four ranks, two per "node": peer memory inside a node, the ring across nodes."""
    results = run_ranks(_two_node_rank, 4, "auto")
    assert all(k == "ok" for k, _ in results.values()), results
    for rank in range(4):
        kinds = results[rank][1]["kinds"]
        for peer in range(4):
            expected = 0 if peer == rank else (1 if peer // 2 == rank // 2 else 2)
            assert kinds[peer] == expected, (rank, kinds)
    # Asking for peer memory to a rank of another node is refused on every rank.
    refused = run_ranks(_two_node_rank, 4, "p2p")
    assert all(k == "ok" and "is not on the local node" in v["error"] for k, v in refused.values()), refused


def test_auto_policy_threshold():
    policy = AutoTransportPolicy()
    assert policy.select(can_p2p=True, payload_bytes=16 * 1024, remote_transport=Transport.RDMA) == Transport.P2P
    assert policy.select(can_p2p=True, payload_bytes=16 * 1024 + 1, remote_transport=Transport.RDMA) == Transport.RDMA
    assert policy.select(can_p2p=False, payload_bytes=8, remote_transport=Transport.PROXY) == Transport.PROXY
    assert policy.select(can_p2p=True, payload_bytes=None, remote_transport=Transport.PROXY) == Transport.P2P
    with pytest.raises(ValueError):
        policy.select(can_p2p=True, payload_bytes=1, remote_transport=Transport.EFA)
    with pytest.raises(ValueError):
        AutoTransportPolicy(-1)


def test_topology_codec_and_skew():
    info = TopologyInfo(2, 5, "node:abc")
    blob = info.to_bytes()
    assert TopologyInfo.from_bytes(blob) == info
    assert blob[:12] == struct.pack("<III", 2, 2, 1)
    with pytest.raises(ValueError, match="version 1"):
        TopologyInfo.from_bytes(encode_bundle(1, 2, [b"\0\0\0\0h"]))
    with pytest.raises(ValueError, match="hostname cannot be empty"):
        TopologyInfo.from_bytes(encode_bundle(2, 2, [b"\0\0\0\0"]))


def test_connection_codec_errors():
    good = struct.pack("<II", 1, 1) + struct.pack("<i", 3)
    rank, records = _decode_connections(encode_bundle(3, 0, [good]))
    assert rank == 0 and records[1].transport == Transport.P2P and records[1].device == 3
    with pytest.raises(ValueError, match="duplicate peer"):
        _decode_connections(encode_bundle(3, 0, [good, good]))
    with pytest.raises(ValueError, match="unknown connection transport 9"):
        _decode_connections(encode_bundle(3, 0, [struct.pack("<II", 1, 9)]))
    with pytest.raises(ValueError, match="invalid P2P connection-info size"):
        _decode_connections(encode_bundle(3, 0, [struct.pack("<II", 1, 1) + b"xx"]))


def test_region_codec_filters_by_target():
    from aboleth_b200.runtime import AllocationHandle, AllocationProvider
    handle = AllocationHandle(provider=AllocationProvider.IB_VERBS, peer=1, device=0, generation=1,
                              address=64, allocation_length=64, allocation_size=64,
                              mapping_offset=0, offset=0, length=64, rkey=7).to_bytes()
    rec = lambda target, name: struct.pack("<IH", target, len(name)) + name + handle  # noqa: E731
    blob = encode_bundle(3, 1, [rec(0, b"a"), rec(2, b"a"), rec(0, b"b")])
    rank, regions = _decode_regions(blob, target_rank=0)
    assert rank == 1 and sorted(regions) == ["a", "b"] and regions["a"].rkey == 7
    with pytest.raises(ValueError, match="duplicate targeted region"):
        _decode_regions(encode_bundle(3, 1, [rec(0, b"a"), rec(0, b"a")]), target_rank=0)


def _asymmetric(rank, world_size):
    boot = TcpStoreBootstrap.from_env(timeout=30)
    world = World(rank, world_size, device="cpu", bootstrap=boot)
    try:
        world.connect_all("p2p" if rank == 0 else "proxy", remote_transport="proxy")
    except RuntimeError as error:
        live = len(world.runtime._endpoints)
        world.close()
        if rank == 0:
            import time
            time.sleep(2.0)  # rank 0 hosts the store: outlive the peers' last read
        return str(error), live
    return "connected", -1


def test_asymmetric_transport_choice_rolls_back():
    results = run_ranks(_asymmetric, 2)
    for rank in range(2):
        kind, (message, live) = results[rank]
        assert kind == "ok" and "asymmetric" in message and live == 0


def test_single_rank_world_and_validation():
    with World(0, 1, device="cpu") as world:
        world.connect_all("p2p")
        arena = world.runtime.allocate(256)
        reg = world.register(arena)
        table = world.exchange_regions([world.region("x", reg)], tag="solo")
        assert table.addresses("x").tolist() == [arena.data_ptr()]
        assert table.endpoint_handles.tolist() == [0]
        with pytest.raises(ValueError, match="outside its registration"):
            world.region("bad", reg, offset=200, length=100)
        with pytest.raises(ValueError, match="cannot be empty"):
            world.region("", reg)
        with pytest.raises(RuntimeError, match="already connected"):
            world.connect_all("p2p")
    with pytest.raises(ValueError, match="bootstrap is required"):
        World(0, 2, device="cpu")


def test_symmetric_arena_needs_a_process_group_and_reports_no_multicast_without_a_gpu():
    import pytest
    import torch

    from aboleth_b200.symmetric import SymmetricArena, multicast_supported

    assert multicast_supported() is False or torch.cuda.is_available()
    with pytest.raises(RuntimeError, match="process group"):
        SymmetricArena(1024, torch.device("cpu"))
