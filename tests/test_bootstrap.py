"""Bundle framing and the three bootstrap carriers (CPU only).

Strategy follows the reference's test/python/test_bootstrap.py: real TCPStore on
127.0.0.1 with multiprocessing ranks; a missing peer times out; framing errors
are reported by kind.
"""
import multiprocessing as mp
import struct
import threading

import pytest

from aboleth_b200.bootstrap import (LocalBootstrap, PipeBootstrap, PipeBootstrapCoordinator,
                                    TcpStoreBootstrap, decode_bundle, encode_bundle)
from tests._ranks import run_ranks


def test_bundle_roundtrip_and_layout():
    blob = encode_bundle(3, 5, [b"ab", b"", b"xyz"])
    assert blob[:12] == struct.pack("<III", 3, 5, 3)
    assert blob[12:16] == struct.pack("<I", 2)
    assert decode_bundle(blob, version=3, kind="t") == (5, (b"ab", b"", b"xyz"))


def test_bundle_errors():
    blob = encode_bundle(3, 1, [b"abcd"])
    with pytest.raises(ValueError, match="truncated Aboleth t bundle"):
        decode_bundle(blob[:5], version=3, kind="t")
    with pytest.raises(ValueError, match="unsupported Aboleth t-bundle version 3"):
        decode_bundle(blob, version=4, kind="t")
    with pytest.raises(ValueError, match="truncated Aboleth t record"):
        decode_bundle(blob[:-1], version=3, kind="t")
    with pytest.raises(ValueError, match="trailing bytes"):
        decode_bundle(blob + b"\0", version=3, kind="t")


def _tcp_rank(rank, world):
    boot = TcpStoreBootstrap.from_env(timeout=30)
    a = boot.all_gather("first", bytes([rank]) * (rank + 1))
    b = boot.all_gather("second", f"r{rank}".encode())
    boot.barrier()
    return {k: v.hex() for k, v in a.items()}, {k: v.decode() for k, v in b.items()}


def test_tcp_store_all_gather_three_ranks():
    results = run_ranks(_tcp_rank, 3)
    assert all(kind == "ok" for kind, _ in results.values()), results
    for rank in range(3):
        first, second = results[rank][1]
        assert first == {r: (bytes([r]) * (r + 1)).hex() for r in range(3)}
        assert second == {r: f"r{r}" for r in range(3)}


def _tcp_missing(rank, world):
    boot = TcpStoreBootstrap.from_env(timeout=3)
    try:
        boot.all_gather("lonely", b"x")
    except TimeoutError as error:
        return str(error)
    return "no timeout"


def test_missing_peer_times_out():
    # Rank 1 never starts: rank 0 must give up with a TimeoutError naming it.
    results = run_ranks(_tcp_missing, 2, expect_ranks=[0], timeout=60)
    kind, value = results[0]
    # The store itself may time out waiting for the second worker to join.
    assert kind == "error" or "did not receive rank 1" in value


def test_from_env_requires_variables(monkeypatch):
    for name in ("MASTER_ADDR", "MASTER_PORT", "RANK", "WORLD_SIZE"):
        monkeypatch.delenv(name, raising=False)
    with pytest.raises(RuntimeError, match="MASTER_ADDR is unset"):
        TcpStoreBootstrap.from_env()


def test_pipe_bootstrap_with_coordinator_thread():
    world = 3
    pairs = [mp.Pipe() for _ in range(world)]
    coordinator = PipeBootstrapCoordinator({r: pairs[r][0] for r in range(world)}, world)
    server = threading.Thread(target=coordinator.serve, args=(2,), kwargs={"timeout": 20})
    server.start()
    out = {}

    def rank_main(r):
        boot = PipeBootstrap(r, world, pairs[r][1])
        out[r] = (boot.all_gather("a", bytes([r])), boot.all_gather("b", b"z"))

    threads = [threading.Thread(target=rank_main, args=(r,)) for r in range(world)]
    [t.start() for t in threads]
    [t.join() for t in threads]
    server.join()
    for r in range(world):
        assert out[r][0] == {i: bytes([i]) for i in range(world)}
        assert out[r][1] == {i: b"z" for i in range(world)}


def test_pipe_coordinator_timeout_is_broadcast():
    world = 2
    pairs = [mp.Pipe() for _ in range(world)]
    coordinator = PipeBootstrapCoordinator({r: pairs[r][0] for r in range(world)}, world)
    errors = {}

    def rank0():
        try:
            PipeBootstrap(0, world, pairs[0][1]).all_gather("t", b"")
        except RuntimeError as error:
            errors[0] = str(error)

    t = threading.Thread(target=rank0)
    t.start()
    with pytest.raises(TimeoutError, match=r"ranks \[1\] did not reach bootstrap t"):
        coordinator.all_gather("t", timeout=0.5)
    t.join()
    assert "did not reach bootstrap" in errors[0]


def test_pipe_coordinator_rejects_wrong_tag():
    world = 1
    a, b = mp.Pipe()
    coordinator = PipeBootstrapCoordinator({0: a}, world)
    b.send({"kind": "aboleth_all_gather", "tag": "other", "rank": 0, "payload": b""})
    with pytest.raises(RuntimeError, match="invalid bootstrap message"):
        coordinator.all_gather("mine", timeout=2)
    assert b.recv()["kind"] == "aboleth_bootstrap_error"


def test_local_bootstrap():
    assert LocalBootstrap().all_gather("x", b"p") == {0: b"p"}
