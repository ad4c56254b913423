"""Failure detection on the host: heartbeats over the bootstrap store (CPU ranks only)."""
import time

import pytest

from aboleth_b200.utils.liveness import Heartbeat, PeerLost
from tests._ranks import run_ranks


class _Store(dict):
    """In-process stand-in for a key-value store."""

    def set(self, key, value):
        self[key] = bytes(value)

    def check(self, keys):
        return all(k in self for k in keys)


def test_states_follow_the_beats_with_a_fake_clock():
    store, now = _Store(), [0.0]
    a = Heartbeat(store, 0, 3, interval=0.1, timeout=1.0, clock=lambda: now[0])
    b = Heartbeat(store, 1, 3, interval=0.1, timeout=1.0, clock=lambda: now[0])
    a.beat(), b.beat()
    a._seen = {}
    assert a.peers() == {1: "alive", 2: "alive"}  # rank 2 has its grace period
    now[0] = 0.9
    b.beat()
    assert a.peers() == {1: "alive", 2: "alive"}
    now[0] = 1.5  # rank 2 never beat; rank 1 beat at 0.9
    assert a.peers() == {1: "alive", 2: "lost"}
    with pytest.raises(PeerLost, match=r"no heartbeat from rank\(s\) \[2\]") as info:
        a.check()
    assert info.value.lost == (2,) and info.value.left == ()
    now[0] = 2.5
    assert a.peers()[1] == "lost"
    b.leave()
    with pytest.raises(PeerLost, match=r"rank\(s\) \[1\] left"):
        a.check()
    with pytest.raises(ValueError):
        Heartbeat(store, 0, 2, interval=1.0, timeout=0.5)
    with pytest.raises(ValueError):
        Heartbeat(store, 2, 2)


def _rank(rank, world_size, plan):
    from aboleth_b200.bootstrap import TcpStoreBootstrap

    boot = TcpStoreBootstrap.from_env(timeout=30)
    hb = Heartbeat(boot._store, rank, world_size, interval=0.05, timeout=1.0).start()
    boot.barrier("started")
    hb.check()  # everyone is here
    boot.barrier("checked")
    events = []
    if plan == "leave" and rank == 2:
        hb.leave()  # orderly: between steps, nothing in flight
        boot.barrier("after")
        return ["left"]
    if plan == "silent" and rank == 2:
        hb.stop()  # stands in for a rank that hangs or dies: it stops beating, says nothing
        time.sleep(2.5)
        boot.barrier("after")
        return ["silent"]
    deadline = time.monotonic() + 10.0
    while time.monotonic() < deadline:
        try:
            hb.check()
        except PeerLost as error:
            events.append((error.lost, error.left))
            break
        time.sleep(0.05)
    boot.barrier("after")
    hb.stop()
    return events


@pytest.mark.parametrize("plan,expected", [("leave", ((), (2,))), ("silent", ((2,), ()))])
def test_ranks_learn_on_the_host_that_a_peer_is_gone(plan, expected):
    results = run_ranks(_rank, 3, plan, timeout=90)
    assert all(kind == "ok" for kind, _ in results.values()), results
    assert results[0][1] == [expected] and results[1][1] == [expected]
