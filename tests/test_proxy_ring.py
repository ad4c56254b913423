"""Host-proxy ring on plain memory: a CPU thread stands in for the GPU producer.

Mirrors the reference's fault tests (experiments/python/aboleth_proxy_error.py:
bad key => status 2 and the batch still retires).
"""
import ctypes

import pytest
import torch

from aboleth_b200 import Runtime, Transport, abi
from aboleth_b200.runtime import _lib


def _submit(endpoint, commands, timeout=5.0):
    desc = endpoint.descriptor()
    array = (abi.ProxyCommand * len(commands))(*commands)
    seq = _lib().ab200_proxy_host_submit(ctypes.byref(desc), array, len(commands), timeout)
    return desc, seq


def _poll(desc, seq, timeout=5.0):
    return _lib().ab200_proxy_host_poll(ctypes.byref(desc), seq, timeout)


@pytest.fixture
def rt():
    runtime = Runtime("cpu")
    yield runtime
    runtime.close()


def test_write_then_strong_signal(rt):
    ep = rt.create_local_endpoint(Transport.PROXY)
    src = rt.allocate(4096)
    dst = rt.allocate(4096 + 8)
    src[:4096] = torch.arange(4096, dtype=torch.int32).to(torch.uint8)
    cmds = [abi.ProxyCommand(src.data_ptr(), dst.data_ptr(), 4096, 0, 0, abi.PROXY_WRITE),
            abi.ProxyCommand(77, dst.data_ptr() + 4096, 8, 0, 0, abi.PROXY_STRONG_SIGNAL)]
    desc, seq = _submit(ep, cmds)
    assert seq == 0 and _poll(desc, seq) == abi.STATUS_OK
    assert torch.equal(dst[:4096], src[:4096])
    assert dst[4096:].view(torch.int64).item() == 77
    assert ep.state() == (1, 1, 0)
    stats = ep.stats()
    assert stats["batches"] == 1 and stats["commands"] == 2 and stats["bytes"] == 4096
    assert ep.submit_mode == "proxy" and ep.max_inline_bytes == 8 and ep.capacity == 64 * 256


def test_ring_wraps_and_stays_ordered(rt):
    ep = rt.create_local_endpoint(Transport.RDMA)  # queue names resolve to the ring
    assert ep.handle & 7 == abi.KIND_BITS["proxy"]
    cell = rt.allocate(8)
    desc = None
    for i in range(200):  # > 64 slots
        desc, seq = _submit(ep, [abi.ProxyCommand(i + 1, cell.data_ptr(), 8, 0, 0,
                                                  abi.PROXY_WEAK_SIGNAL)])
        assert seq == i
    assert _poll(desc, 199) == abi.STATUS_OK
    assert cell.view(torch.int64).item() == 200


def test_bad_key_fails_endpoint_but_retires(rt):
    ep = rt.create_local_endpoint(Transport.PROXY)
    src, dst = rt.allocate(64), rt.allocate(64)
    reg = rt.register(src)
    ok = [abi.ProxyCommand(src.data_ptr(), dst.data_ptr(), 64, reg.lkey, 0, abi.PROXY_WRITE)]
    desc, seq = _submit(ep, ok)
    assert _poll(desc, seq) == abi.STATUS_OK
    bad = [abi.ProxyCommand(src.data_ptr(), dst.data_ptr(), 64, 0xdead, 0, abi.PROXY_WRITE)]
    desc, seq = _submit(ep, bad)
    assert _poll(desc, seq) == abi.STATUS_COMPLETION_FAILURE
    # Out of range under a valid key is refused the same way on a fresh endpoint.
    ep2 = rt.create_local_endpoint(Transport.PROXY)
    over = [abi.ProxyCommand(src.data_ptr() + 32, dst.data_ptr(), 64, reg.lkey, 0, abi.PROXY_WRITE)]
    desc2, seq2 = _submit(ep2, over)
    assert _poll(desc2, seq2) == abi.STATUS_COMPLETION_FAILURE
    # The failed endpoint keeps retiring later batches without executing them.
    desc, seq = _submit(ep, ok)
    assert _poll(desc, seq) == abi.STATUS_COMPLETION_FAILURE
    assert ep.state() == (3, 3, abi.STATUS_COMPLETION_FAILURE)


def test_injected_failure_and_malformed_opcode(rt):
    ep = rt.create_local_endpoint(Transport.PROXY)
    cell = rt.allocate(8)
    ep.inject_failure(abi.STATUS_COMPLETION_FAILURE, 1)
    desc, seq = _submit(ep, [abi.ProxyCommand(5, cell.data_ptr(), 8, 0, 0, abi.PROXY_WEAK_SIGNAL)])
    assert _poll(desc, seq) == abi.STATUS_COMPLETION_FAILURE
    assert cell.view(torch.int64).item() == 0  # not executed
    ep2 = rt.create_local_endpoint(Transport.PROXY)
    desc2, seq2 = _submit(ep2, [abi.ProxyCommand(0, 0, 0, 0, 0, 9)])
    assert _poll(desc2, seq2) == abi.STATUS_MALFORMED


def test_poll_timeout_reports_status_1(rt):
    ep = rt.create_local_endpoint(Transport.PROXY)
    desc = ep.descriptor()
    assert _poll(desc, 0, timeout=0.2) == abi.STATUS_TIMEOUT  # nothing was submitted


def test_endpoint_config_versioning(rt):
    cfg = abi.EndpointConfig()
    assert rt.create_local_endpoint(Transport.PROXY, config=cfg) is not None
    small = abi.EndpointConfig()
    small.struct_size = 16  # an older caller: trailing fields default
    assert rt.create_local_endpoint(Transport.PROXY, config=small) is not None
    big = abi.EndpointConfig()
    big.struct_size = 200
    with pytest.raises(RuntimeError, match="larger than this runtime knows"):
        rt.create_local_endpoint(Transport.PROXY, config=big)
    with pytest.raises(RuntimeError, match="qp_type must be 0"):
        rt.create_local_endpoint(Transport.PROXY, config=abi.EndpointConfig(qp_type=1))
    with pytest.raises(RuntimeError, match="hca must be empty"):
        rt.create_local_endpoint(Transport.PROXY, config=abi.EndpointConfig(hca=b"mlx5_0"))


def test_queue_snapshot_returns_what_the_producer_wrote(rt):
    """The ring keeps a retired batch's commands until it wraps: a snapshot returns them byte for
    byte, batch by batch; batches not produced yet, or already overwritten, are refused."""
    ep = rt.create_local_endpoint(Transport.PROXY)
    src, dst = rt.allocate(4096), rt.allocate(4096 + 8)
    first = [abi.ProxyCommand(src.data_ptr(), dst.data_ptr(), 1024, 0, 0, abi.PROXY_WRITE),
             abi.ProxyCommand(5, dst.data_ptr() + 4096, 8, 0, 0, abi.PROXY_STRONG_SIGNAL)]
    second = [abi.ProxyCommand(src.data_ptr() + 1024, dst.data_ptr() + 1024, 512, 0, 0, abi.PROXY_WRITE)]
    for commands in (first, second):
        desc, seq = _submit(ep, commands)
        assert _poll(desc, seq) == abi.STATUS_OK
    snapshot = ep.snapshot_queue()
    assert [len(batch) for batch in snapshot] == [2, 1]
    assert snapshot[0] == [bytes(c) for c in first] and snapshot[1] == [bytes(c) for c in second]
    assert ep.snapshot_queue(1, 1) == [snapshot[1]]
    with pytest.raises(RuntimeError, match="not retired"):
        ep.snapshot_queue(0, 3)
    for _ in range(70):                                   # wrap the 64-slot ring
        desc, seq = _submit(ep, second)
        assert _poll(desc, seq) == abi.STATUS_OK
    with pytest.raises(RuntimeError, match="overwritten"):
        ep.snapshot_queue(0, 1)
    assert ep.snapshot_queue(71, 1) == [snapshot[1]]
