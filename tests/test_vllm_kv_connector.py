"""The KV connector's control plane on CPU: scheduler bookkeeping of both roles, the completion board,
the worker's ticket handling against a fake runtime, and the class built on the installed vLLM base."""
import pytest

from aboleth_b200.integrations.vllm_kv_connector import (CompletionBoard, PullBatch, PullOrder, PullScheduler,
                                                         PullWorker, vllm_kv_connector_class)
from aboleth_b200.kv.profile import KVRuntimeOverrides


def test_prefill_side_keeps_blocks_and_describes_them():
    prefill = PullScheduler(rank=0, block_size=16)
    assert prefill.finished("r1", None, [3, 4], True) == (False, None)
    assert prefill.finished("r1", {"do_remote_decode": True}, [3, 4], False) == (False, None)   # aborted
    keep, params = prefill.finished("r1", {"do_remote_decode": True}, [3, 4, 9], True)
    assert keep and params == {"do_remote_prefill": True, "do_remote_decode": False,
                               "remote_block_ids": [3, 4, 9], "remote_rank": 0, "remote_request_id": "r1"}
    assert prefill.held == {"r1"}
    prefill.released(["r1", "unknown"])
    assert prefill.held == frozenset()


def test_decode_side_counts_whole_blocks_and_orders_one_pull():
    decode = PullScheduler(rank=1, block_size=16)
    params = {"do_remote_prefill": True, "remote_block_ids": [3, 4, 9], "remote_rank": 0,
              "remote_request_id": "r1"}
    assert decode.matched_tokens(None, 40, 0) == (0, False)
    # 40 prompt tokens, 3 remote blocks = 48 tokens of cache: two whole blocks below the last token
    assert decode.matched_tokens(params, 40, 0) == (32, True)
    assert decode.matched_tokens(params, 40, 16) == (16, True)
    assert decode.matched_tokens(params, 40, 32) == (0, False)
    # a prompt that ends exactly on a block boundary still recomputes its last token
    assert decode.matched_tokens(params, 48, 0) == (32, True)
    decode.allocated("d7", params, [20, 21, 22], 32)
    decode.allocated("d7", params, [20, 21, 22, 23], 0)       # the second call after the load: no new pull
    batch = decode.drain()
    assert batch.orders == [PullOrder("d7", (20, 21), (3, 4), 0, "r1")]
    assert decode.drain().orders == []
    with pytest.raises(ValueError):
        decode.allocated("d8", {"do_remote_prefill": True, "remote_block_ids": [1]}, [5, 6], 32)


class _Store:
    def __init__(self):
        self.data = {}

    def add(self, key, amount):
        self.data[key] = int(self.data.get(key, 0)) + amount
        return self.data[key]

    def set(self, key, value):
        self.data[key] = value.encode() if isinstance(value, str) else value

    def get(self, key):
        return self.data[key]


class _Event:
    def __init__(self):
        self.done = False

    def query(self):
        return self.done


class _Ticket:
    def __init__(self, layers):
        self.completion = _Event()
        self.layer_events = {name: _Event() for name in layers}


class _Runtime:
    def __init__(self):
        self.registered, self.pulls, self.checked = None, [], 0

    def register_kv_caches(self, caches, *, consumer_order):
        self.registered = consumer_order

    def start_layered_pull_blocks(self, **kw):
        self.pulls.append(kw)
        return _Ticket(self.registered)

    def check(self):
        self.checked += 1


def test_worker_waits_per_layer_and_reports_each_completion_once():
    store = _Store()
    runtime, waited = _Runtime(), []
    decode = PullWorker(runtime, CompletionBoard(store), wait_event=waited.append)
    prefill = PullWorker(_Runtime(), CompletionBoard(store), wait_event=waited.append, producer=True)
    decode.register({"layer.0": object(), "layer.1": object()})
    assert runtime.registered == ("layer.0", "layer.1")
    assert not decode.has_active_layer_events
    decode.start(PullBatch([PullOrder("d7", (20, 21), (3, 4), 0, "r1"), PullOrder("d8", (5,), (6,), 0, "r2")]))
    assert runtime.pulls[0] == {"local_block_ids": [20, 21], "remote_block_ids": [3, 4], "remote_rank": 0}
    decode.wait_for_layer("layer.1")
    assert len(waited) == 2                      # one event per pull in flight
    assert decode.retire() == set() and prefill.released_by_peer() == set()
    decode._inflight["d7"][0].completion.done = True
    assert decode.retire() == {"d7"} and runtime.checked == 1
    assert decode.retire() == set()
    assert decode.released_by_peer() == set()    # the decode side never reads its own posts back
    assert prefill.released_by_peer() == {"r1"}  # the prefill side may free r1's blocks now
    assert prefill.released_by_peer() == set()
    decode._inflight["d8"][0].completion.done = True
    assert decode.retire() == {"d8"} and prefill.released_by_peer() == {"r2"}
    assert not decode.has_active_layer_events


def test_runtime_overrides_from_engine_options():
    o = KVRuntimeOverrides.from_mapping({"aboleth_kv_copy_workers": "8", "consumers_per_readiness": 2, "other": 1})
    assert (o.copy_workers, o.consumers_per_readiness, o.copy_engine_threshold) == (8, 2, None)
    with pytest.raises(ValueError):
        KVRuntimeOverrides.from_mapping({"copy_workers": 0})


def test_connector_class_fills_the_installed_interface():
    cls = vllm_kv_connector_class()
    if cls is None:
        pytest.skip("vLLM is not importable")
    from vllm.distributed.kv_transfer.kv_connector.v1.base import KVConnectorBase_V1
    assert issubclass(cls, KVConnectorBase_V1) and cls.__name__ == "AbolethConnector"
    assert not getattr(cls, "__abstractmethods__", None)       # every abstract method is implemented
    assert cls.requires_piecewise_for_cudagraph({}) is True
