"""A KV connector for a prefill / decode pair of vLLM engines over :class:`VLLMKVPeerRuntime`.

The reference adds its connector to vLLM as part of a source patch
(integrations/vllm/0001-aboleth-all2all-backend.patch:229-478): a subclass of that commit's NIXL
connector whose data movement is replaced by the compiled KV pull and whose control plane (block
ids, completion notifications) stays NIXL's.  The installed vLLM has no NIXL module to inherit
from, so this connector is self-contained on ``KVConnectorBase_V1``:

* control plane: the prefill engine returns ``kv_transfer_params`` with its block ids when a
  request finishes (``request_finished``) and keeps the blocks until the decode side reports the
  pull complete; the decode engine's scheduler reads those parameters
  (``get_num_new_matched_tokens`` / ``update_state_after_alloc``) and hands the worker one
  :class:`PullOrder` per request (``build_connector_meta``).  Completion travels back through the
  two-rank world's store (:class:`CompletionBoard`), not through a second transport.
* data plane: the decode worker pulls with ``start_layered_pull_blocks`` (one event per readiness
  group), ``wait_for_layer_load`` makes the current stream wait for the layer's event, and
  ``get_finished`` retires pulls whose completion event has fired.

:class:`PullScheduler` and :class:`PullWorker` hold all the logic and need no vLLM;
:func:`vllm_kv_connector_class` wraps them in a subclass of the installed base (``None`` when vLLM
is absent).  Same limits as the reference's: one prefill and one decode engine, tensor and
pipeline parallel size 1, equal block geometry on both sides.
"""
from __future__ import annotations

import functools
from dataclasses import dataclass, field
from typing import Any, Callable, Iterable, Optional

CONNECTOR_NAME = "AbolethConnector"


@dataclass(frozen=True)
class PullOrder:
    """One request's pull: which remote blocks land in which local blocks."""

    request_id: str
    local_block_ids: tuple
    remote_block_ids: tuple
    remote_rank: int
    remote_request_id: str


@dataclass
class PullBatch:
    """What the scheduler hands the worker for one step (the connector metadata's payload)."""

    orders: list = field(default_factory=list)


class PullScheduler:
    """Scheduler-side bookkeeping of both roles."""

    def __init__(self, *, rank: int, block_size: int):
        self.rank, self.block_size = rank, block_size
        self._waiting: dict[str, PullOrder] = {}      # decode: allocated, not yet handed to the worker
        self._held: set[str] = set()                  # prefill: finished requests whose blocks are kept

    # -- decode side ---------------------------------------------------------------------------
    def matched_tokens(self, params: Optional[dict], prompt_tokens: int, computed_tokens: int) -> tuple[int, bool]:
        """How many prompt tokens the remote prefill can supply beyond ``computed_tokens`` (whole blocks
        only), and whether they arrive asynchronously."""
        if not params or not params.get("do_remote_prefill") or not params.get("remote_block_ids"):
            return 0, False
        available = min(len(params["remote_block_ids"]) * self.block_size, prompt_tokens)
        # The last prompt token is always recomputed locally so that the decode engine samples from it.
        usable = (min(available, prompt_tokens - 1) // self.block_size) * self.block_size
        fresh = usable - computed_tokens
        return (fresh, True) if fresh > 0 else (0, False)

    def allocated(self, request_id: str, params: Optional[dict], local_block_ids: Iterable[int],
                  external_tokens: int) -> None:
        """Blocks were allocated for ``external_tokens`` remote tokens: record the pull."""
        if external_tokens <= 0 or not params or not params.get("do_remote_prefill"):
            return
        count = external_tokens // self.block_size
        remote = tuple(params["remote_block_ids"])[:count]
        local = tuple(local_block_ids)[:count]
        if len(remote) != len(local) or not remote:
            raise ValueError(f"request {request_id}: {len(local)} local blocks for {len(remote)} remote blocks")
        self._waiting[request_id] = PullOrder(request_id, local, remote, int(params.get("remote_rank", 1 - self.rank)),
                                              str(params.get("remote_request_id", request_id)))
        params["do_remote_prefill"] = False     # a second allocation call must not start a second pull

    def drain(self) -> PullBatch:
        batch = PullBatch(list(self._waiting.values()))
        self._waiting.clear()
        return batch

    # -- prefill side ----------------------------------------------------------------------------
    def finished(self, request_id: str, params: Optional[dict], block_ids: list,
                 finished_by_length: bool) -> tuple[bool, Optional[dict]]:
        """A request ended on the prefill engine.  Its blocks are kept (``True``) and described to the
        decode engine when the caller asked for a remote decode."""
        if not params or not params.get("do_remote_decode") or not finished_by_length or not block_ids:
            return False, None
        self._held.add(request_id)
        return True, {"do_remote_prefill": True, "do_remote_decode": False, "remote_block_ids": list(block_ids),
                      "remote_rank": self.rank, "remote_request_id": request_id}


    def released(self, request_ids: Iterable[str]) -> None:
        """The decode side has read these requests' blocks: the engine frees them now."""
        self._held.difference_update(request_ids)

    @property
    def held(self) -> frozenset:
        return frozenset(self._held)


class CompletionBoard:
    """Pull completions from the decode rank to the prefill rank through a key-value store
    (``set`` / ``get`` / ``add``, as the bootstrap's store offers)."""

    def __init__(self, store, *, prefix: str = "aboleth_kv_done"):
        self.store, self.prefix, self._read = store, prefix, 0

    def post(self, remote_request_id: str) -> None:
        index = int(self.store.add(f"{self.prefix}/count", 1))
        self.store.set(f"{self.prefix}/{index}", remote_request_id)

    def collect(self) -> set:
        done = set()
        posted = int(self.store.add(f"{self.prefix}/count", 0))
        while self._read < posted:
            self._read += 1
            value = self.store.get(f"{self.prefix}/{self._read}")
            done.add(value.decode() if isinstance(value, bytes) else str(value))
        return done


class PullWorker:
    """Worker-side: starts pulls, waits per layer, retires finished ones."""

    def __init__(self, runtime, board: Optional[CompletionBoard], *, wait_event: Callable[[Any], None],
                 producer: bool = False):
        self.runtime, self.board, self._wait_event = runtime, board, wait_event
        self.producer = producer                  # the prefill side reads the board, the decode side writes it
        self._inflight: dict[str, tuple] = {}     # request id -> (ticket, order)

    def register(self, kv_caches: dict) -> None:
        self.runtime.register_kv_caches(kv_caches, consumer_order=tuple(kv_caches))

    def start(self, batch: PullBatch) -> int:
        for order in batch.orders:
            ticket = self.runtime.start_layered_pull_blocks(local_block_ids=list(order.local_block_ids),
                                                            remote_block_ids=list(order.remote_block_ids),
                                                            remote_rank=order.remote_rank)
            self._inflight[order.request_id] = (ticket, order)
        return len(batch.orders)

    @property
    def has_active_layer_events(self) -> bool:
        return bool(self._inflight)

    def wait_for_layer(self, layer_name: str) -> None:
        for ticket, _ in self._inflight.values():
            event = ticket.layer_events.get(layer_name)
            if event is not None:
                self._wait_event(event)

    def retire(self) -> set:
        """Request ids whose pull has completed; each is reported to the prefill side once."""
        done = {rid for rid, (ticket, _) in self._inflight.items() if ticket.completion.query()}
        for rid in done:
            _, order = self._inflight.pop(rid)
            if self.board is not None and not self.producer:
                self.board.post(order.remote_request_id)
        if done:
            self.runtime.check()
        return done

    def released_by_peer(self) -> set:
        """Prefill side: requests whose blocks the decode side has finished reading (nothing on the
        decode side, which only posts)."""
        return self.board.collect() if self.board is not None and self.producer else set()


@functools.lru_cache(maxsize=1)
def vllm_kv_connector_class() -> Optional[type]:
    """``AbolethConnector`` as a subclass of the installed vLLM's ``KVConnectorBase_V1``; ``None``
    when vLLM (or that interface) is not importable."""
    try:
        from vllm.distributed.kv_transfer.kv_connector.v1.base import (KVConnectorBase_V1, KVConnectorMetadata,
                                                                        KVConnectorRole)
    except Exception:  # noqa: BLE001 - absent, or a layout this adapter does not know
        return None

    class AbolethConnectorMetadata(KVConnectorMetadata):
        def __init__(self, batch: PullBatch):
            self.batch = batch

    class AbolethConnector(KVConnectorBase_V1):
        """1P1D KV migration: the decode engine pulls the prefill engine's blocks over NVLink."""

        @classmethod
        def requires_piecewise_for_cudagraph(cls, extra_config) -> bool:
            return True     # wait_for_layer_load must run between layers

        def __init__(self, vllm_config, role, kv_cache_config=None):
            super().__init__(vllm_config, role, kv_cache_config)
            config = vllm_config.kv_transfer_config
            rank = config.kv_rank if config.kv_rank is not None else (0 if config.kv_role == "kv_producer" else 1)
            if (config.kv_parallel_size or 1) not in (1, 2):
                raise NotImplementedError("AbolethConnector supports one prefill and one decode engine")
            self.kv_rank = int(rank)
            self.scheduler_side = self.worker_side = None
            if role == KVConnectorRole.SCHEDULER:
                self.scheduler_side = PullScheduler(rank=self.kv_rank,
                                                    block_size=vllm_config.cache_config.block_size)
            else:
                import torch

                from ..kv.profile import KVRuntimeOverrides
                from .vllm_kv import VLLMKVPeerRuntime
                extra = config.kv_connector_extra_config or {}
                port = int(extra.get("aboleth_store_port", config.kv_port + 1000))
                runtime = VLLMKVPeerRuntime(rank=self.kv_rank, world_size=2, device=torch.cuda.current_device(),
                                            host=config.kv_ip, port=port,
                                            overrides=KVRuntimeOverrides.from_mapping(extra))
                store = getattr(runtime.bootstrap, "store", None)
                board = CompletionBoard(store) if store is not None else None
                self.worker_side = PullWorker(runtime, board, producer=config.kv_role == "kv_producer",
                                              wait_event=lambda e: torch.cuda.current_stream().wait_event(e))

        # -- worker ----------------------------------------------------------------------------
        def register_kv_caches(self, kv_caches):
            self.worker_side.register(kv_caches)

        def start_load_kv(self, forward_context, **kwargs) -> None:
            metadata = self._get_connector_metadata()
            if isinstance(metadata, AbolethConnectorMetadata):
                self.worker_side.start(metadata.batch)

        def wait_for_layer_load(self, layer_name: str) -> None:
            if self.worker_side.has_active_layer_events:
                self.worker_side.wait_for_layer(layer_name)

        def save_kv_layer(self, layer_name, kv_layer, attn_metadata, **kwargs) -> None:
            return      # the decode side pulls; the prefill side has nothing to push

        def wait_for_save(self):
            return

        def get_finished(self, finished_req_ids):
            received = self.worker_side.retire()
            released = self.worker_side.released_by_peer()
            return (released or None), (received or None)

        def shutdown(self):
            if self.worker_side is not None:
                self.worker_side.runtime.close()

        # -- scheduler ---------------------------------------------------------------------------
        def get_num_new_matched_tokens(self, request, num_computed_tokens):
            return self.scheduler_side.matched_tokens(request.kv_transfer_params, request.num_prompt_tokens,
                                                      num_computed_tokens)

        def update_state_after_alloc(self, request, blocks, num_external_tokens):
            ids = blocks.get_block_ids()
            self.scheduler_side.allocated(request.request_id, request.kv_transfer_params,
                                          ids[0] if ids and isinstance(ids[0], (list, tuple)) else ids,
                                          num_external_tokens)

        def build_connector_meta(self, scheduler_output):
            return AbolethConnectorMetadata(self.scheduler_side.drain())

        def update_connector_output(self, connector_output):
            self.scheduler_side.released(getattr(connector_output, "finished_sending", None) or ())

        def request_finished(self, request, block_ids):
            by_length = getattr(getattr(request, "status", None), "name", "") == "FINISHED_LENGTH_CAPPED"
            return self.scheduler_side.finished(request.request_id, request.kv_transfer_params, block_ids, by_length)

    AbolethConnector.Metadata = AbolethConnectorMetadata
    return AbolethConnector


def register_kv_connector() -> bool:
    """Register :data:`CONNECTOR_NAME` with the installed vLLM's connector factory."""
    if vllm_kv_connector_class() is None:
        return False
    try:
        from vllm.distributed.kv_transfer.kv_connector.factory import KVConnectorFactory
    except Exception:  # noqa: BLE001
        return False
    registry = getattr(KVConnectorFactory, "_registry", {})
    if CONNECTOR_NAME not in registry:
        KVConnectorFactory.register_connector(CONNECTOR_NAME, __name__, "_connector_for_factory")
    return True


def __getattr__(name: str):
    # The factory imports a class by module path and attribute name.
    if name == "_connector_for_factory":
        cls = vllm_kv_connector_class()
        if cls is None:
            raise AttributeError(name)
        return cls
    raise AttributeError(name)
