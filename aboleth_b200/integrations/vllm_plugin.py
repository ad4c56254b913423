"""Adapters that give an installed vLLM the ``aboleth`` all2all backend.

The reference carries this as a source patch against one vLLM commit
(integrations/vllm/0001-aboleth-all2all-backend.patch:96-136 manager, :751-955
prepare/finalize).  A patch cannot follow the installed version, so here the two
classes are built at run time as subclasses of whatever the installed vLLM calls
``All2AllManagerBase`` and ``FusedMoEPrepareAndFinalizeModular``, and delegate to
:class:`~aboleth_b200.integrations.vllm_all2all.AbolethAll2AllManager` and
:class:`~aboleth_b200.integrations.vllm_all2all.AbolethPrepareAndFinalize`.

    classes = vllm_classes()              # None when vLLM is not importable
    report = install()                    # names the hooks it could place

``install`` places three hooks, each only when the installed vLLM has the spot it
expects, and reports which it placed:

* ``all2all.ALL2ALL_MANAGERS["aboleth"]`` (or the module attribute
  ``AbolethAll2AllManager``) so that a communicator can construct the manager;
* ``CudaCommunicator.__init__`` wrapped so that ``all2all_backend == "aboleth"``
  builds that manager instead of raising "Unknown all2all backend";
* ``aboleth_b200.integrations.vllm_plugin.make_prepare_finalize`` as the factory a
  MoE layer calls for this backend.

Written against the interface of vLLM 0.22 (``prepare`` returns the 5-tuple
``(a1q, a1q_scale, expert_tokens_meta, topk_ids, topk_weights)`` in the Standard
activation format; ``finalize`` writes ``output`` in place).  Constraints are the
reference's: expert parallel == data parallel, tensor parallel 1.
"""
from __future__ import annotations

import functools
from typing import Any, Callable, Optional

import torch

from .vllm_all2all import AbolethAll2AllManager, AbolethPrepareAndFinalize

BACKEND_NAME = "aboleth"


@functools.lru_cache(maxsize=1)
def vllm_classes() -> Optional[dict[str, type]]:
    """Build the adapter classes against the installed vLLM, or return ``None``."""
    try:
        from vllm.distributed.device_communicators.base_device_communicator import All2AllManagerBase
        from vllm.model_executor.layers.fused_moe import modular_kernel as mk
    except Exception:  # noqa: BLE001 - absent, or a layout this adapter does not know
        return None
    base = getattr(mk, "FusedMoEPrepareAndFinalizeModular", None) or getattr(mk, "FusedMoEPrepareAndFinalize")

    class VllmAbolethAll2AllManager(All2AllManagerBase):
        """The engine-facing manager: owns the World of this engine process."""

        def __init__(self, cpu_group, tcp_store_group=None, *, device: Optional[int] = None):
            try:
                super().__init__(cpu_group, tcp_store_group)
            except TypeError:  # older signature: (cpu_group)
                super().__init__(cpu_group)
            self.inner = AbolethAll2AllManager(cpu_group, tp_size=1, device=device)

        def get_handle(self, kwargs: dict, **options):
            return self.inner.get_handle(kwargs, **options)

        # vLLM's naive dispatch/combine entry points do not apply: tokens move inside
        # prepare/finalize, as with the other modular backends.
        def dispatch(self, *args, **kwargs):
            raise NotImplementedError("the aboleth backend dispatches in prepare()")

        def combine(self, *args, **kwargs):
            raise NotImplementedError("the aboleth backend combines in finalize()")

        def destroy(self):
            self.inner.destroy()

    class VllmAbolethPrepareAndFinalize(base):
        """vLLM's prepare/finalize contract over the fused dispatch and combine kernels."""

        def __init__(self, inner: AbolethPrepareAndFinalize, *, max_tokens_per_rank: int,
                     num_dispatchers: int):
            super().__init__()
            self.inner = inner
            self._max_tokens = int(max_tokens_per_rank)
            self._dispatchers = int(num_dispatchers)

        @property
        def activation_format(self):
            return mk.FusedMoEActivationFormat.Standard

        def topk_indices_dtype(self) -> Optional[torch.dtype]:
            return torch.int32

        def max_num_tokens_per_rank(self) -> Optional[int]:
            return self._max_tokens

        def num_dispatchers(self) -> int:
            return self._dispatchers

        def output_is_reduced(self) -> bool:
            # finalize() leaves every token of this rank complete: the sum over the
            # ranks that ran its experts happens in the combine kernel.
            return True

        def supports_async(self) -> bool:
            return True

        def _result(self, prepared):
            meta = None
            make = getattr(mk, "ExpertTokensMetadata", None)
            if make is not None:
                meta = make(expert_num_tokens=prepared.local_counts, expert_num_tokens_cpu=None)
            return (prepared.expert_input, prepared.scales, meta, prepared.global_ids,
                    prepared.expert_weights)

        def prepare(self, a1, topk_weights, topk_ids, num_experts, expert_map,
                    apply_router_weight_on_input, quant_config=None, defer_input_quant=False):
            if num_experts != self.inner.num_experts:
                raise ValueError(f"layer was planned for {self.inner.num_experts} experts, got {num_experts}")
            prepared = self.inner.prepare(a1, topk_weights, topk_ids,
                                          apply_router_weight_on_input=apply_router_weight_on_input)
            return self._result(prepared)

        def prepare_async(self, a1, topk_weights, topk_ids, num_experts, expert_map,
                          apply_router_weight_on_input, quant_config=None, defer_input_quant=False):
            receiver = self.inner.prepare_async(a1, topk_weights, topk_ids, slot=self.inner.slot,
                                                apply_router_weight_on_input=apply_router_weight_on_input)
            return lambda: self._result(receiver())

        def _reduced(self, fused_expert_output, topk_weights, topk_ids, apply_router_weight_on_input,
                     weight_and_reduce_impl):
            if fused_expert_output.dim() == 3:  # (rows, top-k, hidden): the experts left the reduction to us
                if weight_and_reduce_impl is None:
                    raise ValueError("an unreduced expert output needs a weight_and_reduce_impl")
                return weight_and_reduce_impl.apply(
                    output=None, fused_expert_output=fused_expert_output, topk_weights=topk_weights,
                    topk_ids=topk_ids, apply_router_weight_on_input=apply_router_weight_on_input)
            return fused_expert_output

        def finalize(self, output, fused_expert_output, topk_weights, topk_ids,
                     apply_router_weight_on_input, weight_and_reduce_impl=None) -> None:
            self.inner.finalize(output, self._reduced(fused_expert_output, topk_weights, topk_ids,
                                                      apply_router_weight_on_input, weight_and_reduce_impl))

        def finalize_async(self, output, fused_expert_output, topk_weights, topk_ids,
                           apply_router_weight_on_input, weight_and_reduce_impl=None) -> Callable:
            reduced = self._reduced(fused_expert_output, topk_weights, topk_ids,
                                    apply_router_weight_on_input, weight_and_reduce_impl)
            return self.inner.finalize_async(output, reduced, slot=self.inner.slot)

    return {"manager": VllmAbolethAll2AllManager, "prepare_finalize": VllmAbolethPrepareAndFinalize}


def make_prepare_finalize(manager: Any, layer_facts: dict, *, max_tokens_per_rank: int,
                          num_dispatchers: int, num_slots: int = 1, layer_name: str = ""):
    """What a MoE layer calls for this backend: one prepare/finalize object per layer.

    ``manager`` is the engine's manager (the adapter or the plain one); ``layer_facts``
    are the facts :meth:`AbolethMoERuntimeManager.get_handle` reads (``num_experts``,
    ``hidden_dim``, ``dtype``, ``quant_dtype`` ...).
    """
    classes = vllm_classes()
    if classes is None:
        raise RuntimeError("vLLM is not importable: use AbolethPrepareAndFinalize directly")
    inner_manager = getattr(manager, "inner", manager)
    inner = AbolethPrepareAndFinalize(inner_manager, layer_facts, num_slots=num_slots, layer_name=layer_name)
    return classes["prepare_finalize"](inner, max_tokens_per_rank=max_tokens_per_rank,
                                       num_dispatchers=num_dispatchers)


def install() -> dict[str, bool]:
    """Place the hooks described in the module docstring; report which were placed."""
    report = {"classes": False, "manager_registry": False, "communicator": False}
    classes = vllm_classes()
    if classes is None:
        return report
    report["classes"] = True
    from vllm.distributed.device_communicators import all2all

    registry = getattr(all2all, "ALL2ALL_MANAGERS", None) or getattr(all2all, "ALL2ALL_BACKENDS", None)
    if isinstance(registry, dict):
        registry[BACKEND_NAME] = classes["manager"]
    setattr(all2all, "AbolethAll2AllManager", classes["manager"])
    report["manager_registry"] = True
    try:
        from vllm.distributed.device_communicators.cuda_communicator import CudaCommunicator
    except Exception:  # noqa: BLE001
        return report
    original = CudaCommunicator.__init__
    if getattr(original, "_aboleth_wrapped", False):
        report["communicator"] = True
        return report

    @functools.wraps(original)
    def wrapped(self, *args, **kwargs):
        try:
            original(self, *args, **kwargs)
        except ValueError as error:
            # The stock constructor knows a fixed list of names; ours is the one it refuses.
            if BACKEND_NAME not in str(error) or "all2all" not in str(error).lower():
                raise
            self.all2all_manager = classes["manager"](getattr(self, "cpu_group", None),
                                                      getattr(self, "tcp_store_group", None))

    wrapped._aboleth_wrapped = True  # type: ignore[attr-defined]
    CudaCommunicator.__init__ = wrapped
    report["communicator"] = True
    return report
