"""``--all2all-backend aboleth`` for a vLLM-style engine: manager and prepare/finalize.

The reference ships this as a patch against one vLLM commit
(integrations/vllm/0001-aboleth-all2all-backend.patch:96-136,751-955).  Here the same
two classes are plain Python over this package's runtime, usable by the in-repo
serving model (``aboleth_b200.models.mixtral``) and registrable with an installed
vLLM whose ``FusedMoEPrepareAndFinalize`` interface matches (``register_with_vllm``).
Constraints are the reference's: expert parallel == data parallel >= 2 (1 is allowed
here for single-GPU runs), tensor parallel 1.
"""
from __future__ import annotations

import contextlib

from typing import Optional

import torch

from ..bootstrap import TorchDistributedBootstrap
from ..moe.family import uniform_token_bound
from ..world import World
from .compiled_vllm import AbolethMoERuntimeManager, ModularMoERuntime, PreparedExperts


class AbolethAll2AllManager:
    """Owns the World and the MoE runtime manager of one engine process."""

    def __init__(self, cpu_group=None, *, tp_size: int = 1, device: Optional[int] = None,
                 world: Optional[World] = None):
        if tp_size != 1:
            raise ValueError("the aboleth all2all backend requires tensor parallel size 1")
        self.cpu_group = cpu_group
        if world is None:
            import torch.distributed as dist
            if cpu_group is not None:
                bootstrap = TorchDistributedBootstrap(cpu_group)
                rank, size = bootstrap.rank, bootstrap.world_size
            elif dist.is_available() and dist.is_initialized():
                raise ValueError("pass the engine's CPU (gloo) group as cpu_group")
            else:
                bootstrap, rank, size = None, 0, 1
            world = World(rank, size, device=device, bootstrap=bootstrap)
            world.connect_all("auto", remote_transport="proxy")
        self.world = world
        self.runtime = AbolethMoERuntimeManager(world=world, internode=False)

    def get_handle(self, kwargs: dict, **options):
        return self.runtime.get_handle(kwargs, **options)

    def destroy(self) -> None:
        self.runtime.close()
        self.world.close()


class AbolethPrepareAndFinalize:
    """Dispatch before the experts, combine after them; one instance per MoE layer."""

    def __init__(self, manager: AbolethAll2AllManager, layer_facts: dict, *, num_slots: int = 1,
                 placement_strategy: str = "linear", layer_name: str = ""):
        self.manager = manager
        self.num_experts = layer_facts["num_experts"]
        self.slot = 0
        self._wave_bound: Optional[int] = None
        family = manager.get_handle(layer_facts, num_slots=num_slots,
                                    placement_strategy=placement_strategy)
        self.runtime = ModularMoERuntime(family, layer_name=layer_name, slot_provider=lambda: self.slot)

    def _wave_uniform_tokens(self, tokens: int) -> int:
        """Every rank must select the same shape variant: agree on the maximum token count."""
        if not self.runtime.has_decode_sibling:
            return tokens
        if self._wave_bound is not None:
            return max(tokens, self._wave_bound)
        return uniform_token_bound(tokens, self.manager.cpu_group)

    @contextlib.contextmanager
    def wave(self, tokens: int):
        """One forward pass: agree on the token bound once (one host all-reduce) instead of in every
        layer.  An engine that already knows the maximum over the data-parallel ranks installs it with
        :meth:`set_wave_bound` instead and pays no host collective at all."""
        previous = self._wave_bound
        self._wave_bound = (uniform_token_bound(tokens, self.manager.cpu_group)
                            if self.runtime.has_decode_sibling else tokens)
        try:
            yield self._wave_bound
        finally:
            self._wave_bound = previous

    def set_wave_bound(self, bound: Optional[int]) -> None:
        """Install (or clear, with ``None``) a token bound every rank already agrees on."""
        self._wave_bound = bound

    def prepare(self, a1: torch.Tensor, topk_weights: torch.Tensor, topk_ids: torch.Tensor, *,
                quantized_input: bool = False, apply_router_weight_on_input: bool = False) -> PreparedExperts:
        return self.runtime.prepare(
            a1, topk_weights, topk_ids, num_experts=self.num_experts, expert_map=True,
            apply_router_weight_on_input=apply_router_weight_on_input,
            required_tokens=self._wave_uniform_tokens(a1.shape[0]), quantized_input=quantized_input,
            defer_input_quant=False)

    def finalize(self, output: torch.Tensor, fused_expert_output: torch.Tensor,
                 expert_offsets: Optional[torch.Tensor] = None) -> None:
        self.runtime.finalize(output, fused_expert_output, expert_offsets)

    # Dual-batch overlap: the two halves of a layer are separate calls, so an engine can
    # interleave another micro-batch (another slot) between them.
    def prepare_async(self, *args, slot: int = 0, **kwargs):
        self.slot = slot
        prepared = self.prepare(*args, **kwargs)
        return lambda: prepared

    def finalize_async(self, output, fused_expert_output, *, slot: int = 0, **kwargs):
        self.slot = slot
        self.finalize(output, fused_expert_output, **kwargs)
        return lambda: None


def register_with_vllm() -> bool:
    """Give an installed vLLM the ``aboleth`` backend (see :mod:`.vllm_plugin`).
    Returns False (and changes nothing) when vLLM is absent or its layout differs."""
    from . import vllm_plugin

    report = vllm_plugin.install()
    return report["classes"] and report["manager_registry"]
