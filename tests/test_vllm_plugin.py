"""The adapters for an installed vLLM, checked on CPU against its real base classes.

Nothing here moves a token: the inner backend is a recording stand-in.  What is
checked is that the adapter satisfies every abstract member of the installed
``FusedMoEPrepareAndFinalizeModular``, that it maps vLLM's argument lists and result
tuple onto the backend's, and that ``install`` places its hooks once.
"""
import pytest
import torch

from aboleth_b200.integrations import vllm_plugin
from aboleth_b200.integrations.compiled_vllm import PreparedExperts



@pytest.fixture(scope="module")
def classes():
    # Imported here, not at collection: loading vLLM takes tens of seconds.
    found = vllm_plugin.vllm_classes()
    if found is None:
        pytest.skip("vLLM is not importable")
    return found


class _Inner:
    num_experts = 8
    slot = 0

    def __init__(self):
        self.calls = []

    def prepare(self, a1, topk_weights, topk_ids, *, apply_router_weight_on_input=False):
        self.calls.append(("prepare", tuple(a1.shape), apply_router_weight_on_input))
        rows = 2 * a1.shape[0]
        return PreparedExperts(expert_input=torch.zeros(rows, a1.shape[1]),
                               local_counts=torch.tensor([3, 1], dtype=torch.int32),
                               global_ids=torch.zeros(rows, topk_ids.shape[1], dtype=torch.int32),
                               expert_weights=torch.ones(rows, topk_ids.shape[1]),
                               scales=None)

    def prepare_async(self, *args, slot=0, **kwargs):
        self.calls.append(("prepare_async", slot))
        prepared = self.prepare(*args, **kwargs)
        return lambda: prepared

    def finalize(self, output, fused_expert_output, expert_offsets=None):
        self.calls.append(("finalize", tuple(fused_expert_output.shape)))
        output.copy_(fused_expert_output[: output.shape[0]])

    def finalize_async(self, output, fused_expert_output, *, slot=0):
        self.calls.append(("finalize_async", slot))
        self.finalize(output, fused_expert_output)
        return lambda: None


class _Reduce:
    def apply(self, output, fused_expert_output, topk_weights, topk_ids, apply_router_weight_on_input):
        return (fused_expert_output * topk_weights.unsqueeze(-1)).sum(dim=1)


def test_adapter_satisfies_the_installed_interface_and_maps_arguments(classes):
    from vllm.model_executor.layers.fused_moe import modular_kernel as mk

    inner = _Inner()
    adapter = classes["prepare_finalize"](inner, max_tokens_per_rank=128, num_dispatchers=8)
    assert isinstance(adapter, mk.FusedMoEPrepareAndFinalize)
    assert adapter.activation_format == mk.FusedMoEActivationFormat.Standard
    assert adapter.topk_indices_dtype() == torch.int32 and adapter.max_num_tokens_per_rank() == 128
    assert adapter.num_dispatchers() == 8 and adapter.output_is_reduced() and adapter.supports_async()

    a1 = torch.randn(4, 16)
    weights, ids = torch.rand(4, 2), torch.zeros(4, 2, dtype=torch.int32)
    a1q, scales, meta, out_ids, out_weights = adapter.prepare(a1, weights, ids, 8, None, False, None, False)
    assert a1q.shape == (8, 16) and scales is None and out_ids.shape == (8, 2) and out_weights.shape == (8, 2)
    assert meta.expert_num_tokens.tolist() == [3, 1] and meta.expert_num_tokens_cpu is None
    with pytest.raises(ValueError, match="planned for 8 experts"):
        adapter.prepare(a1, weights, ids, 16, None, False, None, False)
    assert adapter.prepare_async(a1, weights, ids, 8, None, True, None, False)()[0].shape == (8, 16)
    assert inner.calls[-1] == ("prepare", (4, 16), True)

    output = torch.zeros(4, 16)
    reduced = torch.arange(8 * 16, dtype=torch.float32).view(8, 16)
    adapter.finalize(output, reduced, out_weights, out_ids, False, None)  # experts already reduced
    assert torch.equal(output, reduced[:4]) and inner.calls[-1] == ("finalize", (8, 16))
    unreduced = torch.ones(8, 2, 16)
    adapter.finalize(output, unreduced, torch.full((8, 2), 0.5), out_ids, False, _Reduce())
    assert torch.equal(output, torch.ones(4, 16)) and inner.calls[-1] == ("finalize", (8, 16))
    with pytest.raises(ValueError, match="needs a weight_and_reduce_impl"):
        adapter.finalize(output, unreduced, out_weights, out_ids, False, None)
    assert adapter.finalize_async(output, reduced, out_weights, out_ids, False, None)() is None


def test_install_places_each_hook_once(classes):
    from vllm.distributed.device_communicators import all2all
    from vllm.distributed.device_communicators.base_device_communicator import All2AllManagerBase
    from vllm.distributed.device_communicators.cuda_communicator import CudaCommunicator

    report = vllm_plugin.install()
    assert report == {"classes": True, "manager_registry": True, "communicator": True}
    assert issubclass(all2all.AbolethAll2AllManager, All2AllManagerBase)
    first = CudaCommunicator.__init__
    assert vllm_plugin.install()["communicator"] and CudaCommunicator.__init__ is first  # not wrapped twice
