#!/usr/bin/env python
"""Run the aboleth prepare / finalize adapter inside the installed vLLM's modular MoE kernel.

    torchrun --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 --master-port 29641 \
        examples/vllm_modular_moe.py

One process per GPU, expert parallel == data parallel == ranks, tensor parallel 1.  The MoE
layer is vLLM's own ``FusedMoEKernel``: its ``prepare`` / ``finalize`` half is
``VllmAbolethPrepareAndFinalize`` (``aboleth_b200.integrations.vllm_plugin``: the fused dispatch
and combine of this package behind vLLM's ``FusedMoEPrepareAndFinalizeModular`` interface), its
expert half is vLLM's stock ``TritonExperts``.  vLLM drives the adapter exactly as a model's MoE
layer does (asynchronous prepare, expert kernel on the dispatched records with the rank's expert
map, asynchronous finalize); nothing of vLLM is patched.  Every rank checks its tokens against a
dense fp32 evaluation of all experts and rank 0 prints one JSON line.  Weights are random-init
(same seed everywhere), tokens differ per rank and so do the token counts.
"""
import json
import os
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))


def main() -> int:
    import torch
    import torch.distributed as dist

    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", 0)))
    dev = torch.device("cuda")
    if world > 1:
        dist.init_process_group("gloo")          # the engine's CPU group; the data path is peer memory
    record = {"example": "vllm_modular_moe", "ranks": world}
    try:
        import vllm
        from vllm.config import VllmConfig, set_current_vllm_config
        from vllm.model_executor.layers.fused_moe import modular_kernel as mk
        from vllm.model_executor.layers.fused_moe.activation import MoEActivation
        from vllm.model_executor.layers.fused_moe.config import (FUSED_MOE_UNQUANTIZED_CONFIG, FusedMoEConfig,
                                                                 FusedMoEParallelConfig, RoutingMethodType)
        from vllm.model_executor.layers.fused_moe.experts.triton_moe import TritonExperts
        from vllm.v1.worker.workspace import init_workspace_manager
    except Exception as error:  # noqa: BLE001 - an absent or different vLLM is an outcome, not a crash
        record["unavailable"] = f"{type(error).__name__}: {error}"
        if rank == 0:
            print(json.dumps(record))
        return 0
    record["vllm"] = vllm.__version__

    from aboleth_b200.integrations import vllm_plugin
    from aboleth_b200.integrations.vllm_all2all import AbolethAll2AllManager

    experts, top_k, hidden, ffn, capacity = 8, 2, 1024, 2048, 128
    local = experts // world
    tokens = 96 - 32 * (rank % 2)                     # ranks disagree on the batch size, as DP ranks do
    g = torch.Generator(device=dev).manual_seed(1234)
    w1 = (torch.randn(experts, 2 * ffn, hidden, generator=g, device=dev) * 0.03).to(torch.bfloat16)
    w2 = (torch.randn(experts, hidden, ffn, generator=g, device=dev) * 0.03).to(torch.bfloat16)
    router = (torch.randn(experts, hidden, generator=g, device=dev) * 0.1).to(torch.bfloat16)
    gx = torch.Generator(device=dev).manual_seed(99 + rank)
    x = torch.randn(tokens, hidden, generator=gx, device=dev).to(torch.bfloat16)
    probs = torch.softmax((x @ router.t()).float(), -1)
    topk_weights, topk_ids = torch.topk(probs, top_k, -1)
    topk_weights = (topk_weights / topk_weights.sum(-1, keepdim=True)).contiguous()
    topk_ids = topk_ids.to(torch.int32).contiguous()
    expert_map = torch.full((experts,), -1, dtype=torch.int32, device=dev)
    expert_map[rank * local:(rank + 1) * local] = torch.arange(local, dtype=torch.int32, device=dev)

    manager = AbolethAll2AllManager(dist.group.WORLD if world > 1 else None)
    facts = dict(dtype=torch.bfloat16, num_experts=experts, num_local_experts=local,
                 num_max_tokens_per_rank=capacity, hidden=hidden, num_topk=top_k)
    try:
        scope = set_current_vllm_config(VllmConfig())
    except Exception:  # noqa: BLE001 - the kernels below do not need an engine configuration
        import contextlib
        scope = contextlib.nullcontext()
    with scope:
        init_workspace_manager(dev)
        prepare_finalize = vllm_plugin.make_prepare_finalize(manager, facts, max_tokens_per_rank=capacity,
                                                             num_dispatchers=world, layer_name="example.moe")
        parallel = FusedMoEParallelConfig(tp_size=1, pcp_size=1, dp_size=world, ep_size=world, tp_rank=0,
                                          pcp_rank=0, dp_rank=rank, ep_rank=rank, sp_size=1, use_ep=True,
                                          all2all_backend=vllm_plugin.BACKEND_NAME, enable_eplb=False)
        moe = FusedMoEConfig(num_experts=experts, experts_per_token=top_k, hidden_dim=hidden,
                             intermediate_size_per_partition=ffn, num_local_experts=local,
                             num_logical_experts=experts, activation=MoEActivation.SILU, device=dev,
                             routing_method=RoutingMethodType.RenormalizeNaive, moe_parallel_config=parallel,
                             in_dtype=torch.bfloat16, max_num_tokens=capacity)
        kernel = mk.FusedMoEKernel(prepare_finalize, TritonExperts(moe, FUSED_MOE_UNQUANTIZED_CONFIG))
        outputs = []
        for _ in range(3):                            # epochs advance, buffers are reused
            outputs.append(kernel.apply(hidden_states=x, w1=w1[rank * local:(rank + 1) * local].contiguous(),
                                        w2=w2[rank * local:(rank + 1) * local].contiguous(),
                                        topk_weights=topk_weights, topk_ids=topk_ids,
                                        activation=MoEActivation.SILU, global_num_experts=experts,
                                        expert_map=expert_map, apply_router_weight_on_input=False).clone())
        torch.cuda.synchronize()

    want = torch.zeros(tokens, hidden, dtype=torch.float32, device=dev)
    for e in range(experts):
        gate = (topk_weights * (topk_ids == e)).sum(-1, keepdim=True)
        rows = gate.squeeze(-1) > 0
        if rows.any():
            h = x[rows].float() @ w1[e].float().t()
            act = (torch.nn.functional.silu(h[:, :ffn]) * h[:, ffn:]).to(torch.bfloat16).float()
            want[rows] += gate[rows] * (act @ w2[e].float().t())
    errors = [((o.float() - want).norm() / want.norm()).item() for o in outputs]
    worst = torch.tensor([max(errors)], dtype=torch.float64)
    if world > 1:
        dist.all_reduce(worst, op=dist.ReduceOp.MAX)
    record.update(tokens_per_rank=[96 - 32 * (r % 2) for r in range(world)], experts=experts, top_k=top_k,
                  hidden=hidden, ffn=ffn, prepare_finalize=type(prepare_finalize).__name__,
                  experts_kernel="vllm TritonExperts", worst_relative_error=float(worst.item()),
                  ok=bool(worst.item() < 2e-2))
    if rank == 0:
        print(json.dumps(record))
    manager.destroy()
    if world > 1:
        dist.destroy_process_group()
    return 0 if record["ok"] else 1


if __name__ == "__main__":
    raise SystemExit(main())
