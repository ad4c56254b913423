"""The compiled MoE plan drives the executor: launch geometry and buffer decisions follow the
endpoint profile the plan was compiled against."""
import pytest
import torch

from aboleth_b200.endpoint_profiles import SEED_PROFILES, EndpointProfile
from aboleth_b200.moe import MoESpec
from aboleth_b200.moe.compiled_plan import compile_moe_plan
from aboleth_b200.moe.native import LaunchBinding

FINE = {"p2p": EndpointProfile("test:fine-grained", "p2p", "B200", "none", "NV18", 16384, 16, 4),
        "proxy": SEED_PROFILES["B200_HOSTRING"]}


def test_binding_follows_the_endpoint_profile():
    decode = MoESpec(capacity=128, hidden=7168, top_k=8, experts=256, ranks=8)
    prefill = MoESpec(capacity=4096, hidden=7168, top_k=8, experts=256, ranks=8)
    seed_decode = LaunchBinding.from_plan(decode, compile_moe_plan(decode))
    seed_prefill = LaunchBinding.from_plan(prefill, compile_moe_plan(prefill))
    # 128 tokens need 4 of the seed profile's 16 lanes: latency path; 4096 tokens saturate them.
    assert (seed_decode.by_warp, seed_decode.dispatch_lanes) == (False, 4)
    assert (seed_prefill.by_warp, seed_prefill.dispatch_lanes) == (True, 16)
    assert seed_prefill.send_warps == 7 and seed_prefill.return_block == 128 and seed_decode.return_block == 64
    assert seed_prefill.received_rows == 8 * 4096 and seed_prefill.borrow_tokens and seed_prefill.forward_expert_output
    # A profile with 16 KiB per endpoint and 4 sender warps fans the same 128 tokens over every lane.
    fine = LaunchBinding.from_plan(decode, compile_moe_plan(decode, profiles=FINE))
    assert fine.by_warp and fine.dispatch_lanes == 16 and fine.send_warps == 3 and fine.profile == "test:fine-grained"


@pytest.mark.gpu
def test_manifest_reports_what_the_plan_made_the_executor_launch():
    import aboleth_b200 as ab
    from aboleth_b200.moe import NativeMoESlot
    from aboleth_b200.moe.reference import standin_layer_reference
    from aboleth_b200.ops import standin_expert

    torch.cuda.set_device(0)
    spec = MoESpec(capacity=128, hidden=1024, top_k=4, experts=32, ranks=1)
    g = torch.Generator(device="cuda").manual_seed(3)
    x = torch.randn(100, 1024, generator=g, device="cuda").to(torch.bfloat16)
    logits = torch.randn(100, 32, generator=g, device="cuda")
    launched = {}
    with ab.World(0, 1, device=0) as world:
        world.connect_all("p2p")
        # hidden 1024: 100 records are ~100 KiB per peer, one lane of the seed profile, 16 of the fine one
        fine = {"p2p": EndpointProfile("test:fine-grained", "p2p", "B200", "none", "NV18", 4096, 16, 4),
                "proxy": SEED_PROFILES["B200_HOSTRING"]}
        for name, profiles in (("seed", None), ("fine", fine)):
            plan = compile_moe_plan(spec, world, profiles=profiles)
            slot = NativeMoESlot.create(world, spec, tag=f"bind-{name}", plan=plan)
            res = slot.dispatch(x, logits=logits)
            standin_expert(res.expert_input, res.expert_scales, slot.expert_output, res.expert_ids,
                           res.expert_weights, res.expert_pos, res.recv_counts, world=1, capacity=128, group=128)
            out = slot.combine(slot.expert_output).float()
            torch.cuda.synchronize()
            slot.check()
            expected, tol = standin_layer_reference(x, slot.topk_ids[:100].long(), slot.topk_weights[:100], fp8=True)
            assert bool(((out - expected).abs().amax(-1) <= tol).all())
            launched[name] = slot.manifest()
    seed, fine = launched["seed"], launched["fine"]
    assert seed["plan_binding"]["by_warp"] is False and fine["plan_binding"]["by_warp"] is True
    assert seed["launched"]["dispatch"]["by_warp"] is False and seed["launched"]["dispatch"]["grid"] == 100
    assert fine["launched"]["dispatch"]["by_warp"] is True and fine["launched"]["dispatch"]["grid"] == 100
    assert seed["launched"]["combine"]["send_warps"] == 7 and fine["launched"]["combine"]["send_warps"] == 3
    assert seed["launched"]["combine"]["grid"] != fine["launched"]["combine"]["grid"]
