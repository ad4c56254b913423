"""Mixtral-style EP model on one GPU (EP = 1): the MoE layer against an fp32 restatement."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_moe_layer_and_generate_tiny():
    import aboleth_b200 as ab
    from aboleth_b200.models import MixtralConfig, MixtralEP

    cfg = MixtralConfig(layers=2, hidden=256, experts=4, top_k=2, ffn=512, heads=4, kv_heads=2,
                        vocab=128, max_seq=64)
    with ab.World(0, 1, device=0) as world:
        world.connect_all("p2p")
        model = MixtralEP(cfg, world, max_batch=4, max_prompt=16, seed=3)
        g = torch.Generator(device="cuda").manual_seed(1)
        x = torch.randn(37, 256, generator=g, device="cuda").to(torch.bfloat16)
        layer = model.layers[0]
        got = model.moe_layer(x, layer).float()
        want = model.reference_moe_layer(x, layer, layer["w13"], layer["w2"])
        torch.cuda.synchronize()
        model.check()
        rel = ((got - want).norm() / want.norm()).item()
        assert rel < 2e-2, rel
        # decode-sized call selects the small variant and still matches
        got2 = model.moe_layer(x[:3].contiguous(), layer).float()
        assert ((got2 - want[:3]).norm() / want[:3].norm()).item() < 2e-2
        prompts = torch.randint(0, 128, (4, 16), generator=g, device="cuda")
        out = model.generate(prompts, 5)
        torch.cuda.synchronize()
        model.check()
        assert out.shape == (4, 5) and int(out.min()) >= 0 and int(out.max()) < 128
        # greedy decoding is deterministic
        assert torch.equal(out, model.generate(prompts, 5))
        # the decode attention path agrees with a prefill that includes the same position
        full = model.forward(prompts, 0)
        model.forward(prompts[:, :15].contiguous(), 0)
        step = model.forward(prompts[:, 15:16].contiguous(), 15)
        torch.cuda.synchronize()
        assert ((full - step).norm() / full.norm()).item() < 3e-2


def test_decode_graph_replays_the_eager_step():
    import aboleth_b200 as ab
    from aboleth_b200.models import MixtralConfig, MixtralEP

    cfg = MixtralConfig(layers=2, hidden=256, experts=4, top_k=2, ffn=512, heads=4, kv_heads=2,
                        vocab=128, max_seq=64)
    with ab.World(0, 1, device=0) as world:
        world.connect_all("p2p")
        model = MixtralEP(cfg, world, max_batch=4, max_prompt=16, seed=3)
        g = torch.Generator(device="cuda").manual_seed(2)
        prompts = torch.randint(0, 128, (4, 16), generator=g, device="cuda")
        with torch.no_grad():
            eager = model.generate(prompts, 6)
            model.enable_decode_graph()
            # the capture ran decode steps at position 0 of the cache: prefill again, then replay
            graphed = model.generate(prompts, 6)
            first = model.forward(prompts, 0).argmax(-1)
            a = model.forward(first[:, None], 16).clone()
            model.forward(prompts, 0)
            b = model.decode(first[:, None], 16).clone()
        torch.cuda.synchronize()
        model.check()
        assert torch.equal(eager, graphed)
        assert ((a - b).norm() / a.norm()).item() < 2e-2


def test_fp8_experts_run_block_scaled_end_to_end():
    """e4m3 dispatch with power-of-two 1 x 128 scales -> permute with scales -> grouped block-scaled
    GEMMs against e4m3 weights with 128 x 128 scales -> combine.  The oracle multiplies the
    dequantised weights in fp32; the difference is the e4m3 rounding of the activations."""
    import aboleth_b200 as ab
    from aboleth_b200.models import MixtralConfig, MixtralEP
    from aboleth_b200.ops import check_gemm_status

    cfg = MixtralConfig(layers=1, hidden=256, experts=4, top_k=2, ffn=512, heads=4, kv_heads=2,
                        vocab=128, max_seq=64)
    with ab.World(0, 1, device=0) as world:
        world.connect_all("p2p")
        model = MixtralEP(cfg, world, max_batch=4, max_prompt=16, seed=3, fp8_experts=True)
        g = torch.Generator(device="cuda").manual_seed(1)
        x = torch.randn(37, 256, generator=g, device="cuda").to(torch.bfloat16)
        layer = model.layers[0]
        w13, w2 = model.dequantised_experts(layer)
        for tokens in (37, 3):     # the prefill variant, then the decode-sized one
            got = model.moe_layer(x[:tokens].contiguous(), layer).float()
            want = model.reference_moe_layer(x[:tokens], layer, w13, w2)
            torch.cuda.synchronize()
            model.check()
            check_gemm_status("cuda")
            rel = ((got - want).norm() / want.norm()).item()
            assert rel < 6e-2, rel
        out = model.generate(torch.randint(0, 128, (4, 16), generator=g, device="cuda"), 3)
        torch.cuda.synchronize()
        model.check()
        check_gemm_status("cuda")
        assert out.shape == (4, 3)
