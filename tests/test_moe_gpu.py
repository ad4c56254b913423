"""Fused EP dispatch/combine and the standalone MoE kernels against fp32 PyTorch oracles.

Several ranks are emulated on one GPU (LocalMoEGroup): every rank's send half
runs before any rank's receive half, so no kernel ever waits on another launch.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _inputs(spec, n_per_rank, seed, device, integer=False):
    g = torch.Generator(device="cpu").manual_seed(seed)
    toks, ids, wts = [], [], []
    for r in range(spec.ranks):
        n = n_per_rank[r]
        if integer:
            x = torch.randint(-4, 5, (n, spec.hidden), generator=g).float()
        else:
            x = torch.randn(n, spec.hidden, generator=g)
        i = torch.stack([torch.randperm(spec.experts, generator=g)[:spec.top_k] for _ in range(n)]) \
            if n else torch.zeros(0, spec.top_k, dtype=torch.int64)
        w = torch.randint(1, 8, (n, spec.top_k), generator=g).float() / 8
        toks.append(x.to(torch.bfloat16).to(device))
        ids.append(i.to(torch.int32).to(device))
        wts.append(w.to(device))
    return toks, ids, wts


@pytest.mark.parametrize("by_warp", [False, True])
@pytest.mark.parametrize("value_type", ["f8E4M3FN", "bf16"])
@pytest.mark.parametrize("ranks,counts", [(1, [7]), (2, [16, 5]), (4, [0, 1, 9, 16])])
def test_dispatch_standin_combine_matches_oracle(value_type, ranks, counts, by_warp):
    from aboleth_b200.moe import LocalMoEGroup, MoESpec
    from aboleth_b200.moe.reference import standin_layer_reference
    from aboleth_b200.ops import standin_expert

    spec = MoESpec(capacity=16, hidden=256, top_k=2, experts=16, ranks=ranks, value_type=value_type)
    group = LocalMoEGroup(spec)
    for slot in group.slots:
        slot.by_warp = by_warp
    toks, ids, wts = _inputs(spec, counts, 1, "cuda")
    for r in range(ranks):  # some unused choices
        if counts[r] > 1:
            ids[r][0, 1] = -1
    for layer in range(2):  # second layer checks epoch advance and counter self-cleaning
        results = group.dispatch(toks, ids=ids, weights=wts)
        ys = []
        for r, res in enumerate(results):
            y = group.slots[r].expert_output
            standin_expert(res.expert_input, res.expert_scales, y, res.expert_ids,
                           res.expert_weights, res.expert_pos, res.recv_counts,
                           world=ranks, capacity=spec.capacity, group=spec.scale_group)
            ys.append(y)
        outs = group.combine(ys)
        torch.cuda.synchronize()
        group.check()
        for r in range(ranks):
            expected, tol = standin_layer_reference(toks[r], ids[r], wts[r], fp8=spec.fp8)
            err = (outs[r].float() - expected).abs().amax(dim=-1) if counts[r] else torch.zeros(0)
            assert bool((err.cpu() <= tol.cpu()).all()), (layer, r, err.max().item(), tol.min().item())
        assert [int(s.epoch.item()) for s in group.slots] == [layer + 2] * ranks


@pytest.mark.parametrize("by_warp", [False, True])
def test_dispatch_records_are_rank_deduplicated_and_exact(by_warp):
    from aboleth_b200.moe import LocalMoEGroup, MoESpec

    spec = MoESpec(capacity=8, hidden=128, top_k=4, experts=8, ranks=2, value_type="bf16")
    group = LocalMoEGroup(spec)
    for slot in group.slots:
        slot.by_warp = by_warp
    toks, ids, wts = _inputs(spec, [8, 3], 2, "cuda", integer=True)
    results = group.dispatch(toks, ids=ids, weights=wts)
    torch.cuda.synchronize()
    group.check()
    owners = spec.owners()
    for dst in range(2):
        res = results[dst]
        for src in range(2):
            want = {}
            for t in range(toks[src].shape[0]):
                mine = [(int(e), float(w)) for e, w in zip(ids[src][t].tolist(), wts[src][t].tolist())
                        if owners[e] == dst]
                if mine:
                    want[t] = mine
            assert int(res.recv_counts[src]) == len(want)
            meta = group.slots[dst].recv_meta[src * 8: src * 8 + len(want)].cpu()
            seen = set()
            for row in range(len(want)):
                t, nsel = int(meta[row, 0]), int(meta[row, 1])
                seen.add(t)
                got_ids = meta[row, 2:2 + nsel].tolist()
                got_w = meta[row, 2 + 4:2 + 4 + nsel].view(torch.float32).tolist()
                assert list(zip(got_ids, got_w)) == want[t]
                assert meta[row, 2 + nsel:2 + 4].tolist() == [-1] * (4 - nsel)
                assert torch.equal(res.expert_input[src * 8 + row].cpu(), toks[src][t].cpu())
                slot = int(group.slots[src].source_slots[t, dst])
                assert slot == row
            assert seen == set(want)
    counts = sum(r.expert_counts for r in results).cpu()
    expect = torch.zeros(8, dtype=torch.int32)
    for src in range(2):
        for e in ids[src].flatten().tolist():
            expect[e] += 1
    assert torch.equal(counts, expect)


@pytest.mark.parametrize("by_warp", [False, True])
def test_weighted_combine_with_permute_is_exact_for_integers(by_warp):
    from aboleth_b200.moe import LocalMoEGroup, MoESpec
    from aboleth_b200.ops import expert_offsets, permute

    spec = MoESpec(capacity=8, hidden=128, top_k=2, experts=4, ranks=2, value_type="bf16")
    group = LocalMoEGroup(spec)
    for slot in group.slots:
        slot.by_warp = by_warp
    toks, ids, _ = _inputs(spec, [8, 6], 3, "cuda", integer=True)
    wts = [torch.ones_like(i, dtype=torch.float32) for i in ids]
    results = group.dispatch(toks, ids=ids, weights=wts)
    ys, offs = [], []
    for r, res in enumerate(results):
        offsets, total = expert_offsets(res.expert_counts_by_source)
        x_perm = torch.zeros(spec.ranks * spec.capacity * spec.top_k, spec.hidden,
                             dtype=torch.bfloat16, device="cuda")
        permute(res.expert_input, x_perm, res.expert_ids, res.expert_pos, offsets, res.recv_counts,
                world=2, capacity=8)
        y = x_perm.clone()
        counts = res.expert_counts.cpu().tolist()
        o = offsets[0].cpu().tolist()  # row 0 of the table: where each expert's group starts
        for e in range(4):  # expert e multiplies by e + 1
            y[o[e]:o[e] + counts[e]] *= (e + 1)
        ys.append(y)
        offs.append(offsets)
        assert int(total.item()) == sum(counts)
    outs = group.combine(ys, expert_offsets=offs)
    torch.cuda.synchronize()
    group.check()
    for r in range(2):
        mult = (ids[r].float() + 1).sum(dim=-1, keepdim=True)
        assert torch.equal(outs[r].float(), toks[r].float() * mult)


def test_full_width_rows_by_warp_and_by_cta_agree():
    """hidden 7168 (14 warp steps, 56 scale groups): both send paths give identical records."""
    from aboleth_b200.moe import LocalMoEGroup, MoESpec

    spec = MoESpec(capacity=24, hidden=7168, top_k=8, experts=64, ranks=2)
    toks, ids, wts = _inputs(spec, [24, 17], 11, "cuda")
    outs = []
    for by_warp in (False, True):
        group = LocalMoEGroup(spec)
        for slot in group.slots:
            slot.by_warp = by_warp
        res = group.dispatch(toks, ids=ids, weights=wts)
        torch.cuda.synchronize()
        group.check()
        per_rank = []
        for r in range(2):
            slot = group.slots[r]
            rows = []
            for src in range(2):
                n = int(res[r].recv_counts[src])
                seg = slice(src * 24, src * 24 + n)
                order = torch.argsort(slot.recv_meta[seg, 0])
                rows.append((slot.recv_meta[seg][order].cpu(),
                             slot.recv_payload[seg].view(torch.uint8)[order].cpu()))
            per_rank.append(rows)
        outs.append(per_rank)
    for r in range(2):
        for src in range(2):
            assert torch.equal(outs[0][r][src][0], outs[1][r][src][0])
            assert torch.equal(outs[0][r][src][1], outs[1][r][src][1])


def test_fused_router_matches_standalone_and_torch():
    from aboleth_b200.moe import LocalMoEGroup, MoESpec
    from aboleth_b200.moe.reference import router_reference
    from aboleth_b200.ops import router_topk

    spec = MoESpec(capacity=32, hidden=256, top_k=8, experts=256, ranks=2)
    group = LocalMoEGroup(spec)
    g = torch.Generator().manual_seed(4)
    toks = [torch.randn(32, 256, generator=g).to(torch.bfloat16).cuda() for _ in range(2)]
    logits = [torch.randn(32, 256, generator=g).cuda() for _ in range(2)]
    results = group.dispatch(toks, logits=logits)
    torch.cuda.synchronize()
    group.check()
    for r in range(2):
        ref_ids, ref_w = router_reference(logits[r], 8)
        ids, w = router_topk(logits[r], 8)
        assert torch.equal(ids, ref_ids) and torch.allclose(w, ref_w, rtol=1e-4, atol=1e-6)
        assert torch.equal(results[r].topk_ids[:32], ref_ids)
        assert torch.allclose(results[r].topk_weights[:32], ref_w, rtol=1e-4, atol=1e-6)
    ids_r, w_r = router_topk(logits[0], 8, renormalize=True)
    assert torch.allclose(w_r.sum(-1), torch.ones(32, device="cuda"), atol=1e-5)


@pytest.mark.parametrize("round_scale", [False, True])
def test_quant_fp8_matches_reference(round_scale):
    from aboleth_b200.moe.reference import quant_fp8_reference
    from aboleth_b200.ops import quant_fp8

    x = (torch.randn(37, 7168, generator=torch.Generator().manual_seed(5)) * 3).to(torch.bfloat16).cuda()
    x[3] = 0  # amax floor path
    q, s = quant_fp8(x, round_scale=round_scale)
    q_ref, s_ref = quant_fp8_reference(x, round_scale=round_scale)
    assert torch.equal(s, s_ref)
    # The kernel divides approximately: a value on a rounding tie may land on the
    # neighbouring e4m3 code.  Anything else is an error.
    diff = (q.view(torch.uint8).to(torch.int16) - q_ref.view(torch.uint8).to(torch.int16)).abs()
    assert int(diff.max()) <= 1 and float((diff != 0).float().mean()) < 1e-3


def test_bounded_wait_reports_timeout_without_hanging():
    """A receive half whose peers never publish gives up and reports status 1."""
    from aboleth_b200.moe import LocalMoEGroup, MoESpec
    from aboleth_b200.ops.comm import tier1_exercise

    # Tier-1 wait with a 50 ms budget on a flag nobody sets.
    flag = torch.zeros(4, dtype=torch.int64, device="cuda")
    status = torch.zeros(2, dtype=torch.int64, device="cuda")
    endpoints = torch.tensor([flag.data_ptr() | 1], dtype=torch.int64, device="cuda")
    buf = torch.zeros(64, dtype=torch.uint8, device="cuda")
    tier1_exercise(endpoints, status, dst=buf.data_ptr(), src=buf.data_ptr() + 32,
                   flag=flag[1:].data_ptr(), inline_dst=flag[2:].data_ptr(),
                   wait_flag=flag.data_ptr(), epoch=1, wait_epoch=1, timeout_ns=50_000_000,
                   nbytes=16)
    torch.cuda.synchronize()
    assert status.tolist() == [1, 0x400]
    assert flag.tolist()[1:3] == [1, 4]
