"""Two-GPU tests: one process per GPU, bring-up over TcpStoreBootstrap on 127.0.0.1.

Peer memory is mapped through CUDA IPC; kernels on different GPUs wait on each
other's flags (bounded).  A rank that withholds its send makes the peer's wait
expire with status 1 - the failure is made on the host, no GPU is faulted.
"""
import os

import pytest
import torch

from tests._ranks import run_ranks

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]


def _setup(rank, world_size):
    import aboleth_b200 as ab

    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    boot = ab.TcpStoreBootstrap.from_env(timeout=60)
    world = ab.World(rank, world_size, device=rank, bootstrap=boot)
    world.connect_all("p2p")
    return ab, boot, world


def _alltoall_rank(rank, world_size, nbytes, lanes, mode):
    ab, boot, world = _setup(rank, world_size)
    from aboleth_b200.ops import alltoall, check_payload, fill_payload

    n = world_size
    arena = world.runtime.allocate(2 * n * nbytes + n * lanes * 8)
    reg = world.register(arena)
    table = world.exchange_regions([
        world.region("recv", reg, offset=n * nbytes, length=n * nbytes),
        world.region("flags", reg, offset=2 * n * nbytes, length=n * lanes * 8)], tag="t")
    flags = arena[2 * n * nbytes:].view(torch.int64)
    status = torch.zeros(2, dtype=torch.int64, device="cuda")
    for p in range(n):
        fill_payload(arena[p * nbytes:], nbytes, 5, rank, p)
    torch.cuda.synchronize()
    boot.barrier("filled")
    alltoall(arena, table.addresses("recv"), table.addresses("flags"), flags, status, stride=nbytes,
             nbytes=nbytes, epoch0=0, rank=rank, world=n, lanes=lanes, rounds=4, chain=2, mode=mode)
    errors = torch.zeros(1, dtype=torch.int64, device="cuda")
    for s in range(n):
        if s != rank:
            check_payload(arena[n * nbytes + s * nbytes:], nbytes, 5, s, rank, errors)
    torch.cuda.synchronize()
    boot.barrier("done")
    out = (int(errors.item()), status.tolist(), flags.view(n, lanes).tolist())
    world.close()
    return out


@pytest.mark.parametrize("mode", ["vector", "bulk"])
def test_alltoall_two_gpus(mode):
    results = run_ranks(_alltoall_rank, 2, 1 << 20, 8, mode, timeout=180)
    for rank in range(2):
        kind, value = results[rank]
        assert kind == "ok", value
        errors, status, flags = value
        assert errors == 0 and status == [0, 0]
        assert flags[1 - rank] == [4] * 8 and flags[rank] == [0] * 8


def _ep_rank(rank, world_size, withhold):
    ab, boot, world = _setup(rank, world_size)
    from aboleth_b200.moe import MoESpec
    from aboleth_b200.moe.reference import standin_layer_reference
    from aboleth_b200.parallel import ExpertParallelLayer

    spec = MoESpec(capacity=64, hidden=1024, top_k=4, experts=16, ranks=world_size)
    layer = ExpertParallelLayer(world, spec, tag="ep")
    g = torch.Generator(device="cuda").manual_seed(10 + rank)
    x = torch.randn(48 + rank, 1024, generator=g, device="cuda").to(torch.bfloat16)
    logits = torch.randn(48 + rank, 16, generator=g, device="cuda")
    boot.barrier("ready")
    if withhold and rank == 1:
        boot.barrier("after")
        world.close()
        return "withheld"
    worst = 0.0
    for _ in range(1 if withhold else 3):
        out = layer.forward(x, logits).float()
        torch.cuda.synchronize()
        if withhold:
            break
        layer.check()
        n = x.shape[0]
        expected, tol = standin_layer_reference(x, layer.slot.topk_ids[:n].long(),
                                                layer.slot.topk_weights[:n], fp8=True)
        worst = max(worst, float(((out - expected).abs().amax(-1) / tol).max()))
    status = layer.slot.status.tolist()
    boot.barrier("after")
    world.close()
    return worst, status


def test_ep_layer_two_gpus_matches_oracle():
    results = run_ranks(_ep_rank, 2, False, timeout=180)
    for rank in range(2):
        kind, value = results[rank]
        assert kind == "ok", value
        worst, status = value
        assert worst <= 1.0 and status == [0, 0]


def test_peer_that_never_sends_times_out_with_status_1():
    results = run_ranks(_ep_rank, 2, True, timeout=180)
    assert results[1] == ("ok", "withheld")
    kind, value = results[0]
    assert kind == "ok", value
    _, status = value
    assert status[0] == 1 and status[1] == 0x1000 + 1  # dispatch wait on rank 1 gave up


def _kv_pull_rank(rank, world_size):
    """Rank 0 plays the prefill engine (its caches hold the data), rank 1 pulls remapped blocks."""
    ab, boot, world = _setup(rank, world_size)
    from aboleth_b200.integrations import VLLMKVPeerRuntime

    runtime = VLLMKVPeerRuntime(rank=rank, world_size=2, device=rank, world=world)
    g = torch.Generator(device="cuda").manual_seed(7)  # same seed: rank 1 knows what rank 0 holds
    reference = {f"layer{i}": torch.randint(0, 255, (32, 2, 8, 128), generator=g, device="cuda",
                                            dtype=torch.uint8) for i in range(5)}
    caches = {k: (v.clone() if rank == 0 else torch.zeros_like(v)) for k, v in reference.items()}
    runtime.register_kv_caches(caches, consumer_order=tuple(caches))
    boot.barrier("registered")
    local_ids, remote_ids = [20, 21, 22, 3], [4, 5, 6, 30]
    ok = True
    if rank == 1:
        ticket = runtime.start_layered_pull_blocks(local_block_ids=local_ids, remote_block_ids=remote_ids,
                                                   remote_rank=0)
        ticket.completion.synchronize()
        runtime.check()
        for name, cache in caches.items():
            ok = ok and bool(torch.equal(cache[local_ids], reference[name][remote_ids]))
            rest = [b for b in range(32) if b not in local_ids]
            ok = ok and int(cache[rest].max().item()) == 0
    boot.barrier("pulled")   # rank 0 keeps its caches mapped until rank 1 has read them
    out = (ok, runtime.last_run_count, runtime.last_physicalization)
    runtime.close()
    world.close()
    return out


def test_kv_pull_between_two_engines():
    results = run_ranks(_kv_pull_rank, 2, timeout=180)
    for rank in range(2):
        kind, value = results[rank]
        assert kind == "ok", value
    ok, runs, physical = results[1][1]
    assert ok and runs == 2 and physical.endswith("generated_p2p")


def _probe_rank(rank, world_size):
    ab, boot, world = _setup(rank, world_size)
    from aboleth_b200.endpoint_probe import calibrate

    profile, result = calibrate(world, fit_bytes=(65536, 1 << 20, 4 << 20), holdout_bytes=(8 << 20,),
                                lanes=(1, 4, 16), warps=(1, 8), trials=2, tag="probe")
    out = (None if profile is None else (profile.max_lanes, profile.sender_warps), result.get("reason"),
           result["world"]["senders"] if "world" in result else 0)
    boot.barrier("probed")
    world.close()
    return out


def test_endpoint_probe_two_gpus():
    results = run_ranks(_probe_rank, 2, timeout=180)
    for rank in range(2):
        kind, value = results[rank]
        assert kind == "ok", value
        profile, reason, senders = value
        assert reason is None and senders == 2
        assert profile is None or profile[0] in (4, 16)
    assert results[0][1] == results[1][1]  # the fit uses world rates: every rank derives the same profile


def _tp_rank(rank, world_size, multicast):
    """Both fused TP kernels on real peers, bf16 and block-scaled e4m3; with ``multicast`` the
    all-gather pushes through an NVLink multicast mapping (``multimem.st``)."""
    ab, boot, world = _setup(rank, world_size)
    import torch.distributed as dist

    from aboleth_b200.ops import pack_scales_mx
    from aboleth_b200.parallel import AllGatherGemm, GemmReduceScatter
    from aboleth_b200.symmetric import multicast_supported

    if multicast:
        if not multicast_supported():
            world.close()
            return "no multicast on this fabric"
        port = int(os.environ["MASTER_PORT"]) + 1
        dist.init_process_group("nccl", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world_size,
                                device_id=torch.device("cuda", rank))
    m_local, k, n = 512, 1024, 520
    g = torch.Generator(device="cuda").manual_seed(11)            # same seed: every rank knows every shard
    shards = [torch.randint(-2, 3, (m_local, k), generator=g, device="cuda").float() for _ in range(world_size)]
    scales = [torch.exp2(torch.randint(-2, 3, (m_local, k // 128), generator=g, device="cuda").float())
              for _ in range(world_size)]
    b = torch.randint(-2, 3, (n, k), generator=g, device="cuda").float()
    b_s = torch.exp2(torch.randint(-2, 3, (-(-n // 128), k // 128), generator=g, device="cuda").float())
    ag = (AllGatherGemm.create_multicast if multicast else AllGatherGemm.create)(world, m_local, k)
    used_multicast = bool(ag.multicast[0])
    boot.barrier("created")
    fp8 = torch.float8_e4m3fn
    ok = True
    # bf16: small integers are exact in bf16 and in the fp32 accumulator
    full = torch.cat(shards)
    for _ in range(3):
        out = ag(shards[rank].to(torch.bfloat16), b.to(torch.bfloat16))
        torch.cuda.synchronize()
        boot.barrier("ag")
    ag.check()
    ok = ok and bool(torch.equal(out, (full @ b.t()).to(torch.bfloat16)))
    # block-scaled e4m3: the shard crosses with its scale-factor atoms
    b_full = b * b_s.repeat_interleave(128, dim=0)[:n].repeat_interleave(128, dim=1)
    a_full = torch.cat([shards[r] * scales[r].repeat_interleave(128, dim=1) for r in range(world_size)])
    for _ in range(2):
        out = ag.mx(shards[rank].to(fp8), pack_scales_mx(scales[rank], m_local, k, weight=False), b.to(fp8),
                    pack_scales_mx(b_s, n, k, weight=True))
        torch.cuda.synchronize()
        boot.barrier("ag_mx")
    ag.check()
    ok = ok and bool(torch.equal(out, (a_full @ b_full.t()).to(torch.bfloat16)))
    if not multicast:
        rs = GemmReduceScatter.create(world, m_local, n)
        gk = torch.Generator(device="cuda").manual_seed(100 + rank)
        a_part = torch.randint(-2, 3, (world_size * m_local, k), generator=gk, device="cuda").float()
        a_sc = torch.exp2(torch.randint(-2, 3, (world_size * m_local, k // 128), generator=gk, device="cuda").float())
        for _ in range(2):
            got = rs.mx(a_part.to(fp8), pack_scales_mx(a_sc, world_size * m_local, k, weight=False), b.to(fp8),
                        pack_scales_mx(b_s, n, k, weight=True))
            torch.cuda.synchronize()
            boot.barrier("rs_mx")
        rs.check()
        partial = ((a_part * a_sc.repeat_interleave(128, dim=1)) @ b_full.t()).to(torch.bfloat16).float()
        gathered = [torch.zeros_like(partial) for _ in range(world_size)]
        # the oracle needs every rank's partial: exchange them through the store as bytes
        blobs = boot.all_gather("partials", partial.cpu().numpy().tobytes())
        import numpy as np
        for r in range(world_size):
            gathered[r] = torch.from_numpy(np.frombuffer(blobs[r], dtype=np.float32).copy()).view_as(partial).cuda()
        want = sum(gathered)[rank * m_local:(rank + 1) * m_local].to(torch.bfloat16)
        ok = ok and bool(torch.equal(got, want))
    boot.barrier("done")
    if multicast:
        ag._arena.close()
        dist.destroy_process_group()
    world.close()
    return ok, used_multicast


def test_fused_tp_kernels_two_gpus_bf16_and_block_scaled():
    results = run_ranks(_tp_rank, 2, False, timeout=240)
    for rank in range(2):
        kind, value = results[rank]
        assert kind == "ok", value
        assert value == (True, False)


def test_all_gather_gemm_pushes_through_nvlink_multicast():
    results = run_ranks(_tp_rank, 2, True, timeout=240)
    for rank in range(2):
        kind, value = results[rank]
        assert kind == "ok", value
    if results[0][1] == "no multicast on this fabric":
        pytest.skip("no NVLink multicast on this fabric")
    for rank in range(2):
        ok, used = results[rank][1]
        assert ok
    # the mapping is there whenever the fabric offers one; without it the same call falls back to peer stores
    assert results[0][1][1] == results[1][1][1]
