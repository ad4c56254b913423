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
