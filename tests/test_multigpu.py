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
