"""KV page push on one GPU: a rank pushes page runs into its own slot storage."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_canonical_runs():
    from aboleth_b200.kv import canonicalize_block_runs

    assert canonicalize_block_runs([4, 5, 6, 9, 10, 2], [0, 1, 2, 3, 4, 7]) == [(4, 0, 3), (9, 3, 2), (2, 7, 1)]
    assert canonicalize_block_runs([1, 2], [5, 7]) == [(1, 5, 1), (2, 7, 1)]
    with pytest.raises(ValueError):
        canonicalize_block_runs([1], [1, 2])


def test_push_pages_publish_readiness_and_lifecycle():
    import aboleth_b200 as ab
    from aboleth_b200.kv import CompiledKVTransferManager, KVPoolLayout, TransferState

    torch.cuda.set_device(0)
    with ab.World(0, 1, device=0) as world:
        world.connect_all("p2p")
        layout = KVPoolLayout(layers=6, blocks=32, page_bytes=4096, slots=2, slot_pages=8)
        kv = CompiledKVTransferManager(world, layout)
        g = torch.Generator(device="cuda").manual_seed(0)
        kv.pool.copy_(torch.randint(0, 255, kv.pool.shape, generator=g, device="cuda", dtype=torch.uint8))
        record = kv.begin_step("req-1")
        assert record is not None and record.slot == 0 and record.epoch == 1
        blocks = [3, 4, 5, 17, 9, 10]
        launched = kv.start_transfer("req-1", consumer=0, src_blocks=blocks, slot=record.slot,
                                     epoch=record.epoch)
        assert launched == 6 * 3  # three runs per layer
        kv.wait_for_layer("req-1", 0, source=0)
        kv.wait_for_layer("req-1", 5, source=0)
        torch.cuda.synchronize()
        assert kv.status.tolist() == [0, 0]
        assert kv.poll("req-1", source=0) == TransferState.READY
        for layer in range(6):
            got = kv.slot_pages("req-1", layer)[: len(blocks)]
            assert torch.equal(got, kv.pool[layer, blocks])
        kv.release("req-1")
        # Slots are admission-controlled.
        assert kv.begin_step("a").slot == 0 and kv.begin_step("b").slot == 1 and kv.begin_step("c") is None
        kv.abort("a")
        assert kv.begin_step("c").slot == 0
        with pytest.raises(RuntimeError, match="not allowed"):
            kv.ledger.get("a").move(TransferState.READY)
        # A consumer whose producer never pushes gives up with status 1, it does not hang.
        from aboleth_b200.kv import copy as kvcopy
        kvcopy.wait_ready(kv.ready[0, 0, 0:1], 99, kv.status, timeout_ns=20_000_000)
        torch.cuda.synchronize()
        assert kv.status.tolist()[0] == 1 and kv.poll("c", source=0) == TransferState.FAILED


def test_engine_pull_runtime_on_one_device():
    """The decode side pulls remapped blocks of every layer; here both 'ranks' are one device, so the
    peer table is stood in by the local addresses (the kernels only see addresses)."""
    import aboleth_b200 as ab
    from aboleth_b200.integrations import VLLMKVPeerRuntime

    torch.cuda.set_device(0)

    class _Table:
        def __init__(self, caches):
            self.caches = caches

        def addresses(self, name):
            return [self.caches[name[3:]].data_ptr()] * 2

        def close(self):
            pass

    with ab.World(0, 1, device=0) as world:
        world.connect_all("p2p")
        runtime = VLLMKVPeerRuntime(rank=0, world_size=2, device=0, world=world)
        g = torch.Generator(device="cuda").manual_seed(5)
        layers = {f"layer{i}": torch.randint(0, 255, (64, 2, 16, 128), generator=g, device="cuda",
                                             dtype=torch.uint8) for i in range(6)}
        remote = {k: v.clone() for k, v in layers.items()}      # what the prefill rank holds
        world.exchange_regions = lambda regions, tag="": _Table(remote)
        runtime.register_kv_caches(layers, consumer_order=tuple(layers))
        assert runtime.plan.physicalization.direct_destination
        local_ids, remote_ids = [40, 41, 42, 7, 8, 60], [3, 4, 5, 20, 21, 9]
        before = {k: v.clone() for k, v in layers.items()}
        ticket = runtime.start_layered_pull_blocks(local_block_ids=local_ids, remote_block_ids=remote_ids,
                                                   remote_rank=1)
        assert set(ticket.layer_events) == set(layers)
        ticket.completion.synchronize()
        runtime.check()
        assert runtime.last_run_count == 3 and "generated_p2p" in runtime.last_physicalization
        for name, cache in layers.items():
            assert torch.equal(cache[local_ids], remote[name][remote_ids])
            untouched = [b for b in range(64) if b not in local_ids]
            assert torch.equal(cache[untouched], before[name][untouched])
        us = runtime.pull_blocks(local_block_ids=[0, 1], remote_block_ids=[62, 63], remote_rank=1)
        assert us > 0 and torch.equal(layers["layer3"][0:2], remote["layer3"][62:64])
        with pytest.raises(ValueError, match="outside the registered cache"):
            runtime.start_pull_blocks(local_block_ids=[64], remote_block_ids=[0], remote_rank=1)
        with pytest.raises(ValueError, match="other rank"):
            runtime.start_pull_blocks(local_block_ids=[1], remote_block_ids=[0], remote_rank=0)


def test_shared_readiness_cell_is_published_after_the_last_batch():
    """Eight batches of very different sizes publish ONE cell.  A consumer CTA of the same launch
    waits for the cell and sums the destinations at once: with one arrival counter per group the
    sum is the sources' sum every time; a counter per batch would publish after the smallest."""
    from aboleth_b200.kv import copy as kvcopy

    torch.cuda.set_device(0)
    g = torch.Generator(device="cuda").manual_seed(3)
    sizes = [4096, 8 << 20, 16384, 2 << 20, 256, 6 << 20, 65536, 1 << 20]
    workers = 16
    total = sum(sizes)
    src = torch.randint(1, 255, (total,), generator=g, device="cuda", dtype=torch.uint8)
    dst = torch.zeros(total, dtype=torch.uint8, device="cuda")
    cell = torch.zeros(1, dtype=torch.int64, device="cuda")
    observed = torch.zeros(1, dtype=torch.int64, device="cuda")
    status = torch.zeros(2, dtype=torch.int64, device="cuda")
    arrivals = torch.zeros(8, dtype=torch.int32, device="cuda")
    records, at = [], 0
    for s in sizes:
        records.append((src.data_ptr() + at, dst.data_ptr() + at, s, cell.data_ptr()))
        at += s
    batches = kvcopy.pack_batches(records, "cuda")
    group_of, group_target, groups = kvcopy.pack_groups([r[3] for r in records], workers, "cuda")
    assert groups == 1 and group_target.tolist() == [len(sizes) * workers]
    want = int(src.view(torch.int64).sum().item())
    for epoch in range(1, 201):
        dst.zero_()
        kvcopy.push_observed(batches, arrivals, len(sizes), epoch, workers=workers, threads=256,
                             status=status, cell=cell, observed=observed, group_of=group_of,
                             group_target=group_target)
        torch.cuda.synchronize()
        assert status.tolist() == [0, 0], (epoch, status.tolist())
        assert int(observed.item()) == want, epoch
        assert int(cell.item()) == epoch and arrivals.tolist() == [0] * 8
    assert torch.equal(dst, src)
