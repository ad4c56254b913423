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
