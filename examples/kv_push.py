#!/usr/bin/env python
"""KV-cache page push: a producer copies the pages of a request into a consumer's slot, layer by
layer, and publishes one readiness epoch per layer; the consumer waits (bounded) per layer.

    python examples/kv_push.py            # one GPU: the rank is its own consumer
    torchrun --nproc-per-node 2 examples/kv_push.py   # rank 0 pushes to rank 1

Lifecycle of a request: begin_step (admission: a slot and an epoch) -> start_transfer -> wait_for_layer
-> poll == READY -> release.
"""
import argparse

from _world import close_world, open_world


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=8)
    ap.add_argument("--page-bytes", type=int, default=16384)
    args = ap.parse_args()
    world, distributed = open_world()

    import torch

    from aboleth_b200.kv import CompiledKVTransferManager, KVPoolLayout, TransferState

    layout = KVPoolLayout(layers=args.layers, blocks=64, page_bytes=args.page_bytes, slots=2, slot_pages=16)
    kv = CompiledKVTransferManager(world, layout)
    g = torch.Generator(device="cuda").manual_seed(world.rank)
    kv.pool.copy_(torch.randint(0, 255, kv.pool.shape, generator=g, device="cuda", dtype=torch.uint8))
    producer, consumer = 0, world.world_size - 1
    blocks = [3, 4, 5, 17, 9, 10, 11, 12]  # scattered page ids; contiguous runs travel as one copy
    record = kv.begin_step("request-0")
    if world.rank == producer:
        launched = kv.start_transfer("request-0", consumer=consumer, src_blocks=blocks, slot=record.slot,
                                     epoch=record.epoch)
        print(f"rank {world.rank}: pushed {len(blocks)} pages x {args.layers} layers in {launched} copies")
    status = 0
    if world.rank == consumer:
        for layer in range(args.layers):
            kv.wait_for_layer("request-0", layer, source=producer)
        torch.cuda.synchronize()
        state = kv.poll("request-0", source=producer)
        ok = state == TransferState.READY and kv.status.tolist() == [0, 0]
        if world.world_size == 1:  # the producer's pool is local: compare the bytes as well
            ok = ok and all(torch.equal(kv.slot_pages("request-0", layer)[: len(blocks)], kv.pool[layer, blocks])
                            for layer in range(args.layers))
        print(f"rank {world.rank}: state {state.name}, status {kv.status.tolist()}, {'ok' if ok else 'FAILED'}")
        status = 0 if ok else 1
    torch.cuda.synchronize()
    kv.release("request-0")
    close_world(world, distributed)
    return status


if __name__ == "__main__":
    raise SystemExit(main())
