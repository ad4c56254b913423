"""Emitted Tier-2 kernels and the Tier-1 proxy kind, run on one GPU against itself."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _program(nbytes, chain, chained=True):
    from aboleth_b200.compiler import ProgramBuilder

    b = ProgramBuilder("selfloop", threads=128, args=[
        ("src", "ptr"), ("endpoints", "table"), ("dst_table", "table"), ("flag_table", "table"),
        ("my_flag", "ptr"), ("epoch", "u64")])
    e = b.endpoint("endpoints", 0)
    piece = nbytes // chain
    previous = None
    for c in range(chain):
        previous = b.put(e, b.remote("dst_table", 0, offset=c * piece), b.local(f"src + {c * piece}"),
                         bytes=piece, after=previous if chained else None)
    s = b.signal(e, b.remote("flag_table", 0), epoch="epoch", after=previous)
    b.wait_signal("my_flag", "epoch")
    b.wait(s)
    return b


@pytest.mark.parametrize("backend,chained", [("p2p", True), ("proxy", True), ("p2p", False), ("proxy", False)])
def test_emitted_chain_kernel_moves_data_and_publishes_once(backend, chained, tmp_path, monkeypatch):
    import aboleth_b200 as ab
    from aboleth_b200.compiler import LoadedKernel, build_artifact, compilation, compile_program

    monkeypatch.setenv("ABOLETH_CACHE_DIR", str(tmp_path))
    torch.cuda.set_device(0)
    runtime = ab.Runtime(0)
    try:
        endpoint = runtime.create_local_endpoint(ab.Transport(backend))
        nbytes = 1 << 16
        src = torch.arange(nbytes // 4, dtype=torch.int32, device="cuda").view(torch.uint8)
        dst = torch.zeros(nbytes, dtype=torch.uint8, device="cuda")
        flag = torch.zeros(1, dtype=torch.int64, device="cuda")
        status = torch.zeros(2, dtype=torch.int64, device="cuda")
        endpoints = torch.tensor([endpoint.handle], dtype=torch.int64, device="cuda")
        dst_table = torch.tensor([dst.data_ptr(), 0], dtype=torch.int64, device="cuda")
        flag_table = torch.tensor([flag.data_ptr(), 0], dtype=torch.int64, device="cuda")
        with compilation(backend, rank=0, world_size=1):
            compiled = compile_program(_program(nbytes, 8, chained))
        assert compiled.facts["commands"] == 9
        if chained:
            assert compiled.facts["batches"] == 1
        elif backend == "p2p":  # unchained puts share the signal's barrier and release
            assert compiled.facts["system_fences"] == 0 and compiled.facts["deferred_placements"] == 7
        else:                   # adjacent submissions to one endpoint merged
            assert compiled.facts["batches"] == 2
        kernel = LoadedKernel(build_artifact(compiled))
        for epoch in (1, 2):
            dst.zero_()
            torch.cuda.synchronize()
            kernel.launch(1, 128, [src.data_ptr(), endpoints.data_ptr(), dst_table.data_ptr(),
                                   flag_table.data_ptr(), flag.data_ptr(), epoch, status.data_ptr()],
                          stream=torch.cuda.current_stream().cuda_stream)
            torch.cuda.synchronize()
            assert status.tolist() == [0, 0]
            assert torch.equal(dst, src) and flag.item() == epoch
        if backend == "proxy":
            stats = endpoint.stats()
            per_launch = 1 if chained else 2
            assert stats["batches"] == 2 * per_launch and stats["commands"] == 18 and stats["bytes"] == 2 * nbytes
            assert endpoint.state()[:2] == (2 * per_launch, 2 * per_launch)
    finally:
        runtime.close()


def test_tier1_put_signal_through_the_proxy_ring_and_injected_failure():
    import aboleth_b200 as ab
    from aboleth_b200.ops import tier1_exercise

    torch.cuda.set_device(0)
    runtime = ab.Runtime(0)
    try:
        endpoint = runtime.create_local_endpoint(ab.Transport.RDMA)  # served by the ring
        src = torch.arange(1024, dtype=torch.int32, device="cuda").view(torch.uint8)
        dst = torch.zeros_like(src)
        cells = torch.zeros(4, dtype=torch.int64, device="cuda")
        status = torch.zeros(2, dtype=torch.int64, device="cuda")
        table = torch.tensor([0, endpoint.handle], dtype=torch.int64, device="cuda")
        tier1_exercise(table, status, dst=dst.data_ptr(), src=src.data_ptr(), flag=cells.data_ptr(),
                       inline_dst=cells[1:].data_ptr(), wait_flag=cells.data_ptr(), epoch=3, wait_epoch=3,
                       timeout_ns=2_000_000_000, nbytes=src.numel(), peer=1, pieces=4)
        torch.cuda.synchronize()
        assert status.tolist() == [0, 0] and torch.equal(dst, src) and cells.tolist()[:2] == [3, 10]
        # Host-side fault injection: the next batch retires with status 2 and quiet reports it.
        endpoint.inject_failure(ab.abi.STATUS_COMPLETION_FAILURE, 1)
        tier1_exercise(table, status, dst=dst.data_ptr(), src=src.data_ptr(), flag=cells[2:].data_ptr(),
                       inline_dst=cells[3:].data_ptr(), epoch=4, nbytes=64, peer=1)
        torch.cuda.synchronize()
        assert status.tolist()[0] == ab.abi.STATUS_COMPLETION_FAILURE
        assert endpoint.state()[2] == ab.abi.STATUS_COMPLETION_FAILURE
    finally:
        runtime.close()


def test_emitted_chain_and_handwritten_header_put_the_same_commands_on_the_ring(tmp_path, monkeypatch):
    """Differential: the kernel the specializer emits for "eight puts closed by one signal" and the
    hand-written Tier-1 header's put_many_signal must write the same batch into the proxy ring,
    command for command and byte for byte (addresses, sizes, keys, opcodes, the signal's value)."""
    import aboleth_b200 as ab
    from aboleth_b200.compiler import LoadedKernel, build_artifact, compilation, compile_program
    from aboleth_b200.ops import tier1_exercise

    monkeypatch.setenv("ABOLETH_CACHE_DIR", str(tmp_path))
    torch.cuda.set_device(0)
    runtime = ab.Runtime(0)
    try:
        nbytes, epoch = 1 << 16, 7
        src = torch.arange(nbytes // 4, dtype=torch.int32, device="cuda").view(torch.uint8)
        dst = torch.zeros(nbytes, dtype=torch.uint8, device="cuda")
        cells = torch.zeros(4, dtype=torch.int64, device="cuda")       # [flag, inline destination, ...]
        status = torch.zeros(2, dtype=torch.int64, device="cuda")

        # hand-written header: one inline put (its own batch), then put_many_signal of eight pieces
        by_hand = runtime.create_local_endpoint(ab.Transport.PROXY)
        handles = torch.tensor([by_hand.handle], dtype=torch.int64, device="cuda")
        tier1_exercise(handles, status, dst=dst.data_ptr(), src=src.data_ptr(), flag=cells[0:].data_ptr(),
                       inline_dst=cells[1:].data_ptr(), wait_flag=cells[0:].data_ptr(), epoch=epoch,
                       wait_epoch=epoch, nbytes=nbytes, peer=0, pieces=8)
        torch.cuda.synchronize()
        assert status.tolist() == [0, 0] and torch.equal(dst, src) and cells[0].item() == epoch
        hand_batches = by_hand.snapshot_queue()

        # emitted kernel: the same chain from the program builder, through its own endpoint
        dst.zero_()
        cells.zero_()
        emitted = runtime.create_local_endpoint(ab.Transport.PROXY)
        handles2 = torch.tensor([emitted.handle], dtype=torch.int64, device="cuda")
        dst_table = torch.tensor([dst.data_ptr(), 0], dtype=torch.int64, device="cuda")
        flag_table = torch.tensor([cells.data_ptr(), 0], dtype=torch.int64, device="cuda")
        with compilation("proxy", rank=0, world_size=1):
            kernel = LoadedKernel(build_artifact(compile_program(_program(nbytes, 8, chained=True))))
        kernel.launch(1, 128, [src.data_ptr(), handles2.data_ptr(), dst_table.data_ptr(), flag_table.data_ptr(),
                               cells.data_ptr(), epoch, status.data_ptr()],
                      stream=torch.cuda.current_stream().cuda_stream)
        torch.cuda.synchronize()
        assert status.tolist() == [0, 0] and torch.equal(dst, src) and cells[0].item() == epoch
        emitted_batches = emitted.snapshot_queue()

        chain = hand_batches[-1]                       # the batch of put_many_signal
        assert len(chain) == 9 and len(emitted_batches) == 1
        assert emitted_batches[0] == chain
    finally:
        runtime.close()
