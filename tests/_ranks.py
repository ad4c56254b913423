"""Spawn N CPU ranks that meet over a TcpStoreBootstrap on 127.0.0.1."""
import multiprocessing as mp
import os
import socket
import traceback


def free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _entry(fn, rank, world, port, queue, args):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1",
                      MASTER_PORT=str(port))
    try:
        queue.put((rank, "ok", fn(rank, world, *args)))
    except BaseException as error:  # noqa: BLE001
        queue.put((rank, "error", f"{type(error).__name__}: {error}\n{traceback.format_exc()}"))


def run_ranks(fn, world, *args, timeout=120, expect_ranks=None):
    ctx = mp.get_context("spawn")
    queue = ctx.Queue()
    port = free_port()
    ranks = range(world) if expect_ranks is None else expect_ranks
    procs = [ctx.Process(target=_entry, args=(fn, r, world, port, queue, args)) for r in ranks]
    for p in procs:
        p.start()
    results = {}
    try:
        for _ in procs:
            rank, kind, value = queue.get(timeout=timeout)
            results[rank] = (kind, value)
    finally:
        for p in procs:
            p.join(timeout=10)
            if p.is_alive():
                p.terminate()
    return results
