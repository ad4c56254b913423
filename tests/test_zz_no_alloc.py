"""The allocation-free KV push, called through its exported C symbol.

Collected last (file name) so that it also runs after every other GPU test has used the device.
Compares against the allocating entry point on two calls in a row.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

MAX_BATCHES = 4096


def _symbol():
    from aboleth_b200 import _native

    lib = _native.load("kernels")
    fn = lib.ab_kv_push_static
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_uint64, ctypes.c_int, ctypes.c_int,
                   ctypes.c_void_p, ctypes.c_void_p]
    return fn


def test_static_push_matches_allocating_push_twice():
    from aboleth_b200.kv import copy as kvcopy

    torch.cuda.set_device(0)
    fn = _symbol()
    stream = torch.cuda.current_stream().cuda_stream
    g = torch.Generator(device="cuda").manual_seed(7)
    page = 4096
    sizes = [page * 3, page, page * 8 + 16, 48, page * 2]  # one odd tail, one tiny run
    total = sum((s + 255) // 256 * 256 for s in sizes)
    src = torch.randint(0, 255, (total,), generator=g, device="cuda", dtype=torch.uint8)
    status = torch.zeros(2, dtype=torch.int64, device="cuda")
    for call, (epoch, workers) in enumerate([(1, 4), (2, 7)]):
        want = torch.zeros(total, dtype=torch.uint8, device="cuda")
        got = torch.zeros(total, dtype=torch.uint8, device="cuda")
        ready_want = torch.zeros(len(sizes), dtype=torch.int64, device="cuda")
        ready_got = torch.zeros(len(sizes), dtype=torch.int64, device="cuda")

        def records(dst, ready):
            out, at = [], 0
            for i, s in enumerate(sizes):
                out.append((src.data_ptr() + at, dst.data_ptr() + at, s, ready.data_ptr() + 8 * i))
                at += (s + 255) // 256 * 256
            return kvcopy.pack_batches(out, "cuda")

        arrivals = torch.zeros(len(sizes), dtype=torch.int32, device="cuda")
        kvcopy.push(records(want, ready_want), arrivals, len(sizes), epoch, workers=workers, threads=256,
                    status=status)
        batches = records(got, ready_got)
        rc = fn(batches.data_ptr(), len(sizes), epoch, workers, 256, status.data_ptr(), stream)
        assert rc == 0, (call, rc)
        torch.cuda.synchronize()
        assert status.tolist() == [0, 0]
        assert ready_got.tolist() == [epoch] * len(sizes) == ready_want.tolist()
        assert torch.equal(got, want)
        at = 0
        for s in sizes:  # exactly the run was written, nothing past it
            assert torch.equal(got[at:at + s], src[at:at + s])
            assert int(got[at + s:at + (s + 255) // 256 * 256].max().item() if s % 256 else 0) == 0
            at += (s + 255) // 256 * 256


def test_static_push_rejects_sizes_beyond_its_limit():
    torch.cuda.set_device(0)
    fn = _symbol()
    stream = torch.cuda.current_stream().cuda_stream
    status = torch.zeros(2, dtype=torch.int64, device="cuda")
    dummy = torch.zeros(32, dtype=torch.uint8, device="cuda")
    assert fn(dummy.data_ptr(), MAX_BATCHES + 1, 1, 1, 128, status.data_ptr(), stream) == -2
    assert fn(dummy.data_ptr(), 0, 1, 1, 128, status.data_ptr(), stream) == -1
    assert fn(dummy.data_ptr(), 1, 1, 1, 100, status.data_ptr(), stream) == -1
    assert fn(None, 1, 1, 1, 128, status.data_ptr(), stream) == -1
    torch.cuda.synchronize()
    assert status.tolist() == [0, 0]
