"""A Tier-1 client built with -DABOLETH_DEBUG_BOUNDS, run on a GPU: a put inside the registered
window is carried out, a put outside it is skipped and reported, nothing traps.  Every address the
client could touch lies inside one allocation of this test, so even an unchecked write would land
in memory the test owns."""
import ctypes
import shutil
import subprocess
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu

PKG = Path(__file__).resolve().parent.parent / "aboleth_b200"

CLIENT = r'''
#include "aboleth/device.cuh"

__global__ void client(const std::uint64_t *endpoints, unsigned long long *status, unsigned long long dst,
                       unsigned long long src, unsigned long long flag, const aboleth::debug::Window *windows,
                       unsigned count, unsigned long long *violation, unsigned long long outside) {
    aboleth::DeviceContext ctx{endpoints, nullptr, status};
    ctx.bounds = aboleth::debug::Bounds{windows, count, violation};
    // inside the window: carried out and published
    aboleth::put_signal(ctx, 0, aboleth::RemoteRegion{dst, 0}, aboleth::LocalRegion{src, 0}, 1024,
                        aboleth::RemoteRegion{flag, 0}, 5);
    // outside every window: refused before any byte is stored
    aboleth::put(ctx, 0, aboleth::RemoteRegion{outside, 0}, aboleth::LocalRegion{src, 0}, 512);
}

extern "C" int run_client(const std::uint64_t *endpoints, unsigned long long *status, unsigned long long dst,
                          unsigned long long src, unsigned long long flag, const void *windows, unsigned count,
                          unsigned long long *violation, unsigned long long outside, cudaStream_t stream) {
    client<<<1, 1, 0, stream>>>(endpoints, status, dst, src, flag,
                                static_cast<const aboleth::debug::Window *>(windows), count, violation, outside);
    return static_cast<int>(cudaGetLastError());
}
'''


def test_out_of_window_put_is_skipped_and_reported(tmp_path):
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(nvcc).exists():
        pytest.skip("needs nvcc")
    source = tmp_path / "client.cu"
    source.write_text(CLIENT)
    library = tmp_path / "libclient.so"
    subprocess.run([nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-std=c++17", "-DABOLETH_DEBUG_BOUNDS",
                    f"-I{PKG / 'include'}", "-shared", "-Xcompiler", "-fPIC", str(source), "-o", str(library)],
                   check=True)
    lib = ctypes.CDLL(str(library))
    lib.run_client.restype = ctypes.c_int
    lib.run_client.argtypes = [ctypes.c_void_p] * 2 + [ctypes.c_uint64] * 3 + [ctypes.c_void_p, ctypes.c_uint,
                                                                                ctypes.c_void_p, ctypes.c_uint64,
                                                                                ctypes.c_void_p]
    torch.cuda.set_device(0)
    arena = torch.zeros(16384, dtype=torch.uint8, device="cuda")      # destination side, all owned here
    src = torch.arange(1024, device="cuda").to(torch.uint8)
    flag = torch.zeros(1, dtype=torch.int64, device="cuda")
    status = torch.zeros(2, dtype=torch.int64, device="cuda")
    violation = torch.zeros(3, dtype=torch.int64, device="cuda")
    # kind bits 1 = peer memory; the handle itself is not dereferenced by a peer-memory put
    endpoints = torch.tensor([arena.data_ptr() | 1], dtype=torch.int64, device="cuda")
    windows = torch.tensor([arena.data_ptr(), 4096, flag.data_ptr(), 8], dtype=torch.int64, device="cuda")
    outside = arena.data_ptr() + 8192
    rc = lib.run_client(endpoints.data_ptr(), status.data_ptr(), arena.data_ptr(), src.data_ptr(), flag.data_ptr(),
                        windows.data_ptr(), 2, violation.data_ptr(), outside,
                        torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()
    assert torch.equal(arena[:1024], src) and int(flag.item()) == 5      # the legal chain went through
    assert int(arena[4096:].max().item()) == 0                             # the refused put stored nothing
    assert status.tolist()[0] == 3                                         # Status::Malformed
    assert violation.tolist() == [outside, 512, 1]
