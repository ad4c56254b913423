"""Host-side native code under the compiler's sanitizers.

The reference has no sanitizer targets; its safety nets are verifiers and
differential tests.  Here the specializer (parser, verifier, passes, lowerings,
planners) runs over its golden corpus and over deterministic corruptions of it
with AddressSanitizer + UndefinedBehaviorSanitizer, and the host-proxy ring runs
a many-producer stress under ThreadSanitizer.  Both are plain CPU programs.
"""
import shutil
import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
PKG = ROOT / "aboleth_b200"
NATIVE = Path(__file__).resolve().parent / "native"

pytestmark = pytest.mark.skipif(shutil.which("g++") is None, reason="needs g++")


def _build(out: Path, sources, sanitize: str, extra=(), libs=()):
    cmd = ["g++", "-std=c++17", "-O1", "-g", f"-fsanitize={sanitize}", "-fno-omit-frame-pointer",
           f"-I{PKG / 'include'}", *extra, *map(str, sources), "-o", str(out), "-pthread", *libs]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0 and "sanitize" in proc.stderr and "cannot find" in proc.stderr:
        pytest.skip("the sanitizer runtime is not installed")
    assert proc.returncode == 0, proc.stderr[-4000:]


def _corpus(directory: Path) -> int:
    from aboleth_b200.compiler import goldens
    from aboleth_b200.compiler.driver import compile_program
    from aboleth_b200.compiler.options import compilation

    n = 0
    for case in goldens.CASES:
        for backend, passes in (("p2p", "default"), ("rdma", "default"), ("proxy", "none")):
            with compilation(backend, rank=0, world_size=2, passes=passes) as options:
                compiled = compile_program(goldens.CASES[case]())
                (directory / f"{n}.prog").write_text(compiled.source)
                (directory / f"{n}.opts").write_text(options.to_native())
                n += 1
    return n


def test_specializer_survives_corrupted_programs_under_asan_ubsan(tmp_path):
    exe = tmp_path / "spec_sanitize"
    spec = sorted((PKG / "csrc" / "spec").glob("*.cpp"))
    _build(exe, spec + [NATIVE / "spec_sanitize.cpp"], "address,undefined",
           extra=["-fno-sanitize-recover=undefined", f"-I{PKG / 'csrc' / 'spec'}"])
    cases = _corpus(tmp_path)
    from tests import test_compiler
    (tmp_path / "phase.kernel").write_text(test_compiler._KERNEL)
    (tmp_path / "phase.plan").write_text(test_compiler._PLAN)
    import json
    seeds = json.loads((Path(__file__).resolve().parent / "data" / "planner_requests.json").read_text())
    for i, seed in enumerate(seeds):
        (tmp_path / f"planner.{i}.kind").write_text(seed["kind"])
        (tmp_path / f"planner.{i}.req").write_text(seed["request"])
    proc = subprocess.run([str(exe), str(tmp_path), str(cases)], capture_output=True, text=True, timeout=900)
    assert proc.returncode == 0, (proc.stdout + proc.stderr)[-6000:]
    assert "refused" in proc.stdout and "ERROR" not in proc.stderr


def _cuda_home() -> Path:
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    return Path(nvcc).resolve().parent.parent


def test_proxy_ring_with_many_producers_is_race_free_under_tsan(tmp_path):
    cuda = _cuda_home()
    if not (cuda / "include" / "cuda_runtime.h").exists():
        pytest.skip("the CUDA headers are not installed")
    exe = tmp_path / "proxy_ring_stress"
    # The runtime's source is host C++ (no kernels): g++ compiles it as such.
    _build(exe, ["-x", "c++", PKG / "csrc" / "host" / "runtime_core.cu", NATIVE / "proxy_ring_stress.cpp"],
           "thread", extra=[f"-I{cuda / 'include'}"],
           libs=[f"-L{cuda / 'lib64'}", f"-Wl,-rpath,{cuda / 'lib64'}", "-lcudart", "-ldl"])
    proc = subprocess.run([str(exe)], capture_output=True, text=True, timeout=600)
    if "unexpected memory mapping" in proc.stderr:  # the sanitizer cannot place its shadow under this kernel's ASLR
        pytest.skip("ThreadSanitizer cannot start on this machine")
    assert proc.returncode == 0, (proc.stdout + proc.stderr)[-6000:]
    assert "failures: 0" in proc.stdout and "ThreadSanitizer" not in proc.stderr


def test_debug_bounds_rule_on_the_host_and_in_a_debug_build_of_a_client(tmp_path):
    """Debug builds of Tier-1 code refuse peer writes outside the registered windows: the rule is
    checked on the host (with UBSan), and a client compiles for sm_100a with and without it."""
    exe = tmp_path / "debug_bounds_host"
    _build(exe, [NATIVE / "debug_bounds_host.cpp"], "address,undefined", extra=["-fno-sanitize-recover=undefined"])
    proc = subprocess.run([str(exe)], capture_output=True, text=True, timeout=120)
    assert proc.returncode == 0 and "failures: 0" in proc.stdout, proc.stdout + proc.stderr
    nvcc = shutil.which("nvcc")
    if nvcc is None:
        pytest.skip("needs nvcc for the device half")
    client = tmp_path / "client.cu"
    client.write_text('''#include "aboleth/device.cuh"
__global__ void k(const std::uint64_t *eps, unsigned long long *status, unsigned long long dst,
                  unsigned long long src, unsigned long long flag, const void *windows, unsigned count,
                  unsigned long long *violation) {
    aboleth::DeviceContext ctx{eps, nullptr, status};
#ifdef ABOLETH_DEBUG_BOUNDS
    ctx.bounds = aboleth::debug::Bounds{static_cast<const aboleth::debug::Window *>(windows), count, violation};
#endif
    aboleth::put_signal(ctx, 1, aboleth::RemoteRegion{dst, 0}, aboleth::LocalRegion{src, 0}, 4096,
                        aboleth::RemoteRegion{flag, 0}, 1);
    aboleth::put_warp(ctx, aboleth::open(ctx, 1), aboleth::RemoteRegion{dst, 0}, aboleth::LocalRegion{src, 0}, 4096);
    aboleth::put_inline(ctx, 1, aboleth::RemoteRegion{dst, 0}, 7);
    aboleth::signal(ctx, 1, aboleth::RemoteRegion{flag, 0}, 2);
}
''')
    for define in ([], ["-DABOLETH_DEBUG_BOUNDS"]):
        subprocess.run([nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-std=c++17", *define,
                        f"-I{PKG / 'include'}", "-c", str(client), "-o", str(tmp_path / "client.o")], check=True)
