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
    assert proc.returncode == 0, (proc.stdout + proc.stderr)[-6000:]
    assert "failures: 0" in proc.stdout and "ThreadSanitizer" not in proc.stderr
