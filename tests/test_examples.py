"""The programs under examples/ keep working: compile-only forms on CPU, full runs on one GPU."""
import os
import subprocess
import sys
from pathlib import Path

import pytest

EXAMPLES = Path(__file__).resolve().parent.parent / "examples"


def _run(script, *args, cache):
    env = {**os.environ, "ABOLETH_CACHE_DIR": str(cache)}
    return subprocess.run([sys.executable, str(EXAMPLES / script), *args], capture_output=True, text=True,
                          env=env, timeout=600)


@pytest.mark.parametrize("transport", ["p2p", "proxy"])
def test_tier2_chain_compiles_and_reports_the_passes(transport, tmp_path):
    proc = _run("tier2_chain.py", "--compile-only", "--transport", transport, cache=tmp_path)
    assert proc.returncode == 0, proc.stderr
    lines = proc.stdout.splitlines()
    assert sum(line.startswith(("chained", "unchained")) for line in lines) == 4
    naive = next(line for line in lines if line.startswith("unchained passes=none"))
    tuned = next(line for line in lines if line.startswith("unchained passes=default"))
    if transport == "p2p":
        assert "system_fences=7" in naive and "system_fences=0" in tuned and "barriers=1 " in tuned
    else:
        assert "submissions=8" in naive and "submissions=2" in tuned


def test_tier1_client_compiles_against_the_device_library(tmp_path):
    proc = _run("tier1_client.py", "--compile-only", cache=tmp_path)
    assert proc.returncode == 0, proc.stderr
    assert "compiled tier1_client.cu" in proc.stdout


@pytest.mark.gpu
@pytest.mark.parametrize("script,args", [
    ("tier2_chain.py", ()), ("tier2_chain.py", ("--transport", "proxy")), ("tier1_client.py", ()),
    ("moe_layer.py", ()), ("moe_layer.py", ("--bf16",)), ("kv_push.py", ()), ("tp_fused.py", ()),
    ("vllm_modular_moe.py", ()), ("block_scaled_gemm.py", ()), ("fp8_experts.py", ())])
def test_examples_run_on_one_gpu(script, args, tmp_path):
    proc = _run(script, *args, cache=tmp_path)
    assert proc.returncode == 0, proc.stdout + proc.stderr


@pytest.mark.parametrize("transport", ["rdma", "p2p"])
def test_planned_phase_example_splices_and_compiles(transport, tmp_path):
    proc = _run("planned_phase.py", "--transport", transport, cache=tmp_path)
    assert proc.returncode == 0, proc.stderr
    assert "spliced wait: planned_wait %s.p0 interval=4 iteration=it queue_capacity=32" in proc.stdout
    assert "pred=(((it) & 3) == 3)" in proc.stdout  # completes once per planned interval
