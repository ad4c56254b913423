"""Standalone C++ arm of the Tier-1 ladder: builds for sm_100a anywhere, runs in loopback on one GPU."""
import importlib.util
from pathlib import Path

import pytest

_PATH = Path(__file__).resolve().parent.parent / "benchmarks" / "native_bench.py"


def _driver():
    spec = importlib.util.spec_from_file_location("native_bench", _PATH)
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    return module


def test_builds_and_reports_no_gpu_as_77():
    import torch

    driver = _driver()
    assert driver.build().exists()
    if not torch.cuda.is_available():
        code, rows = driver.run(["--iters", "4", "--warmup", "1"])
        assert code == 77 and rows == []


def test_nccl_host_arm_builds_and_needs_two_gpus():
    import torch

    driver = _driver()
    try:
        binary = driver.build_nccl()
    except RuntimeError as error:
        if "not installed" in str(error) or "no nccl.h" in str(error):
            pytest.skip(str(error))
        raise
    assert binary.exists()
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        code, rows = driver.run_nccl(["--iters", "4", "--warmup", "3"])
        assert code == 77 and rows == []


@pytest.mark.gpu
def test_loopback_ladder_on_one_gpu():
    driver = _driver()
    code, rows = driver.run(["--gpus", "1", "--iters", "50", "--warmup", "5", "--bytes", "4096"])
    assert code == 0, rows
    by_name = {row["bench"]: row for row in rows}
    assert set(by_name) == {"pingpong", "window", "alltoall"}
    assert by_name["pingpong"]["loopback"] and 0 < by_name["pingpong"]["round_trip_us"]["p50"] < 1000
    assert by_name["window"]["gbs_per_direction"] > 0
    assert by_name["alltoall"]["wrong_bytes"] == 0


@pytest.mark.gpu
def test_two_ranks_on_two_gpus():
    import torch

    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    driver = _driver()
    code, rows = driver.run(["--gpus", "2", "--iters", "50", "--warmup", "5", "--bytes", "65536"])
    assert code == 0, rows
    by_name = {row["bench"]: row for row in rows}
    assert not by_name["pingpong"]["loopback"] and by_name["alltoall"]["wrong_bytes"] == 0
    assert by_name["alltoall"]["busbw_gbs"] > 0
