"""Execution contracts, KV lifecycle and profiles, record programs, compiled phases (CPU only)."""
import pytest

import aboleth_b200 as ab
from aboleth_b200.execution import (CapacityContract, ExecutionContract, ExecutionFallback, PaddingSemantics,
                                    RankControl, RuntimeGuard, compile_execution_plan)


def _contract(**over):
    args = dict(capacity=CapacityContract(64, True, PaddingSemantics.DEAD, True),
                rank_control=RankControl.LOCKSTEP,
                guards=(RuntimeGuard("count_within_capacity", ExecutionFallback.ERROR),
                        RuntimeGuard("contiguous", ExecutionFallback.EAGER)),
                fallback=ExecutionFallback.EXACT_AGREEMENT)
    args.update(over)
    return ExecutionContract(**args)


def test_fixed_capacity_needs_every_proof():
    contract = _contract()
    assert contract.fixed_capacity_legal
    decision = contract.resolve(10)
    assert (decision.mode, decision.capacity) == ("fixed_capacity", 64)
    # any missing proof falls back, with the live item count
    for change in (dict(rank_control=RankControl.DYNAMIC),
                   dict(capacity=CapacityContract(64, True, PaddingSemantics.PRESERVED, True)),
                   dict(capacity=CapacityContract(64, False, PaddingSemantics.DEAD, True)),
                   dict(capacity=CapacityContract(64, True, PaddingSemantics.DEAD, False))):
        weaker = _contract(**change)
        assert not weaker.fixed_capacity_legal
        assert weaker.resolve(10).mode == "exact_agreement" and weaker.resolve(10).capacity == 10
    assert contract.resolve(10, graph_stable_addresses=False).mode == "exact_agreement"
    assert contract.resolve(10, failed_guards=("contiguous",)).mode == "eager"
    with pytest.raises(RuntimeError, match="guard 'count_within_capacity' failed"):
        contract.resolve(10, failed_guards=("count_within_capacity",))
    with pytest.raises(ValueError, match="outside the contract"):
        contract.resolve(65)
    with pytest.raises(RuntimeError, match="forbids a fallback"):
        _contract(rank_control=RankControl.DYNAMIC, fallback=ExecutionFallback.ERROR).resolve(1)
    with pytest.raises(ValueError, match="two runtime guards are called"):
        _contract(guards=(RuntimeGuard("a", ExecutionFallback.EAGER), RuntimeGuard("a", ExecutionFallback.EAGER)))
    plan = compile_execution_plan(contract, (8, 256, 64))
    assert plan["variants"] == (8, 64) and plan["mode"] == "fixed_capacity"
    described = contract.describe()
    assert described["capacity"]["padding"] == "dead" and described["fixed_capacity_legal"]
    compiled = ab.CompiledExecutionPlan((type("P", (), {"name": "a"})(),), contract)
    assert compiled.phase("a").name == "a" and compiled.resolve(3).mode == "fixed_capacity"
    with pytest.raises(ValueError, match="at least one phase"):
        ab.CompiledExecutionPlan((), contract)


def test_kv_lifecycle_and_profiles():
    from aboleth_b200.kv import TransferState
    from aboleth_b200.kv.lifecycle import TransferLedger

    ledger = TransferLedger(2)
    a, b = ledger.admit("a", 4), ledger.admit("b", 4)
    assert (a.slot, a.epoch, b.slot, b.epoch) == (0, 1, 1, 2) and ledger.admit("c", 4) is None
    with pytest.raises(RuntimeError, match="already in flight"):
        ledger.admit("a", 4)
    a.move(TransferState.TRANSFERRING)
    a.move(TransferState.READY)
    with pytest.raises(RuntimeError, match="not allowed"):
        a.move(TransferState.FAILED)          # a ready transfer can only be consumed or aborted
    a.move(TransferState.CONSUMED)
    assert a.terminal and a.history == [TransferState.ADMITTED, TransferState.TRANSFERRING, TransferState.READY]
    c = ledger.admit("c", 4)
    assert c.slot == 0 and c.epoch == 3       # the freed slot, a fresh epoch
    b.move(TransferState.FAILED, error="status 1")
    assert b.error == "status 1" and [r.request_id for r in ledger.live()] == ["c"]
    assert ledger.admit("a", 4).slot == 1     # a finished request id may come back

    assert ab.select_kv_target_profile("NVIDIA B200").name == "b200-nvlink"
    assert ab.select_kv_target_profile("NVIDIA H200").name == "h200-nvlink"
    assert ab.select_kv_target_profile("something else") is ab.GENERIC_KV_TARGET_PROFILE
    tuned = ab.select_kv_target_profile("NVIDIA H200", overrides=ab.KVRuntimeOverrides(copy_workers=4))
    assert tuned.copy_workers == 4 and tuned.copy_engine_threshold == ab.H200_NVLINK_KV_TARGET_PROFILE.copy_engine_threshold
    assert ab.GENERIC_KV_TARGET_PROFILE.copy_engine_threshold is None


def test_record_programs_and_compiled_phase():
    from aboleth_b200.compiler import compile_program
    from aboleth_b200.records import await_records, send_records

    send = send_records(rank=1, peer_extent=4, capacity=64, width_bytes=512, meta_width_words=12, lanes=4,
                        row_quotient=16, row_remainder=0, reuse=8, ready_stride=8)
    with ab.compilation("proxy", rank=1, world_size=4, queue_capacity=64):
        queued = compile_program(send)
        waiting = compile_program(await_records(ready_stride=8, lanes_per_program=4))
    # payload + metadata + count + signal travel under one reservation; dead padding is trimmed
    assert queued.facts["reservations"] == 1 and queued.facts["strong_signals"] == 1
    assert queued.facts["trimmed_puts"] >= 2 and queued.facts["completion"] == "poll"
    assert waiting.facts["flag_reads"] and waiting.facts["commands"] == 0
    with ab.compilation("p2p", rank=1, world_size=4):
        direct = compile_program(send)
    assert direct.facts["reservations"] == 0 and direct.facts["fences"].count("st.release.sys") == 1

    pattern = ab.build_moe_pattern(ab.MoEPatternSpec(max_tokens=64, hidden=512, top_k=4, num_ranks=4)).compile()
    plan = pattern.compile_plan(ab.PhaseResources(peers={0: "p2p", 2: "p2p", 3: "p2p"}))
    with ab.compilation("p2p", rank=1, world_size=4):
        phase = ab.compile_phase(plan, "return.values", rank=1, capacity=64, width_bytes=1024)
    manifest = phase.manifest()
    assert manifest["strategy"] == "parallel_copy" and manifest["publication"] == "fused_kernel"
    assert manifest["sender_facts"]["strong_signals"] == 1 and manifest["completion_interval"] == 0
    assert phase.binding.sender_threads % 32 == 0 and phase.binding.sender_grid[0] >= 1
    with pytest.raises(KeyError):
        ab.compile_phase(plan, "no.such.phase", rank=1, capacity=64, width_bytes=1024)


def test_gate_skips_with_77_and_passes_exit_codes_through(tmp_path):
    """Requirement gate (reference scripts/run-gated.sh:1-120): 77 = skipped, other codes untouched."""
    import sys

    from aboleth_b200.utils import gated

    assert gated.missing("gpu", gpus=0) == "no GPU" and gated.missing("gpu", gpus=1) is None
    assert gated.missing("multi-gpu", gpus=1) and gated.missing("gpus=4", gpus=8) is None
    assert gated.missing("gpus=4", gpus=2) == "2 GPU(s), 4 needed"
    assert gated.missing("mlx5", verbs_root=tmp_path) == "no mlx5 device"
    (tmp_path / "mlx5_0").mkdir()
    assert gated.missing("mlx5", verbs_root=tmp_path) is None and gated.missing("hca", verbs_root=tmp_path) is None
    assert gated.run_gated(["gpus=2"], [sys.executable, "-c", "raise SystemExit(0)"], gpus=1) == gated.SKIP
    assert gated.run_gated(["gpu"], [sys.executable, "-c", "raise SystemExit(3)"], gpus=1) == 3
    assert gated.run_gated([], [sys.executable, "-c", "import time; time.sleep(30)"], timeout=0.5) == 124
    assert gated.main(["--needs", "gpus=64", "--", sys.executable, "-c", "pass"]) == gated.SKIP
    assert gated.main(["--needs", "gpu"]) == 2  # no command


def test_benchmark_report_tables_and_regression_check(tmp_path, capsys):
    import importlib.util
    import json
    from pathlib import Path

    spec = importlib.util.spec_from_file_location(
        "report", Path(__file__).resolve().parent.parent / "benchmarks" / "report.py")
    report = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(report)
    ref = {"bench": "tp", "n_gpus": 2, "rows": [{"op": "ag", "n": 8, "fused_us": 100.0, "speedup": 1.2},
                                                {"op": "rs", "n": 8, "fused_us": 200.0, "speedup": 1.1}]}
    new = {"bench": "tp", "n_gpus": 2, "rows": [{"op": "ag", "n": 8, "fused_us": 125.0, "speedup": 1.19},
                                                {"op": "rs", "n": 8, "fused_us": 190.0, "speedup": 1.3}]}
    (tmp_path / "ref").mkdir()
    (tmp_path / "new").mkdir()
    (tmp_path / "ref" / "tp.json").write_text(json.dumps(ref))
    (tmp_path / "new" / "tp.json").write_text("some log line\n" + json.dumps(new))
    assert report.direction("fused_us") == -1 and report.direction("busbw_gbs") == 1 and report.direction("op") == 0
    assert report.main([str(tmp_path / "ref")]) == 0
    assert "| ag | 8 | 100 | 1.2 |" in capsys.readouterr().out
    assert report.main(["--compare", str(tmp_path / "ref"), str(tmp_path / "new")]) == 1
    out = capsys.readouterr().out
    assert "fused_us: 100 -> 125" in out and "op=rs" not in out
    assert report.main(["--compare", "--tolerance", "0.5", str(tmp_path / "ref"), str(tmp_path / "new")]) == 0


def test_slurm_launcher_derives_the_rank_environment(tmp_path):
    import subprocess
    import sys

    from aboleth_b200.utils import launch

    assert launch.expand_nodelist("gpu[01-03,07],login1") == ["gpu01", "gpu02", "gpu03", "gpu07", "login1"]
    assert launch.expand_nodelist("n[9-11]-ib") == ["n9-ib", "n10-ib", "n11-ib"]
    assert launch.expand_nodelist("solo") == ["solo"]
    with pytest.raises(ValueError, match="unbalanced"):
        launch.expand_nodelist("gpu[01-03")
    with pytest.raises(ValueError, match="cannot read the range"):
        launch.expand_nodelist("gpu[a-b]")
    slurm = {"SLURM_JOB_NODELIST": "gpu[01-08]", "SLURM_STEP_NODELIST": "gpu[05-06]", "SLURM_PROCID": "9",
             "SLURM_NTASKS": "16", "SLURM_LOCALID": "1", "SLURM_JOB_ID": "4123456"}
    env = launch.slurm_environment(slurm)
    # The store lives on the first node of the step, not of the job.
    assert env["MASTER_ADDR"] == "gpu05" and env["MASTER_PORT"] == "23456"
    assert (env["RANK"], env["WORLD_SIZE"], env["LOCAL_RANK"]) == ("9", "16", "1")
    assert launch.slurm_environment({**slurm, "MASTER_PORT": "29999"})["MASTER_PORT"] == "29999"
    with pytest.raises(RuntimeError, match="run this through srun"):
        launch.slurm_environment({})
    # End to end: the command sees the derived variables.
    import os
    out = subprocess.run([sys.executable, "-m", "aboleth_b200.utils.launch", "--", sys.executable, "-c",
                          "import os; print(os.environ['RANK'], os.environ['MASTER_ADDR'])"],
                         env={**os.environ, **slurm}, capture_output=True, text=True, timeout=120)
    assert out.returncode == 0 and out.stdout.split() == ["9", "gpu05"], out.stderr
    assert launch.main([]) == 2


def test_documents_name_files_that_exist():
    """Every file a document names in backticks or links to is in the tree (the reference lints its
    documents' links the same way, experiments/bench/linkcheck.sh)."""
    import re
    from pathlib import Path

    root = Path(__file__).resolve().parent.parent
    pkg = root / "aboleth_b200"
    bases = [root, pkg, root / "tests", root / "benchmarks", root / "examples", root / "docs",
             pkg / "include", pkg / "include" / "aboleth", pkg / "include" / "aboleth" / "abi",
             *[p for p in pkg.rglob("*") if p.is_dir() and "_lib" not in p.parts and "__pycache__" not in p.parts]]
    generated = {"manifest.json", "kernel.cubin"}  # written at run time
    missing = []
    for document in [root / "README.md", *sorted((root / "docs").glob("*.md"))]:
        text = document.read_text()
        named = set(re.findall(r"\]\(([^)#\s]+)\)", text))
        for tick in re.findall(r"`([^`\s]+)`", text):
            if re.search(r"\.(py|cu|cuh|h|hpp|cpp|md|json|txt|cmake)$", tick) and not set("*{<$") & set(tick):
                named.add(tick)
        for name in sorted(named):
            if name.startswith("http") or name in generated:
                continue
            if not any((base / name).exists() for base in bases):
                missing.append((document.name, name))
    assert not missing, missing
