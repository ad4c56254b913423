"""Tier-2 specializer: pass behaviour, emitted-code facts and golden files (no GPU).

The golden check is the compile-only configuration: the all-to-all program for
world 2, rank 0, 4096 int8 bytes per peer, lowered through the whole pipeline,
with batch count, fence kind and flag writes asserted.
"""
import json
from pathlib import Path

import pytest

from aboleth_b200.compiler import (OPTIMIZATIONS, CompileError, ProgramBuilder, build_artifact,
                                   compilation, compile_program, enabled_optimizations, pipeline_key,
                                   programs)
from aboleth_b200.compiler.driver import _affine
from aboleth_b200.compiler.goldens import all_files

GOLDENS = Path(__file__).parent / "goldens"


def _compile(builder, backend="p2p", **kw):
    kw.setdefault("rank", 0)
    kw.setdefault("world_size", 2)
    with compilation(backend, **kw):
        return compile_program(builder)


def test_goldens_are_current():
    files = all_files()
    assert len(files) > 100
    stale = [n for n, text in files.items()
             if not (GOLDENS / n).exists() or (GOLDENS / n).read_text() != text]
    assert not stale, f"regenerate with python -m aboleth_b200.compiler.goldens --write tests/goldens: {stale[:5]}"


def test_alltoall_p2p_golden_facts():
    c = _compile(programs.alltoall(4096))
    f = c.facts
    assert f["batches"] == 1 and f["commands"] == 2
    assert f["fences"] == ["bar.sync", "st.release.sys", "ld.acquire.sys"]  # no membar.sys before the signal
    assert f["system_fences"] == 0 and f["barriers"] == 1
    assert f["flag_writes"] == ["release.sys:epoch"] and f["flag_reads"] == ["acquire.sys>=epoch"]
    assert f["completion"] == "vacuous" and f["strong_signals"] == 1 and f["weak_signals"] == 0
    assert f["exclusive_issuers"] == 0  # pid + (pid >= RANK) is not proven injective
    assert "submit %t4 %s6 batch=2" in c.ir and "mode=P2PRelease" in c.ir
    assert "t2::put_p2p<512>" in c.cuda  # smallest power of two covering 4096 bytes
    assert "fence_acq_rel_sys" not in c.cuda and c.cuda.count("st_release_sys") == 1


def test_alltoall_proxy_one_reservation_two_commands():
    f = _compile(programs.alltoall(4096), "proxy").facts
    assert (f["reservations"], f["commands"], f["ready_stores"], f["completion_waits"]) == (1, 2, 1, 1)
    assert f["flag_writes"] == ["strong:epoch"]


def test_put_without_signal_gets_barrier_and_system_fence():
    b = ProgramBuilder("lonely", args=[("src", "ptr"), ("ep", "table"), ("tab", "table")])
    e = b.endpoint("ep", 1)
    t = b.put(e, b.remote("tab", 1), b.local("src"), bytes=8192)
    b.wait(t)
    f = _compile(b).facts
    assert f["fences"] == ["bar.sync", "membar.sys"] and f["system_fences"] == 1


def test_standalone_signal_is_weak_and_switch_controls_it():
    b = ProgramBuilder("ack", args=[("ep", "table"), ("tab", "table")])
    e = b.endpoint("ep", 1)
    b.signal(e, b.remote("tab", 1), epoch=7)
    assert _compile(b).facts["weak_signals"] == 1
    assert _compile(b, passes="-plan-publication").facts["strong_signals"] == 1


def test_valid_extent_trimming_and_switch():
    b = ProgramBuilder("trim", args=[("src", "ptr"), ("ep", "table"), ("tab", "table"), ("n", "i64")])
    e = b.endpoint("ep", 1)
    src = b.local("src", valid=("n", 64, 128), at=256)
    t = b.put(e, b.remote("tab", 1), src, bytes=8192)
    b.wait(t)
    on = _compile(b)
    assert "ab_valid_bytes(8192,n,64,128,256)" in on.ir and on.facts["trimmed_puts"] == 1
    off = _compile(b, passes="-valid-extents")
    assert "ab_checked_bytes(8192,n,64,128,256)" in off.ir and off.facts["trimmed_puts"] == 0


def test_inline_forwarding_requires_exact_tiling():
    def program(widths, mention_again=False):
        b = ProgramBuilder("hdr", args=[("stage", "ptr"), ("ep", "table"), ("tab", "table"), ("v", "i64")])
        e = b.endpoint("ep", 1)
        offset = 0
        for w in widths:
            b.store("stage", offset=offset, width=w, value="v")
            offset += w // 8
        if mention_again:
            b.store("stage", offset=64, width=32, value="v")
        t = b.put(e, b.remote("tab", 1), b.local("stage"), bytes=12)
        b.signal(e, b.remote("tab", 1, offset=64), epoch=1, after=t)
        return b

    good = _compile(program([32, 32, 32]))
    assert good.passes["forward-inline-payloads"] == 1 and "post_inline" in good.ir and "store stage" not in good.ir
    assert good.facts["inline_puts"] == 1 and good.facts["cooperative_puts"] == 0
    assert _compile(program([32, 32]))  .passes["forward-inline-payloads"] == 0   # hole at the end
    assert _compile(program([32, 32, 32], True)).passes["forward-inline-payloads"] == 0  # extra store to the base
    assert _compile(program([32, 32, 32]), passes="-forward-inline-payloads").passes["forward-inline-payloads"] == 0
    assert _compile(program([32, 32, 32]), "proxy").passes["forward-inline-payloads"] == 0  # only p2p, rdma, ionic


def test_planned_wait_interval_respects_reuse_policy_and_queue():
    def k(c):
        import re
        return int(re.search(r"interval=(\d+)", c.ir).group(1))

    prog = programs.stream("pipelined", 1, 256, reuse=32)
    assert k(_compile(prog, "rdma")) == 16                       # transport preference 16
    assert k(_compile(prog, "proxy")) == 8                       # proxy prefers 8
    assert k(_compile(prog, "rdma", completion_interval=4)) == 4
    assert k(_compile(prog, "rdma", queue_capacity=9)) == 4      # (9-1)/2 commands
    assert k(_compile(prog, "rdma", passes="-completion-planning")) == 1
    assert k(_compile(programs.stream("pipelined", 1, 256, reuse=6), "rdma")) == 4  # bit_floor(6)


def test_coalescing_and_ordering_only_on_queue_transports():
    prog = programs.stream("chains", 4, 256)
    rdma = _compile(prog, "rdma")
    assert rdma.facts["batches"] == 1 and rdma.facts["reservations"] == 1 and rdma.facts["commands"] == 8
    assert rdma.passes["coalesce-submissions"] == 3 and rdma.passes["order-publications"] == 1
    assert rdma.ir.count("ordering_point") == 1 and rdma.ir.count("chained=") == 3
    off = _compile(prog, "rdma", passes="-coalesce-submissions")
    assert off.facts["batches"] == 4 and off.facts["reservations"] == 4
    p2p = _compile(prog, "p2p")
    assert p2p.facts["batches"] == 4 and p2p.passes["coalesce-submissions"] == 0  # no-op by design


def test_elide_epochs_skips_kernels_that_wait_on_peers():
    prog = programs.stream("pipelined", 2, 256, reuse=4)
    elided = _compile(prog, "rdma")
    assert elided.facts["elided_signals"] == 2
    # A checked publication compares against the epoch this loop published LAST: the value is set up in
    # front of the loop (epoch of the first iteration, minus one) and advances after each published
    # submission (reference: compiler/lib/Transforms/ElideEpochs.cpp:110-174).
    lines = elided.ir.splitlines()
    setup = next(i for i, l in enumerate(lines) if "long long ab_published_0 = (((0) + 1)) - 1" in l)
    loop = next(i for i, l in enumerate(lines) if l.startswith("for round"))
    signal = next(i for i, l in enumerate(lines) if "post_signal" in l and "expected=ab_published_0" in l)
    submit = next(i for i, l in enumerate(lines) if "submit" in l and i > signal)
    advance = next(i for i, l in enumerate(lines) if "ab_published_0 = ((round + 1))" in l)
    assert setup < loop < signal < submit < advance
    assert "expected=" not in _compile(prog, "rdma", passes="-elide-epochs").ir
    b = programs.stream("pipelined", 2, 256, reuse=4)
    b.wait_signal("payload", 1)
    assert _compile(b, "rdma").facts["elided_signals"] == 0


def test_defer_announcement_is_opt_in():
    prog = programs.stream("pipelined", 1, 256, reuse=4)
    assert "deferredAnnouncement" not in _compile(prog, "rdma").ir
    assert "deferredAnnouncement" in _compile(prog, "rdma", passes="+defer-announcement").ir


def test_producer_barrier_placed_once_per_dirty_region():
    c = _compile(programs.fp8_dispatch())
    assert c.facts["producer_barriers"] == 1 and c.ir.count("producerBarrier") == 1
    assert c.facts["batches"] == 1 and c.facts["commands"] == 6 and c.facts["inline_puts"] == 1
    assert c.facts["exclusive_issuers"] == 1          # endpoint index is the program id
    q = _compile(programs.fp8_dispatch(), "rdma", queue_capacity=64)
    assert q.facts["reservations"] == 1 and "planned=iteration" in q.ir


def test_issuer_analysis_patterns():
    def known(expr):
        return json.loads(_affine(expr))

    assert known("pid")["known"] and known("pid")["scale"] == 1
    assert known("pid + 3")["scale"] == 1 and known("2*pid + base")["scale"] == 2
    assert known("(pid + 1) % 8") == {"known": True, "scale": 1, "modular": True, "modulus": 8}
    assert not known("pid + (pid >= RANK)")["known"]
    assert not known("pid * stride")["known"]       # an unknown uniform factor may be zero
    assert not known("pid / 2")["known"]
    assert known("lane*4 + 3")["scale"] == 0          # uniform only: not injective


def test_verifier_diagnostics():
    bad_width = "program p backend=p2p\n%e = endpoint t 0\n%r = remote t 0\n%x = put_inline %e %r values=v:12\n"
    with pytest.raises(CompileError, match="width 12 is not one of 8, 16, 24, 32, 64"):
        compile_program(bad_width)
    too_big = "program p backend=p2p\n%e = endpoint t 0\n%r = remote t 0\n%x = put_inline %e %r values=" + \
        ",".join(["v:64"] * 122) + "\n"
    with pytest.raises(CompileError, match="exceeds the 972-byte limit"):
        compile_program(too_big)
    with pytest.raises(CompileError, match="after=%nope is not defined"):
        compile_program("program p backend=p2p\n%e = endpoint t 0\n%r = remote t 0\n%s = signal %e %r epoch=1 after=%nope\n")
    with pytest.raises(CompileError, match="belongs to another endpoint"):
        compile_program("program p backend=p2p\n%e = endpoint t 0\n%f = endpoint t 1\n%r = remote t 0\n%l = local a\n"
                        "%t = put %e %r %l bytes=8\n%s = signal %f %r epoch=1 after=%t\n")
    with pytest.raises(CompileError, match="has no wait_group"):
        compile_program("program p backend=p2p\n%e = endpoint t 0\n%g = begin_group %e\n")
    with pytest.raises(CompileError, match="written for transport 'gin'"):
        compile_program("program p backend=gin\n")
    with pytest.raises(ValueError, match="unknown transport 'gin'"):
        compilation("gin").__enter__()
    with pytest.raises(CompileError, match="written for transport 'rdma'"):
        compile_program("program p backend=rdma\n")
    # Operations that the passes index by position are refused when they come up short.
    with pytest.raises(CompileError, match="remote: expects <table> <peer>"):
        compile_program("program p backend=p2p\n%e = endpoint t 0\n%r = remote t\n")
    with pytest.raises(CompileError, match="endpoint: expects <table> <index>"):
        compile_program("program p backend=p2p\n%e = endpoint t\n")
    with pytest.raises(CompileError, match="needs a %name = in front"):
        compile_program("program p backend=p2p\nendpoint t 0\n")
    with pytest.raises(CompileError, match="for: expects <var> <begin> <end>"):
        compile_program("program p backend=p2p\nfor i 4 {\n}\n")


def test_passes_grammar_and_key_coverage(monkeypatch):
    assert enabled_optimizations("none") == frozenset()
    assert enabled_optimizations("all") == frozenset(OPTIMIZATIONS)
    assert "elide-epochs" not in enabled_optimizations("-elide-epochs")
    assert "defer-announcement" in enabled_optimizations("default,+defer-announcement")
    with pytest.raises(ValueError, match="not \\+name or -name"):
        enabled_optimizations("elide-epochs")
    monkeypatch.setenv("ABOLETH_PASSES", "-plan-publication")
    assert "plan-publication" not in enabled_optimizations()
    monkeypatch.delenv("ABOLETH_PASSES")
    # Every option and every switch moves the artefact key.
    text = programs.alltoall(4096).text()
    base = compilation("p2p").__enter__()
    keys = {pipeline_key(text, base)}
    from dataclasses import replace
    for change in (dict(backend="proxy"), dict(queue_capacity=64), dict(completion_interval=2),
                   dict(strict_registrations=True), dict(gpu_resident_queues=True), dict(inline_bytes=16),
                   dict(p2p_copy="scalar"), dict(endpoint_profile="seed"), dict(plan_hash="abc"),
                   dict(coop_min=512), dict(coop_elements=1024), dict(arch="sm_100")):
        keys.add(pipeline_key(text, replace(base, **change)))
    for name in OPTIMIZATIONS:
        flipped = base.passes ^ {name}
        keys.add(pipeline_key(text, replace(base, passes=frozenset(flipped))))
    assert len(keys) == 1 + 12 + len(OPTIMIZATIONS)


def test_emitted_kernels_compile_for_sm_100a(tmp_path, monkeypatch):
    monkeypatch.setenv("ABOLETH_CACHE_DIR", str(tmp_path))
    for backend in ("p2p", "rdma"):
        with compilation(backend, rank=0, world_size=2):
            art = build_artifact(compile_program(programs.stream("fused", 8, 1024)))
        assert art.cubin.exists() and art.cubin_bytes > 0 and art.spill_bytes == 0
        assert art.manifest()["n_regs"] > 0
    again = build_artifact(_compile(programs.stream("fused", 8, 1024), "rdma"))
    assert again.cubin == art.cubin  # cache hit under the same key


def test_scheduled_ir_dump_and_utils(tmp_path, monkeypatch):
    """ABOLETH_DUMP_SCHEDULED_IR writes program, scheduled IR, emitted source and facts per compilation."""
    import json

    from aboleth_b200.compiler import compilation, compile_program
    from aboleth_b200.compiler.programs import alltoall
    from aboleth_b200.utils import host_range, provenance, ranges_enabled

    monkeypatch.setenv("ABOLETH_DUMP_SCHEDULED_IR", str(tmp_path))
    with compilation("proxy", rank=1, world_size=4, queue_capacity=64):
        compiled = compile_program(alltoall())
    (folder,) = list(tmp_path.iterdir())
    assert folder.name.startswith("alltoall-proxy-")
    assert {p.name for p in folder.iterdir()} == {"program.txt", "scheduled.ir", "kernel.cu", "facts.json"}
    assert json.loads((folder / "facts.json").read_text())["facts"] == compiled.facts
    assert (folder / "kernel.cu").read_text() == compiled.cuda
    record = provenance()
    assert {"time", "host", "git", "torch", "env"} <= set(record)
    assert "ABOLETH_DUMP_SCHEDULED_IR" in record["env"]
    monkeypatch.delenv("ABOLETH_NVTX", raising=False)
    assert not ranges_enabled()
    with host_range("noop"):
        pass


def test_ladder_programs_batch_as_the_benchmarks_expect():
    from aboleth_b200.compiler import compilation, compile_program
    from aboleth_b200.compiler.programs import pingpong, windowed

    with compilation("p2p", rank=0, world_size=2):
        lead = compile_program(pingpong(4096, chain=4)).facts
        echo = compile_program(pingpong(4096, leader=False)).facts
        window = compile_program(windowed(65536, window=8)).facts
    # a chain is one batch closed by one release; a window without a signal ends in one system fence
    assert (lead["batches"], lead["commands"], lead["strong_signals"], lead["system_fences"]) == (1, 5, 1, 0)
    assert echo["flag_reads"] == lead["flag_reads"] == ["acquire.sys>=(epoch0 + round + 1)"]
    assert (window["batches"], window["commands"], window["system_fences"]) == (1, 8, 1)
    with compilation("proxy", rank=0, world_size=2, queue_capacity=64):
        queued = compile_program(windowed(65536, window=8)).facts
    assert queued["reservations"] == 1 and queued["completion"] == "poll"


def _independent_puts(chain=8, *, poll_first=False):
    from aboleth_b200.compiler import ProgramBuilder

    b = ProgramBuilder("independent", threads=128, args=[
        ("src", "ptr"), ("endpoints", "table"), ("dst_table", "table"), ("flag_table", "table"),
        ("my_flag", "ptr"), ("epoch", "u64")])
    e = b.endpoint("endpoints", 0)
    tokens = [b.put(e, b.remote("dst_table", 0, offset=c * 1024), b.local(f"src + {c * 1024}"), bytes=1024)
              for c in range(chain)]
    if poll_first:
        b.wait(tokens[0])
    s = b.signal(e, b.remote("flag_table", 0), epoch="epoch", after=tokens[-1])
    b.wait_signal("my_flag", "epoch")
    b.wait(s)
    return b


def test_unchained_puts_coalesce_on_the_ring_and_share_one_release_on_peer_memory():
    """Puts that are not chained by `after` form one submission each.  On the ring adjacent
    submissions to one endpoint merge (segments recorded, verifier accepts a chain that ends at a
    segment boundary).  On peer memory a submission that nothing polls leaves its placement to the
    next submission's barrier + release, so eight puts and a signal cost one barrier and no
    system fence; a poll of an early put or the switch being off keeps the fence."""
    from aboleth_b200.compiler import compilation, compile_program

    with compilation("proxy", rank=0, world_size=1):
        ring = compile_program(_independent_puts())
    assert ring.passes["form-batches"] == 8 and ring.passes["coalesce-submissions"] == 6
    assert ring.facts["batches"] == 2 and ring.facts["commands"] == 9
    with compilation("p2p", rank=0, world_size=1):
        peer = compile_program(_independent_puts())
    assert (peer.facts["barriers"], peer.facts["system_fences"], peer.facts["deferred_placements"]) == (1, 0, 7)
    assert peer.cuda.count("fence_acq_rel_sys();  // no signal follows") == 0
    with compilation("p2p", rank=0, world_size=1, passes="none"):
        naive = compile_program(_independent_puts())
    assert (naive.facts["barriers"], naive.facts["system_fences"], naive.facts["deferred_placements"]) == (8, 7, 0)
    with compilation("p2p", rank=0, world_size=1):
        polled = compile_program(_independent_puts(poll_first=True))
    # the polled first put keeps its fence; the other seven are placed by the signal's barrier + release
    assert (polled.facts["barriers"], polled.facts["system_fences"], polled.facts["deferred_placements"]) == (2, 1, 7)


def test_pipeline_is_a_fixed_point_on_its_own_output():
    """Scheduled IR fed back through the same pipeline comes out unchanged, and lowers to the same
    CUDA C++ (the reference runs each pass twice under its IDEMPOTENT test option,
    test/compiler/CMakeLists.txt)."""
    from pathlib import Path

    goldens = Path(__file__).resolve().parent / "goldens"
    checked = 0
    for scheduled in sorted(goldens.glob("*.ir")):
        _, backend, variant, _ = scheduled.name.split(".")
        text = scheduled.read_text()
        with compilation(backend, rank=0, world_size=2, passes=variant):
            again = compile_program(text)
        assert again.ir == text, scheduled.name
        assert again.cuda == scheduled.with_suffix(".cu").read_text(), scheduled.name
        assert all(count == 0 for name, count in again.passes.items()
                   if name in ("form-batches", "coalesce-submissions")), (scheduled.name, again.passes)
        checked += 1
    assert checked >= 80


_PLAN = """program moe.plan kind=transport_program
phase dispatch program_id=3 interval=8 capacities=64,32
phase dispatch.tail program_id=3 interval=4 capacities=128
fragment send program_id=3 params=table:i64,peer:i64,dst:i64,src:i64,n:i64,it:i64 {
  %e = endpoint table peer
  %r = remote_at dst
  %l = local src
  %t = put %e %r %l bytes=n
  planned_wait %t iteration=it
}
fragment publish program_id=4 params=ep:i64,flag:i64,epoch:i64 {
  %e = endpoint ep 0
  %r = remote_at flag
  %s = signal %e %r epoch=epoch
}
"""

_KERNEL = """program k backend=rdma
arg endpoints table
arg slots ptr
arg staging ptr
arg flags ptr
arg count u64
%mine = endpoint endpoints 1
for i 0 4 {
  invoke_phase 3 endpoints (i%2) (slots+i*4096) staging count*16 i
}
invoke_phase 4 %mine flags 7
"""


def test_transport_phases_are_spliced_from_an_external_program():
    from aboleth_b200.compiler import materialize_phases

    ir = materialize_phases(_KERNEL, _PLAN)
    assert "invoke_phase" not in ir
    # The loop body is the fragment with its parameters replaced and its values renamed.
    assert "%e.p0 = endpoint endpoints (i%2)" in ir and "%r.p0 = remote_at (slots+i*4096)" in ir
    assert "bytes=(count*16)" in ir  # an expression stays one operand
    # The resolved plan: the smallest interval and the smallest peer capacity of the bound phases.
    assert "planned_wait %t.p0 interval=4 iteration=i queue_capacity=32" in ir
    # An endpoint value passed for an i64 placeholder replaces the binding itself.
    assert "%s.p1 = signal %mine %r.p1 epoch=7" in ir and "endpoint %mine" not in ir
    # The spliced program goes through the whole pipeline.
    with compilation("rdma", rank=0, world_size=2):
        compiled = compile_program(_KERNEL, plan=_PLAN)
    assert compiled.cuda and "invoke_phase" not in compiled.ir
    with compilation("rdma", rank=0, world_size=2), pytest.raises(CompileError, match="materialise the phases first"):
        compile_program(_KERNEL)

    def broken(kernel=_KERNEL, plan=_PLAN):
        return lambda: materialize_phases(kernel, plan)

    for make, message in (
            (broken(kernel=_KERNEL.replace("invoke_phase 4", "invoke_phase 9")), "references missing transport fragment 9"),
            (broken(kernel=_KERNEL.replace(" flags 7", " flags")), "argument count does not match fragment 'publish'"),
            (broken(kernel=_KERNEL.replace("invoke_phase 4 %mine", "invoke_phase x %mine")), "programId must be an integer"),
            (broken(plan=_PLAN + "fragment again program_id=4 params=a:i64 {\n}\n"), "duplicate programId 4"),
            (broken(plan=_PLAN.replace("interval=8", "interval=0")), "requires a resolved completion interval"),
            # A pointer may stand for an i64 only where the fragment binds it, not where it computes with it.
            (broken(kernel=_KERNEL.replace("staging count*16 i", "staging slots i")), "argument #4 has type ptr"),
            (broken(plan=_PLAN.replace("ep:i64", "ep:ptr")), "argument #0 has type endpoint, but fragment 'publish' expects ptr")):
        with pytest.raises(CompileError, match=message):
            make()


def test_user_predicated_completion_is_self_reclaimed_and_must_be_retired():
    """wait(token, predicate=p) with a predicate the user wrote: the submission is marked selfReclaim
    on a queue transport, and the kernel must end with an unconditional wait or a drain."""
    def kernel(tail: str) -> str:
        return ("program k backend=rdma\narg t table\narg buf ptr\narg it u64\n%e = endpoint t 1\n"
                "for i 0 8 {\n  %r = remote t 1\n  %l = local buf\n  %p = put %e %r %l bytes=64\n"
                "  wait %p pred=((i&3)==3)\n}\n" + tail)

    with compilation("rdma", rank=0, world_size=2):
        drained = compile_program(kernel("drain %e\n"))
        assert "selfReclaim" in drained.ir and drained.passes["self-reclaim"] == 1
        with pytest.raises(CompileError, match="deferred by a user-written predicate is never retired on %e"):
            compile_program(kernel(""))
    with compilation("rdma", rank=0, world_size=2, passes="-self-reclaim"):
        unmarked = compile_program(kernel("drain %e\n"))  # the switch only controls the marking
        assert "selfReclaim" not in unmarked.ir
        with pytest.raises(CompileError, match="never retired"):
            compile_program(kernel(""))
    with compilation("p2p", rank=0, world_size=2):  # completion is vacuous on peer memory
        assert "selfReclaim" not in compile_program(kernel("").replace("backend=rdma", "backend=p2p")).ir


def test_builder_states_phase_invocations():
    from aboleth_b200.compiler import ProgramBuilder, materialize_phases

    b = ProgramBuilder("k", args=[("endpoints", "table"), ("flags", "ptr"), ("it", "u64")])
    mine = b.endpoint("endpoints", 1)
    b.invoke_phase(4, mine, "flags + 8", "it + 1")
    text = b.text(backend="rdma", rank=0, world_size=2)
    assert f"invoke_phase 4 {mine} (flags + 8) (it + 1)" in text
    ir = materialize_phases(text, _PLAN)
    assert f"signal {mine} %r.p0 epoch=(it + 1)" in ir
    other = ProgramBuilder("other")
    with pytest.raises(TypeError, match="cannot cross programs"):
        other.invoke_phase(4, mine)


def test_fragment_names_do_not_capture_the_kernels_names():
    """A loop variable or a let of the fragment is renamed per invocation, so an argument expression
    that mentions the kernel's own variable of the same name keeps meaning the kernel's."""
    from aboleth_b200.compiler import materialize_phases

    plan = ("program p kind=transport_program\n"
            "fragment rows program_id=2 params=table:i64,dst:i64,src:i64 {\n"
            "  let stride 4096\n  %e = endpoint table 1\n  for i 0 4 {\n    %r = remote_at (dst+i*stride)\n"
            "    %l = local (src+i*stride)\n    %t = put %e %r %l bytes=4096\n    wait %t\n  }\n}\n")
    kernel = ("program k backend=rdma\narg endpoints table\narg out ptr\narg in ptr\n"
              "for i 0 2 {\n  invoke_phase 2 endpoints (out+i*16384) (in+i*16384)\n}\n")
    ir = materialize_phases(kernel, plan)
    assert "for i_p0 0 4 {" in ir and "let stride_p0 4096" in ir
    assert "remote_at ((out+i*16384)+i_p0*stride_p0)" in ir  # the kernel's i and the fragment's stay apart
    with compilation("rdma", rank=0, world_size=2):
        assert compile_program(kernel, plan=plan).cuda
    with pytest.raises(CompileError, match="'dst' is a parameter of the fragment"):
        materialize_phases(kernel, plan.replace("let stride 4096", "let dst 4096"))
