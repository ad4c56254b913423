"""Patterns, physicalisation, transport-program planning and the artifact forms (CPU only)."""
import pytest

import aboleth_b200 as ab
from aboleth_b200.planning import RegionAccess as A


def test_moe_pattern_graph_and_plan():
    spec = ab.MoEPatternSpec(max_tokens=64, hidden=512, top_k=4, num_ranks=4, scale_width=4, value_type="fp8")
    compiled = ab.build_moe_pattern(spec).compile()
    kinds = [(op["kind"], op["name"]) for op in compiled.dataflow.operations]
    assert kinds == [("transfer", "dispatch.values"), ("transfer", "dispatch.scales"),
                     ("transfer", "dispatch.count"), ("opaque_stage", "experts"),
                     ("transfer", "return.values"), ("opaque_stage", "combine"), ("use", "output.consumer")]
    # the staging copy after the experts is forwarded into the donated return source
    assert [r["name"] for r in compiled.dataflow.removed] == ["return.stage"]
    assert "expert.output" in compiled.dataflow.unallocated_regions
    plan = compiled.compile_plan(ab.PhaseResources(peers={1: "p2p", 2: "p2p", 3: "p2p"}))
    assert plan.phase_schedule("dispatch.count").strategy == "inline_transport"
    assert plan.phase_schedule("return.values").strategy == "parallel_copy"
    assert plan.phase_schedule("return.values").publication_strategy == "fused_kernel"
    with pytest.raises(ValueError, match="exactly one layer in flight"):
        ab.MoEPatternSpec(max_tokens=1, hidden=8, top_k=1, experts_asynchronous=False, expert_max_inflight=2)


def test_kv_migration_compiles_to_direct_pages():
    spec = ab.KVCacheMigrationSpec(max_pages=256, page_bytes=16384, num_ranks=2, max_consumers=4)
    assert spec.required_slots == 2 and spec.slot_count == 2
    plan = ab.compile_kv_cache_migration(spec)
    ph = plan.physicalization
    assert ph.name == "parallel-batched-direct-pages" and ph.direct_destination
    assert ph.pages_per_transfer == 16 and ph.readiness == "consumer" and ph.slot_count == 2
    assert plan.fallback_phase is not None
    assert plan.select_phase(contiguous_page_runs=False, consumer_partitioned=True)[1] == 1
    assert plan.select_phase(contiguous_page_runs=True, consumer_partitioned=True)[1] == 16
    assert plan.select_transfer_engine(transfer_bytes=1 << 30, run_count=4) == "generated_p2p"
    with_engine = ab.compile_kv_cache_migration(spec, target_profile=ab.H200_NVLINK_KV_TARGET_PROFILE)
    assert with_engine.select_transfer_engine(transfer_bytes=64 << 20, run_count=4) == "copy_engine"
    assert with_engine.select_transfer_engine(transfer_bytes=64 << 20, run_count=1000) == "generated_p2p"
    described = plan.describe()
    assert described["layout_contract"]["contiguous_page_runs"] and described["execution"]["mode"] == "eager"
    # pages that are not contiguous runs move one at a time
    single = ab.compile_kv_cache_migration(spec, layout_contract=ab.KVCacheLayoutContract(contiguous_page_runs=False))
    assert single.physicalization.pages_per_transfer == 1 and single.fallback_phase is None
    with pytest.raises(ValueError, match="slots cannot cover a consumer"):
        ab.KVCacheMigrationSpec(max_pages=8, page_bytes=64, slots=1)


def _program():
    ring = dict(length=4096, stride=4096, period=4 * 4096, count=8)
    return (
        ab.TransportKernel("pack", writes=(A(1, **ring),)),
        ab.TransportPhase("dispatch", commands=3, iterations=8, payload_bytes=65536,
                          peer_transports=("rdma", "p2p"), peer_capacities=(64, 0),
                          reads=(A(1, **ring),), writes=(A(2, length=4096, count=8),)),
        ab.TransportKernel("experts", reads=(A(2, length=4096),), writes=(A(3, length=4096),),
                           asynchronous=True, event_ordered=True, max_inflight=2, opaque=True),
        ab.TransportPhase("return", commands=1, iterations=8, payload_bytes=65536, peer_transports=("rdma",),
                          peer_capacities=(64,), reads=(A(3, length=4096, count=8),),
                          writes=(A(4, length=4096, count=8),)),
        ab.TransportKernel("gather", reads=(A(4, length=4096),), writes=(A(5, length=4096),)),
    )


def test_transport_program_deadlines_and_lifetimes():
    plans = ab.plan_transport_program(_program(), cyclic=True)
    d = plans["dispatch"]
    # a four-slot ring: the source is rewritten four iterations later, by next iteration's pack
    assert (d.reuse_distance, d.completion_interval) == (4, 4) and d.requires_final_drain
    assert (d.completion_before, d.completion_iteration_delta) == ("pack", 1)
    assert (d.publication_before, d.publication_iteration_delta) == ("experts", 0)
    r = plans["return"]
    assert (r.reuse_distance, r.completion_interval, r.completion_before) == (1, 1, "experts")
    lifetimes = ab.plan_output_lifetimes(_program(), cyclic=True)
    assert lifetimes["experts"].pool_depth == 2 and lifetimes["experts"].last_consumer == "return"
    assert "gather" not in lifetimes  # nobody reads its output inside the program
    # without the wrap nothing overwrites the ring: completion may wait for the end
    straight = ab.plan_transport_program(_program(), cyclic=False)
    assert straight["dispatch"].completion_before == "program_end"
    # a queue that cannot hold one iteration, and an interval longer than the lifetime, are refused
    bad = list(_program())
    bad[1] = ab.TransportPhase("dispatch", commands=3, iterations=8, peer_transports=("rdma",),
                               peer_capacities=(2,), reads=bad[1].reads)
    with pytest.raises(Exception, match="cannot hold one iteration"):
        ab.plan_transport_facts(bad)
    bad[1] = ab.TransportPhase("dispatch", commands=3, iterations=8, peer_transports=("rdma",),
                               peer_capacities=(64,), reads=_program()[1].reads, explicit_interval=8)
    with pytest.raises(Exception, match="exceeds region lifetime"):
        ab.plan_transport_facts(bad)
    # an access that cannot be bounded overlaps everything
    unknown = (ab.TransportPhase("a", iterations=2, peer_transports=("p2p",), peer_capacities=(0,),
                                 reads=(A(1, length=8, count=2),)),
               ab.TransportKernel("k", writes=(A(9, unknown=True),)))
    assert ab.plan_transport_program(unknown)["a"].completion_before == "k"


def test_physicalize_and_realize_artifacts():
    compiled = ab.build_moe_pattern(ab.MoEPatternSpec(max_tokens=64, hidden=512, top_k=4, num_ranks=4)).compile()
    attachments = [
        ab.PhaseBinding("experts", None, "return.values", "expert_kernel", "epilogue", 4, "fused_kernel",
                        artifact=ab.Artifact.BINDABLE_EPILOGUE),
        ab.PhaseBinding(None, "experts", "dispatch", "pack_kernel", "after_pack", 4, "fused_kernel",
                        operations=("dispatch.values", "dispatch.count"), artifact=ab.Artifact.STANDALONE_KERNEL),
    ]
    phys = ab.physicalize_pattern(compiled, attachments)
    manifest = phys.manifest("dispatch")
    assert manifest.program_id == 1 and len(manifest.transfers) == 2 and manifest.signal is not None
    assert manifest.slot_names[0] == "dispatch_endpoint" and "dispatch_count_live" in manifest.slot_names
    with ab.compilation("p2p"):
        epilogue = ab.realize_bindable_epilogue(phys.binding("return.values"), reuse=4)
    assert "__device__ __forceinline__ void return_values_fragment(" in epilogue.source
    assert "__global__" not in epilogue.source and epilogue.facts["strong_signals"] == 1
    call = epilogue.call(**{n: n for n, _ in epilogue.parameters})
    assert call.startswith("return_values_fragment(return_values_endpoint, ") and call.endswith("nullptr);")
    text = ab.invoke_transport_program(manifest, "dispatch", **{n: "x" for n in manifest.slot_names})
    assert text.count("static_cast") == len(manifest.slot_names)
    with pytest.raises(ValueError, match="missing slots"):
        ab.invoke_transport_program(manifest, "dispatch")
    with ab.compilation("proxy"):
        queued = ab.compile_fragment_artifact(phys.binding("dispatch"))
    assert queued.facts["reservations"] >= 1 and queued.facts["backend"] == "proxy"
    # errors: removed operation, double attachment, wrong declared form
    with pytest.raises(ValueError, match="removed by the simplifier"):
        ab.physicalize_pattern(compiled, [ab.PhaseBinding("experts", None, "return.stage", "k", "p", 1, "fused_kernel")])
    with pytest.raises(ValueError, match="attached twice"):
        ab.physicalize_pattern(compiled, attachments + [
            ab.PhaseBinding(None, "experts", "again", "k", "p", 1, "fused_kernel", operations=("dispatch.count",))])
    with pytest.raises(ValueError, match="not standalone_kernel"):
        ab.realize_standalone_kernel(phys.binding("return.values"))
    with pytest.raises(ValueError, match="two roles"):
        from aboleth_b200.transport_binding import (BoundScalar, PublicationBinding, RegionBinding, RegionSide,
                                                    TransportProgramBinding)
        side = RegionSide(BoundScalar("p", "i64"), BoundScalar("k", "i32"))
        TransportProgramBinding("x", ("x",), "k", "p", BoundScalar("p", "i64"),
                                (RegionBinding(side, RegionSide(BoundScalar("q", "i64"), BoundScalar("k2", "i32")),
                                               BoundScalar("n", "i32"), BoundScalar("live", "i1"), 8, ("x",)),),
                                PublicationBinding(RegionSide(BoundScalar("f", "i64"), BoundScalar("fk", "i32")),
                                                   RegionSide(BoundScalar("g", "i64"), BoundScalar("gk", "i32")),
                                                   BoundScalar("i", "i32"), BoundScalar("m", "i32"))).slots()


def test_runtime_bindings_cover_surviving_regions():
    compiled = ab.build_kv_cache_migration_pattern(ab.KVCacheMigrationSpec(max_pages=8, page_bytes=64)).compile()
    live = sorted({r.name for r in compiled.regions} - set(compiled.dataflow.unallocated_regions))
    bindings = ab.RuntimeBindings((ab.RuntimeBufferBinding("pool", tuple(live)),))
    effects = bindings.effects(compiled, lambda buffer: ab.RegionEffect(buffer, "read", "bind", (0, 8)))
    assert sorted(effects) == live and effects[live[0]].region == "pool"
    with pytest.raises(KeyError, match="no runtime buffer binding"):
        ab.RuntimeBindings((ab.RuntimeBufferBinding("pool", tuple(live[:1])),)).effects(compiled, lambda b: None)
    with pytest.raises(ValueError, match="only one runtime buffer"):
        ab.RuntimeBindings((ab.RuntimeBufferBinding("a", ("x",)), ab.RuntimeBufferBinding("b", ("x",))))


def test_language_functions_build_the_same_program():
    from aboleth_b200 import language as L
    from aboleth_b200.compiler import ProgramBuilder, compile_program

    with L.building("ring", args=[("endpoints", "ptr"), ("buf", "u64"), ("it", "i32")]) as program:
        ep = L.endpoint("endpoints", 0)
        data = ab.put(ep, L.remote_at("buf"), L.local("buf"), bytes=4096)
        ready = ab.signal(ep, L.remote_at("buf + 4096"), epoch="it + 1", after=data)
        ab.planned_wait(ready, "it", 8)
    direct = ProgramBuilder("ring", args=[("endpoints", "ptr"), ("buf", "u64"), ("it", "i32")])
    ep = direct.endpoint("endpoints", 0)
    data = direct.put(ep, direct.remote_at("buf"), direct.local("buf"), bytes=4096)
    ready = direct.signal(ep, direct.remote_at("buf + 4096"), epoch="it + 1", after=data)
    direct.wait(ready, iteration="it", reuse=8)
    assert program.text() == direct.text()
    assert ab.token_type.of(ready) and isinstance(ready, ab.token)
    with ab.compilation("proxy"):
        assert compile_program(program).facts["completion"] == "poll"
    with pytest.raises(RuntimeError, match="open program"):
        ab.drain(ep)
    ab.install_compiler()


def test_endpoint_mesh_on_cpu_runtimes():
    runtimes = {i: ab.Runtime("cpu") for i in range(3)}
    try:
        with ab.EndpointMesh(runtimes, ab.Transport.PROXY) as mesh:
            assert len(mesh.pairs) == 3 and mesh.tables[1].peers == (0, 2)
            assert mesh.endpoint(2, 0).peer == 0 and mesh.endpoint(0, 1).handle & 7 == 2
            assert mesh.tables[0].device_handles.shape == (3,)
        with pytest.raises(RuntimeError, match="closed"):
            mesh.endpoint(0, 1)
        with pytest.raises(ValueError, match="at least two"):
            ab.EndpointMesh({0: runtimes[0]})
    finally:
        for r in runtimes.values():
            r.close()


def test_tier1_operations_as_programs():
    """What each Tier-1 call costs per transport: one reservation / doorbell per call on the ring,
    one release store and no fence per signalled chain on peer memory."""
    from aboleth_b200.tier1 import PROGRAMS, tier1_facts, tier1_program

    assert {"put", "put_inline24", "signal", "put_signal", "put_many_8", "put_many_32_signal",
            "put_many_8_flush", "quiet", "wait_signal"} <= set(PROGRAMS)
    p2p, ring = tier1_facts("p2p"), tier1_facts("proxy")
    chain = p2p["put_many_8_signal"]
    assert (chain["batches"], chain["commands"], chain["strong_signals"], chain["system_fences"]) == (1, 9, 1, 0)
    assert p2p["put_many_32_flush"]["system_fences"] == 1 and p2p["put"]["system_fences"] == 1
    assert p2p["quiet"]["completion_waits"] == 0                      # vacuous on peer memory
    assert p2p["put_inline24"]["inline_puts"] == 1
    queued = ring["put_many_8_signal"]
    assert (queued["batches"], queued["reservations"], queued["commands"], queued["completion_waits"]) == (1, 1, 9, 1)
    assert ring["quiet"]["completion_waits"] == 1
    assert "unsupported" in ring["put_inline24"] and ring["put_inline64"]["inline_puts"] == 1
    with pytest.raises(KeyError, match="unknown Tier-1 operation"):
        tier1_program("put_many_7")


def test_planned_fragments_compile_per_transport():
    from aboleth_b200 import planned_phase as pp

    with ab.compilation("p2p"):
        put = pp.compile_planned_put_artifact(max_bytes=4096, cta_exclusive=True)
        drain = pp.compile_planned_drain_artifact()
    assert [n for n, _ in put.parameters] == [n for n, _ in pp.PUT_SLOTS]
    assert "__device__ __forceinline__ void phase_put_fragment(" in put.source and put.facts["completion"] == "vacuous"
    assert drain.facts["completion_waits"] == 0
    with ab.compilation("proxy", queue_capacity=64):
        put = pp.compile_planned_put_artifact(max_bytes=4096)
        drain = pp.compile_planned_drain_artifact()
        fence = pp.compile_planned_fence_artifact(artifact=ab.Artifact.INLINE_FRAGMENT)
        publish = pp.compile_planned_publish_artifact()
    assert put.facts["reservations"] == 1 and drain.facts["completion_waits"] == 1
    assert fence.artifact == "inline_fragment" and [n for n, _ in publish.parameters] == ["endpoint", "only_if_advanced"]
    with pytest.raises(ValueError, match="max_bytes must be positive"):
        pp.planned_put_program(max_bytes=0)


def test_binding_becomes_a_fragment_that_a_kernel_invokes():
    """A physicalised attachment as a fragment of an external transport program: the kernel states
    invoke_phase with the slots, the splice carries the planned interval, the pipeline lowers it."""
    from aboleth_b200.compiler import compile_program, materialize_phases
    from aboleth_b200.transport_binding import transport_program_text

    compiled = ab.build_moe_pattern(ab.MoEPatternSpec(max_tokens=64, hidden=512, top_k=4, num_ranks=4)).compile()
    phys = ab.physicalize_pattern(compiled, [
        ab.PhaseBinding(None, "experts", "dispatch", "pack_kernel", "after_pack", 4, "fused_kernel",
                        operations=("dispatch.values", "dispatch.count"), artifact=ab.Artifact.STANDALONE_KERNEL)])
    binding = phys.binding("dispatch")
    program_id = phys.manifest("dispatch").program_id
    plan = transport_program_text("moe", [binding.to_fragment(program_id, interval=4, capacities=(64, 32))])
    assert plan.startswith(f"program moe kind=transport_program\nphase dispatch program_id={program_id} "
                           "interval=4 capacities=64,32\n")
    assert "planned_wait" in plan and " reuse=" not in plan
    names = [slot.name for slot in binding.slots()]
    invoke = binding.invoke_text(program_id, **{name: f"a{i}" for i, name in enumerate(names)})
    assert invoke.split()[:3] == ["invoke_phase", str(program_id), "a0"] and len(invoke.split()) == 2 + len(names)
    with pytest.raises(ValueError, match="missing slots"):
        binding.invoke_text(program_id)
    with pytest.raises(ValueError, match="planned interval or a reuse distance"):
        binding.to_fragment(program_id)
    kernel = ("program pack backend=rdma\n" + "".join(f"arg a{i} u64\n" for i in range(len(names))) +
              "for it 0 8 {\n  " + invoke + "\n}\n")
    spliced = materialize_phases(kernel, plan)
    assert "invoke_phase" not in spliced and "interval=4" in spliced and "queue_capacity=32" in spliced
    with ab.compilation("rdma", rank=0, world_size=4):
        lowered = compile_program(kernel, plan=plan)
    assert lowered.cuda and lowered.facts["strong_signals"] >= 1
    # A fragment may keep a reuse distance of its own instead of a planned interval.
    own = binding.to_fragment(program_id, reuse=2)
    assert "phase " not in own and " reuse=2" in own


def test_publication_strategy_follows_resources_and_realisation():
    """Every publication strategy is reachable, and which one a phase gets follows from what the
    client's kernels offer (reference selection: python/aboleth/pattern.py:887-1079)."""
    from aboleth_b200.pattern import P2PRealizationProfile, _select_schedule

    profile = P2PRealizationProfile(
        direct_destination_kernel="direct_k",
        direct_publication_kernels=(("coalesced_kernel", "pub_k"), ("separate_kernel", "pub_k"),
                                    ("packed_doorbell", None)),
        parallel_copy_kernel="copy_k",
        parallel_publication_kernels=(("fused_kernel", None), ("coalesced_kernel", "pub_k"),
                                      ("consumer_prologue", None), ("separate_kernel", "pub_k")))
    peers = {1: "p2p", 2: "p2p"}

    def pick(resources, **facts):
        return _select_schedule("phase", 1 << 20, "p2p", 4, 8, resources, ("dst",), **facts)

    base = dict(peers=peers, realization=profile)
    # indexed items with a proven direct destination: written in place
    s = pick(ab.PhaseResources(**base), per_item=True, retargeted=True)
    assert (s.strategy, s.kernel, s.publication_strategy, s.publication_kernel) == \
        ("direct_destination", "direct_k", "coalesced_kernel", "pub_k")   # no fused form for direct writes here
    s = pick(ab.PhaseResources(**base, coalesce_publication_wait=False), per_item=True, retargeted=True)
    assert s.publication_strategy == "separate_kernel"
    s = pick(ab.PhaseResources(**base, packed_doorbell=True), per_item=True, retargeted=True)
    assert s.publication_strategy == "packed_doorbell" and s.publication_kernel is None
    # the same items without the proof (or with direct writes disabled): staged parallel copy
    s = pick(ab.PhaseResources(**base), per_item=True, retargeted=False)
    assert (s.strategy, s.kernel, s.publication_strategy) == ("parallel_copy", "copy_k", "fused_kernel")
    s = pick(ab.PhaseResources(**base, direct_destination=False, fused_publication=False),
             per_item=True, retargeted=True)
    assert (s.strategy, s.publication_strategy) == ("parallel_copy", "coalesced_kernel")
    # contiguous spans: the consumer's prologue may take the publication over between two ranks
    two = dict(peers={1: "p2p"}, realization=profile, fused_publication=False)
    s = pick(ab.PhaseResources(**two, coalesce_return_with_consumer=True, consumer_grid_size=1))
    assert s.publication_strategy == "consumer_prologue"
    s = pick(ab.PhaseResources(**two, coalesce_return_with_consumer=True, consumer_grid_size=0))
    assert s.publication_strategy == "coalesced_kernel"
    # a cyclic plan double-buffers a contiguous copy; small payloads ride in their producer
    assert pick(ab.PhaseResources(**base, iteration_count=8)).buffer_depth == 2
    small = _select_schedule("phase", 512, "p2p", 1, 1, ab.PhaseResources(**base), ("dst",))
    assert (small.strategy, small.publication_strategy) == ("inline_transport", "inline")
    # queue transports publish with their doorbell
    queued = _select_schedule("phase", 1 << 20, "proxy", 4, 8, ab.PhaseResources(peers={1: "proxy"}), ("dst",))
    assert (queued.strategy, queued.publication_strategy) == ("parallel_copy", "packed_doorbell")
