"""Native planning passes against hand-computed cases (no GPU)."""

import pytest

from aboleth_b200 import abi
from aboleth_b200.compiler import compilation
from aboleth_b200.endpoint_profiles import (SEED_PROFILES, ProbeSample, ProfileStore,
                                            fit_profile, resolve_profiles)
from aboleth_b200.moe import MoESpec, compile_moe_plan
from aboleth_b200.planning import (CommunicationDataflow, CommunicationRegion, RegionEffect,
                                   TransportPhase, plan_endpoint_work, plan_storage, plan_transport,
                                   simplify_communication_dataflow)
from aboleth_b200.shapes import plan_shape_family


def test_shape_family_variants_and_selector():
    f = plan_shape_family("f", minimum=1, maximum=4096, slots=2, iteration_bound=128)
    assert [v.capacity for v in f.variants] == [1, 2, 4, 8, 16, 32, 64, 128, 4096]
    assert [v.control_base for v in f.variants][:3] == [0, 2, 4] and f.uniform_required
    assert f.select(1).capacity == 1 and f.select(100).capacity == 128 and f.select(129).capacity == 4096
    assert f.control_domain(f.select(3), 1) == 2 * 2 + 1
    with pytest.raises(ValueError):
        f.select(5000)
    assert [v.capacity for v in plan_shape_family("g", minimum=5, maximum=100).variants] == [8, 16, 32, 64, 128]
    assert [v.capacity for v in plan_shape_family("h", minimum=1, maximum=100, uniform=False).variants] == [128]
    with compilation("p2p", passes="-shape-specialization"):
        assert [v.capacity for v in plan_shape_family("i", minimum=1, maximum=100).variants] == [128]


def _partition(**kw):
    base = dict(backend="p2p", peers=[1, 2, 3], platform="B200", queueMemory="none", peerLink="NV18",
                availableLanes=16, participantLanes=[16] * 4, participantLinks=["NV18"] * 3)
    base.update(kw)
    return base


def test_endpoint_lanes_slices_and_strides():
    seed = [SEED_PROFILES["B200_NV18"]]
    (l,) = plan_endpoint_work("w", payload_bytes=5 * 262144, max_items=1000, partitions=[_partition()],
                              profiles=seed, rank_count=4)
    assert l.lanes == 8 and l.sender_warps == 8      # ceil(5) -> next power of two 8, under the cap 16
    assert l.slices[0] == (0, 125) and l.slices[-1] == (875, 1000) and l.slice_quotient == 125
    assert l.sender_grid == (3, 8) and l.receiver_grid == (3, 1) and l.receiver_lanes_per_program == 8
    assert l.ready_stride == 16 and l.signal_slots == 4 * 16 and l.count_lane == 0
    # Remainder rows are spread by the quotient/remainder rule.
    (r,) = plan_endpoint_work("w", payload_bytes=4 * 262144, max_items=10, partitions=[_partition()],
                              profiles=seed, rank_count=4)
    assert r.lanes == 4 and r.slices == ((0, 2), (2, 5), (5, 7), (7, 10))
    # Small payloads and unknown platforms stay on one lane.
    (s,) = plan_endpoint_work("w", payload_bytes=1000, max_items=64, partitions=[_partition()], profiles=seed)
    assert s.lanes == 1
    (u,) = plan_endpoint_work("w", payload_bytes=1 << 30, max_items=64,
                              partitions=[_partition(platform="H100")], profiles=seed)
    assert u.lanes == 1 and u.profile_identity == ""
    with compilation("p2p", passes="-endpoint-fanout"):
        (o,) = plan_endpoint_work("w", payload_bytes=1 << 30, max_items=64, partitions=[_partition()], profiles=seed)
        assert o.lanes == 1
    with pytest.raises(Exception, match="common endpoint budget"):
        plan_endpoint_work("w", payload_bytes=1, max_items=64, partitions=[_partition(availableLanes=4)],
                           profiles=seed, rank_count=4)


def test_storage_reached_rows_and_prefix_binding():
    regions = [CommunicationRegion("tokens", 64, 512, immutable=True, valid_count="n"),
               CommunicationRegion("received", 64 * 8, 256), CommunicationRegion("out", 64, 512, escapes=True)]
    effects = [RegionEffect("tokens", "read", "pack", (0, 64), prefix=True),
               RegionEffect("received", "write", "dispatch", (0, 128)),
               RegionEffect("received", "read", "experts", (0, 512), through=128)]
    plan = plan_storage(regions, effects)
    assert plan["tokens"]["prefix_binding"] and plan["tokens"]["physical_rows"] == 64
    assert plan["received"]["reached_rows"] == 128 and plan["received"]["bytes"] == 128 * 256
    assert plan["received"]["last_reader"] == "experts" and plan["out"]["physical_rows"] == 64
    with compilation("p2p", passes="-plan-storage"):
        off = plan_storage(regions, effects)
    assert off["received"]["physical_rows"] == 512 and not off["tokens"]["prefix_binding"]


def test_transport_intervals_modes_and_blob():
    plan = plan_transport({1: "p2p", 2: "p2p", 3: "rdma"}, [
        TransportPhase("dispatch", "rdma", commands=3, reuse=8, queue_capacity=64, completion_before="next_pack"),
        TransportPhase("small_queue", "rdma", commands=4, reuse=64, queue_capacity=17),
        TransportPhase("peer", "p2p", commands=3, reuse=8),
        TransportPhase("unordered", "efa", commands=1, reuse=4)])
    assert plan["launch_partitions"] == [{"backend": "p2p", "peers": [1, 2]}, {"backend": "rdma", "peers": [3]}]
    assert plan["topology"] == "mixed"
    by = {p["name"]: p for p in plan["phases"]}
    assert by["dispatch"]["completion_interval"] == 8 and by["dispatch"]["requires_final_drain"]
    assert by["small_queue"]["completion_interval"] == 4      # min(64, 16, (17-1)/4) = 4
    assert by["peer"]["completion_interval"] == 0 and by["peer"]["publication_mode"] == "P2PRelease"
    assert by["unordered"]["publication_mode"] == "FenceThenSignal" and not by["unordered"]["checked_publication"]
    blob = bytes.fromhex(by["dispatch"]["plan_blob"])
    assert len(blob) == 112
    record = abi.TransportPhasePlan.from_buffer_copy(blob)
    assert (record.abi_version, record.byte_size, record.completion_interval) == (4, 112, 8)
    assert record.topology_kind == 1 and record.completion_before_phase == 3 and record.path_mtu == 4096


def test_dataflow_simplification_rules():
    d = CommunicationDataflow()
    for name, flags in {"a": {}, "b": {}, "staging": {}, "final": dict(registered=True, donated=True),
                        "sent": {}, "unused_dst": {}, "out": dict(escapes=True)}.items():
        d.region(name, 8, 8, **flags)
    d.reduction("one", ["a"], "b")
    d.opaque_stage("experts", ["b"], "staging", bindable_outputs=True)
    d.copy("to_final", "staging", "final")
    d.transfer("ret", "final", "sent")
    d.transfer("dead", "b", "unused_dst")
    d.transform("gather", "sent", "out")
    s = simplify_communication_dataflow(d)
    kinds = {op["name"]: op["kind"] for op in s.operations}
    assert kinds["one"] == "transfer"                      # singleton reduction
    assert not s.has("to_final") and not s.has("dead")     # forwarded copy, dead transfer
    experts = next(op for op in s.operations if op["name"] == "experts")
    assert experts["writes"] == "final" and "staging" in s.unallocated_regions
    with compilation("p2p", passes="-dead-communication,-plan-storage"):
        kept = simplify_communication_dataflow(d)
    assert kept.has("dead") and kept.has("to_final")


def test_moe_plan_reproduces_the_reference_decisions():
    plan = compile_moe_plan(MoESpec(capacity=64, hidden=256, top_k=4, experts=16, ranks=4))
    m = plan.manifest()
    assert set(m["removed"]) == {"expert_copy", "return.metadata", "return.count"}
    assert m["forwarded_expert_output"] and m["prefix_bound_inputs"] == ["tokens"]
    assert m["received_rows"] == 4 * 64                    # not ranks * capacity * top_k
    assert m["phases"]["dispatch"]["publication_mode"] == "P2PRelease"


def test_profile_fit_store_and_resolution(tmp_path, monkeypatch):
    # One lane: 20 GB/s; sixteen lanes approach 94 GB/s (the shape of the H100 NV6 calibration fixture).
    def us(size, lanes):
        return size / (min(20e9 * lanes, 94e9)) * 1e6 + 2.5
    samples = [ProbeSample(size, lanes, 8, us(size, lanes))
               for size in (65536, 262144, 1 << 20, 4 << 20, 16 << 20) for lanes in (1, 2, 4, 8, 16)]
    samples += [ProbeSample(65536, 1, w, t) for w, t in ((1, 6.9), (2, 5.2), (4, 4.4), (8, 4.7))]
    fit = fit_profile(samples, backend="p2p", platform="B200", queue_memory="none", peer_link="NV18",
                      identity="probe:test")
    assert fit is not None and fit.max_lanes == 8 and fit.sender_warps == 4   # 8 lanes reach 95 % of 16
    flat = [ProbeSample(size, lanes, 1, 10.0) for size in (65536, 1 << 20, 4 << 20) for lanes in (1, 2, 4)]
    assert fit_profile(flat, backend="p2p", platform="B200", queue_memory="none", peer_link="NV18",
                       identity="x") is None
    monkeypatch.setenv("ABOLETH_PROFILE_DIR", str(tmp_path))
    store = ProfileStore()
    key = store.key("p2p", "B200", "none", "NV18")
    assert store.load(key) is None
    store.save(key, fit)
    assert store.load(key) == fit and store.list() == [key.replace(":", "_")]
    from aboleth_b200 import Transport
    assert resolve_profiles({1: Transport.P2P}, {1: "NV18"})["p2p"] == fit
    store.retire(key)
    assert resolve_profiles({1: Transport.P2P}, {1: "NV18"})["p2p"] == SEED_PROFILES["B200_NV18"]
    (tmp_path / "broken.json").write_text("{not json")
    assert store.load("broken") is None
    assert SEED_PROFILES["B200_NV18"].bytes_per_endpoint == 262144 and SEED_PROFILES["B200_NV18"].max_lanes == 16
