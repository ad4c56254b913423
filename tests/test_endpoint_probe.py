"""Endpoint probe: partner selection on CPU fakes, the sweep itself on one GPU in loopback."""
from types import SimpleNamespace

import pytest


def _fake_world(rank, hosts, kinds=None):
    topology = {r: SimpleNamespace(rank=r, device=r, hostname=h) for r, h in enumerate(hosts)}
    geography = tuple((p, (kinds or {}).get(p, "p2p")) for p in range(len(hosts)) if p != rank)
    return SimpleNamespace(rank=rank, world_size=len(hosts), topology=topology,
                           transport_geography=geography)


def test_partners_form_a_ring_per_host():
    from aboleth_b200.endpoint_probe import partners

    hosts = ["a", "a", "a", "b", "b"]
    assert partners(_fake_world(0, hosts)) == (1, 2)
    assert partners(_fake_world(2, hosts)) == (0, 1)
    assert partners(_fake_world(3, hosts)) == (4, 4)
    # a lone GPU on its host has nobody to probe; loopback names itself
    assert partners(_fake_world(0, ["a", "b"])) == (None, None)
    assert partners(_fake_world(0, ["a"]), loopback=True) == (0, 0)
    # a partner reached through another transport is not a p2p partner
    assert partners(_fake_world(0, ["a", "a"], kinds={1: "proxy"})) == (None, None)


def test_fit_from_probe_shaped_samples():
    from aboleth_b200.endpoint_profiles import ProbeSample, fit_profile

    samples = []
    for size in (65536, 262144, 1 << 20, 4 << 20, 16 << 20):
        for lanes in (1, 2, 4, 8, 16):
            # a latency floor of 3 us plus bytes over lanes x 40 GB/s, saturating at 8 lanes
            us = 3.0 + size / (min(lanes, 8) * 40e3)
            samples.append(ProbeSample(size, lanes, 8, us))
    profile = fit_profile(samples, backend="p2p", platform="B200", queue_memory="none",
                          peer_link="NV18", identity="probe:test")
    assert profile is not None and profile.max_lanes == 8 and profile.sender_warps == 8
    assert profile.bytes_per_endpoint >= 4096 and profile.source == "probe"


@pytest.mark.gpu
def test_loopback_probe_measures_and_checks():
    import torch

    import aboleth_b200 as ab
    from aboleth_b200.endpoint_probe import calibrate

    torch.cuda.set_device(0)
    with ab.World(0, 1, device=0) as world:
        world.connect_all("p2p")
        profile, result = calibrate(world, loopback=True, fit_bytes=(65536, 1 << 20, 4 << 20),
                                    holdout_bytes=(8 << 20,), lanes=(1, 4, 16), warps=(1, 8), trials=2)
        assert "reason" not in result
        cells = {(s.bytes, s.lanes, s.warps) for s in result["samples"]}
        assert (1 << 20, 16, result["sender_warps"]) in cells and (65536, 1, 1) in cells
        assert all(s.microseconds > 0 for s in result["samples"])
        one = min(s.microseconds for s in result["samples"] if s.bytes == 4 << 20 and s.lanes == 1)
        many = min(s.microseconds for s in result["samples"] if s.bytes == 4 << 20 and s.lanes == 16)
        assert many < one  # sixteen CTAs copy 4 MiB faster than one
        assert profile is None or profile.max_lanes in (4, 16)
