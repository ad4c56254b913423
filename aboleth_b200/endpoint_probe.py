"""Bounded endpoint probe: how one peer link scales with lanes (CTAs) and sender warps.

``measure`` is collective over a connected :class:`World`.  Every rank sends to the next GPU
of its host, so the sends form a permutation and each link carries one stream each way.  Per
lane and iteration: the CTA copies the lane's slice into the partner's receive buffer and
publishes one epoch in the lane's flag (sender-completed throughput; on peer memory the
release store is the completion).  No kernel waits for another rank, so the probe also runs
with a single GPU in ``loopback`` mode (the partner is the rank itself), which measures the
copy engine of the SMs rather than NVLink.

The sweep, sizes, trial counts and the world-rate rule (a trial lasts as long as its slowest
rank) follow the reference (python/aboleth/endpoint_probe.py:25-29,84-224); the kernel is
``probe_send_kernel`` of this package, and the fit is :func:`endpoint_profiles.fit_profile`.

    torchrun --nproc-per-node 2 -m aboleth_b200.endpoint_probe --save
"""
from __future__ import annotations

import argparse
import json
import statistics
import time
from dataclasses import asdict
from typing import Optional, Sequence

import torch

from .endpoint_profiles import EndpointProfile, ProbeSample, ProfileStore, fit_profile

FIT_BYTES = (64 << 10, 256 << 10, 1 << 20, 4 << 20, 16 << 20)
HOLDOUT_BYTES = (512 << 10, 2 << 20, 8 << 20)
PROBE_LANES = {"p2p": (1, 2, 4, 8, 16, 32)}
PROBE_WARPS = (1, 2, 4, 8, 16)
TRIALS = 5                 # measured, after one warm-up trial
TRIAL_BYTES = 32 << 20     # at most, per lane set and trial
ITERATIONS = (4, 32)


def partners(world, *, loopback: bool = False) -> tuple[Optional[int], Optional[int]]:
    """(send to, receive from) among the p2p peers of this rank's host; ``None`` if absent."""
    if loopback:
        return world.rank, world.rank
    topology = world.topology
    host = topology[world.rank].hostname
    group = sorted(r for r, info in topology.items() if info.hostname == host)
    if len(group) < 2:
        return None, None
    at = group.index(world.rank)
    to, source = group[(at + 1) % len(group)], group[at - 1]
    kinds = dict(world.transport_geography)
    return (to if kinds.get(to) == "p2p" else None, source if kinds.get(source) == "p2p" else None)


def _gather(world, tag: str, value):
    if world.world_size == 1:
        return [value]
    images = world.bootstrap.all_gather(tag, json.dumps(value).encode())
    return [json.loads(images[r]) for r in range(world.world_size)]


def _pattern(size: int, rank: int, device) -> torch.Tensor:
    values = torch.arange(size, device=device, dtype=torch.int32) * 7 + rank * 13
    return values.remainder(251).to(torch.uint8)


def measure(world, tag: str = "probe", *, loopback: bool = False,
            fit_bytes: Sequence[int] = FIT_BYTES, holdout_bytes: Sequence[int] = HOLDOUT_BYTES,
            lanes: Sequence[int] = PROBE_LANES["p2p"], warps: Sequence[int] = PROBE_WARPS,
            trials: int = TRIALS) -> dict:
    """``{"samples": [ProbeSample...], "sender_warps", "world", "seconds"}`` or ``{"reason": ...}``."""
    from .ops._kernels import _I, _U64, _VP, call, declare, ptr, stream_ptr

    declare("ab_probe_send", [_VP, _U64, _U64, _VP, _U64, _I, _I, _I, _VP])
    began = time.monotonic()
    to, source = partners(world, loopback=loopback)
    images = _gather(world, tag + ".partners", [to, source])
    if all(image[0] is None for image in images):
        return {"reason": "no rank has a p2p partner on its host"}
    device = world.torch_device
    sizes = sorted(set(fit_bytes) | set(holdout_bytes))
    largest, widest = sizes[-1], max(lanes)
    tensors = {
        "probe_payload": _pattern(largest, world.rank, device),
        "probe_receive": torch.zeros(largest, device=device, dtype=torch.uint8),
        "probe_flags": torch.zeros(widest, device=device, dtype=torch.int64),
    }
    registrations = {name: world.register(t) for name, t in tensors.items()}
    table = world.exchange_regions(
        [world.region(name, registrations[name], t) for name, t in tensors.items()], tag=tag)
    starts = torch.zeros(widest, device=device, dtype=torch.int64)
    cursors = [0] * widest
    try:
        receive = int(table.addresses("probe_receive")[to]) if to is not None else 0
        flags = int(table.addresses("probe_flags")[to]) if to is not None else 0

        def cell(size: int, width: int, nwarps: int) -> list[float]:
            """Per-iteration microseconds of the measured trials on this rank (empty if it does not send)."""
            if to is None:
                return []
            chunk = (size // width) // 16 * 16
            iterations = max(ITERATIONS[0], min(ITERATIONS[1], TRIAL_BYTES // size))
            events = []
            for _ in range(trials + 1):
                begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                begin.record()
                call("ab_probe_send", ptr(tensors["probe_payload"]), receive, flags, ptr(starts), chunk,
                     width, nwarps, iterations, stream_ptr())
                end.record()
                starts[:width] += iterations
                events.append((begin, end))
            torch.cuda.synchronize()
            for lane in range(width):
                cursors[lane] += iterations * (trials + 1)
            return [b.elapsed_time(e) * 1e3 / iterations for b, e in events[1:]]

        def sweep(label: str, cells: Sequence[tuple[int, int, int]]) -> list[ProbeSample]:
            local = []
            for size, width, nwarps in cells:
                local.append(cell(size, width, nwarps))
            gathered = _gather(world, f"{tag}.{label}", local)
            out = []
            for i, (size, width, nwarps) in enumerate(cells):
                per_rank = [statistics.median(image[i]) for image in gathered if image[i]]
                if per_rank:  # a trial lasts as long as its slowest rank
                    out.append(ProbeSample(size, width, nwarps, max(per_rank)))
            return out

        # Both orders of the width axis, so that a warm link does not favour one end of it.
        warp_cells = [(s, 1, w) for s in fit_bytes for w in list(warps) + list(warps)[::-1]]
        warp_samples = sweep("warps", warp_cells)
        at64k = min(fit_bytes, key=lambda b: abs(b - 65536))
        by_warps: dict[int, float] = {}
        for s in warp_samples:
            if s.bytes == at64k:
                by_warps[s.warps] = min(by_warps.get(s.warps, float("inf")), s.microseconds)
        best = min(by_warps.values())
        sender_warps = min(w for w, t in by_warps.items() if t <= best / 0.95)
        lane_cells = [(s, l, sender_warps) for s in sizes for l in list(lanes) + list(lanes)[::-1]]
        lane_samples = sweep("lanes", lane_cells)

        torch.cuda.synchronize()
        cursor_images = _gather(world, tag + ".cursors", cursors)
        problem = ""
        if source is not None:
            # The last cells wrote every 16-byte-aligned slice of the largest size.
            expected = _pattern(largest, source, device)
            span = (largest // widest) // 16 * 16 * widest
            if not torch.equal(tensors["probe_receive"][:span], expected[:span]):
                problem = "payload mismatch"
            elif tensors["probe_flags"].tolist() != cursor_images[source]:
                problem = f"epochs {tensors['probe_flags'].tolist()} != {cursor_images[source]}"
        problems = [(r, p) for r, p in enumerate(_gather(world, tag + ".checked", problem)) if p]
        if problems:
            raise RuntimeError(f"probe check failed on rank {problems[0][0]}: {problems[0][1]}")
    finally:
        table.close()
        for registration in registrations.values():
            registration.close()
    seconds = max(_gather(world, tag + ".seconds", time.monotonic() - began))
    return {"samples": warp_samples + lane_samples, "sender_warps": sender_warps, "seconds": seconds,
            "world": {"ranks": world.world_size, "loopback": loopback, "widths": list(lanes),
                      "senders": sum(1 for image in images if image[0] is not None), "trials": trials}}


def calibrate(world, *, platform: str = "B200", peer_link: str = "NV18", loopback: bool = False,
              store: Optional[ProfileStore] = None, save: bool = False, **kwargs) -> tuple[Optional[EndpointProfile], dict]:
    """Run the probe, fit a profile and (optionally) cache it.  Returns ``(profile or None, measurement)``."""
    result = measure(world, loopback=loopback, **kwargs)
    if "reason" in result:
        return None, result
    lane_samples = [s for s in result["samples"] if s.warps == result["sender_warps"]]
    profile = fit_profile(lane_samples + [s for s in result["samples"] if s.lanes == 1],
                          backend="p2p", platform=platform, queue_memory="none", peer_link=peer_link,
                          identity=f"probe:{platform}_{peer_link}")
    if profile is not None and save and world.rank == 0:
        store = store or ProfileStore()
        store.save(store.key("p2p", platform, "none", peer_link), profile)
    return profile, result


def main(argv=None) -> int:
    import os

    import torch.distributed as dist

    import aboleth_b200 as ab

    ap = argparse.ArgumentParser(prog="aboleth_b200.endpoint_probe")
    ap.add_argument("--save", action="store_true", help="cache the fitted profile")
    ap.add_argument("--loopback", action="store_true", help="single rank: the partner is the rank itself")
    ap.add_argument("--out", default=None, help="write the samples and the fit as JSON")
    args = ap.parse_args(argv)
    rank, size = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    bootstrap = None
    if size > 1:
        dist.init_process_group("gloo", rank=rank, world_size=size)
        bootstrap = ab.TorchDistributedBootstrap(dist.group.WORLD)
    with ab.World(rank, size, device=local, bootstrap=bootstrap) as world:
        world.connect_all("p2p")
        profile, result = calibrate(world, loopback=args.loopback or size == 1, save=args.save)
        if rank == 0:
            record = {"profile": asdict(profile) if profile else None,
                      "reason": result.get("reason"), "sender_warps": result.get("sender_warps"),
                      "seconds": result.get("seconds"), "world": result.get("world"),
                      "samples": [asdict(s) for s in result.get("samples", [])]}
            line = json.dumps(record)
            print(line, flush=True)
            if args.out:
                with open(args.out, "w") as handle:
                    handle.write(line + "\n")
    if size > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
