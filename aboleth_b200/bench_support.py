"""Measurement helpers shared by ``bench.py`` and the benchmark scripts.

Timing rules used everywhere here: CUDA events on the launching stream after
warm-up, ``torch.cuda.synchronize`` on both sides, the maximum over ranks for
anything multi-GPU, and either inputs that rotate through more than the L2
capacity or an explicit L2 flush between timed iterations.
"""
from __future__ import annotations

import statistics
from typing import Optional

import torch

from .moe import MoESpec
from .moe.reference import standin_layer_reference
from .parallel.ep import ExpertParallelLayer
from .world import World

L2_BYTES = 126 * 1024 * 1024
# NVLink 5 per direction per GPU: the rate a one-directional peer copy reached on 8 x B200
# (benchmarks/peer_copy_bench.py measures it) and the nominal link rate.  Fractions are reported
# against both.
NVLINK_GBS = 770.0
NVLINK_NOMINAL_GBS = 900.0

_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0,
          "source": "fallback"}


def set_peaks(peaks: dict) -> None:
    """Roofline denominators measured on the machine at hand (copy bandwidth, cuBLAS rate); the
    benchmark scripts load them from a record beside the checkout when there is one."""
    _PEAKS.update(peaks)


def measured_peaks() -> dict:
    return dict(_PEAKS)


def sync_ranks(distributed: bool) -> None:
    """Device-side alignment of the ranks (one-element all-reduce), then a host sync."""
    if distributed:
        import torch.distributed as dist
        token = torch.zeros(1, device="cuda")
        dist.all_reduce(token)
    torch.cuda.synchronize()


def device_max(value: float, distributed: bool) -> float:
    if not distributed:
        return float(value)
    import torch.distributed as dist
    t = torch.tensor([value], dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def device_max_vector(values: list[float], distributed: bool) -> list[float]:
    if not distributed:
        return list(values)
    import torch.distributed as dist
    t = torch.tensor(values, dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.tolist()


class RankAligner:
    """A kernel that ends on every rank within a flag's flight time of the others: each rank
    stores a flag to every peer and waits (bounded) for all of theirs.  Enqueued right before a
    timed bracket, it takes the ranks' launch skew out of the bracket - the same purpose as the
    reference's timer-alignment all-reduce (experiments/dsl/moe/moe_common.py:173-202), on the
    device instead of through a collective."""

    def __init__(self, world: World, tag: str = "align"):
        self.world, self.epoch = world, 0
        n = world.world_size
        if n == 1:
            return
        self.arena = world.runtime.allocate(2 * n * 16 + n * 8)
        reg = world.register(self.arena, network=False)
        table = world.exchange_regions([
            world.region("align_recv", reg, offset=n * 16, length=n * 16),
            world.region("align_flags", reg, offset=2 * n * 16, length=n * 8)], tag=tag)
        self.tabs = (table.addresses("align_recv"), table.addresses("align_flags"))
        self.flags = self.arena[2 * n * 16:].view(torch.int64)
        self.status = torch.zeros(2, dtype=torch.int64, device=world.torch_device)

    def __call__(self) -> None:
        if self.world.world_size == 1:
            return
        from .ops import alltoall
        alltoall(self.arena, *self.tabs, self.flags, self.status, stride=16, nbytes=16,
                 epoch0=self.epoch, rank=self.world.rank, world=self.world.world_size, lanes=1,
                 rounds=1, mode="vector", threads=32)
        self.epoch += 1


class L2Flusher:
    def __init__(self, device):
        self.buf = torch.empty(2 * L2_BYTES, dtype=torch.uint8, device=device)

    def __call__(self) -> None:
        self.buf.fill_(1)


class EpLayerBench:
    """DeepSeek-V3-shape MoE layer with seeded synthetic inputs."""

    def __init__(self, world: World, *, tokens: int, hidden: int, experts: int, top_k: int,
                 group: int, seed: int, tag: str = "bench", weighted: bool = True):
        # weighted: the expert stage leaves expert-contiguous, unweighted rows and the combine
        # kernel applies the gates (the product path); False: the experts apply the gates and the
        # combine sums one partial row per record (the reference's split).
        self.weighted = weighted
        self.world, self.tokens = world, tokens
        self.spec = MoESpec(capacity=tokens, hidden=hidden, top_k=top_k, experts=experts,
                            ranks=world.world_size, value_type="f8E4M3FN", scale_group=group)
        self.layer = ExpertParallelLayer(world, self.spec, tag=tag)
        dev = world.torch_device
        per_copy = tokens * hidden * 2
        self.copies = min(8, max(2, -(-2 * L2_BYTES // per_copy)))
        self.l2_policy = (f"inputs rotate through {self.copies} buffers "
                          f"({self.copies * per_copy >> 20} MiB) and the receive segments exceed L2")
        g = torch.Generator(device=dev).manual_seed(seed)
        self.x = [torch.randn(tokens, hidden, generator=g, device=dev).to(torch.bfloat16)
                  for _ in range(self.copies)]
        self.logits = [torch.randn(tokens, experts, generator=g, device=dev)
                       for _ in range(self.copies)]
        self.counter = 0
        self.flusher: Optional[L2Flusher] = None
        self.align = RankAligner(world, tag=f"{tag}.align")

    def step(self) -> torch.Tensor:
        i = self.counter % self.copies
        self.counter += 1
        return self.layer.forward(self.x[i], self.logits[i], self._experts(self.weighted))

    def _experts(self, weighted: bool):
        return self.layer.standin_experts_grouped if weighted else self.layer.standin_experts

    def check(self) -> None:
        torch.cuda.synchronize()
        self.layer.check()

    def verify(self) -> int:
        """Rows of one step's output outside the fp8 tolerance of the fp32 oracle."""
        out = self.layer.forward(self.x[0], self.logits[0], self._experts(self.weighted)).float()
        torch.cuda.synchronize()
        ids = self.layer.slot.topk_ids[: self.tokens]
        weights = self.layer.slot.topk_weights[: self.tokens]
        expected, tol = standin_layer_reference(self.x[0], ids.long(), weights, fp8=True,
                                                group=self.spec.scale_group,
                                                amax_floor=self.spec.quant_amax_floor)
        err = (out - expected).abs().amax(dim=-1)
        bad = int((~(err <= tol)).sum().item())  # NaN rows count as errors
        return bad

    def _traffic(self) -> dict:
        """Bytes this rank moved in the last step (records it sent / got back)."""
        s, slot = self.spec, self.layer.slot
        slots = slot.source_slots[: self.tokens]
        sent = (slots >= 0).sum(dim=0).tolist()
        remote = sum(n for d, n in enumerate(sent) if d != slot.rank)
        total = sum(sent)
        record = s.row_bytes + s.metadata_words * 4
        return {"records_total": total, "records_remote": remote,
                "dispatch_remote_bytes": remote * record, "combine_remote_bytes": remote * s.hidden * 2,
                "dispatch_local_hbm_bytes": self.tokens * s.hidden * 2 + total * record,
                "combine_local_hbm_bytes": total * s.hidden * 2 * 2 + self.tokens * s.hidden * 2}

    def phase_times(self, *, steps: int, distributed: bool, flush: bool = False,
                    weighted: Optional[bool] = None) -> dict:
        slot, layer = self.layer.slot, self.layer
        weighted = self.weighted if weighted is None else weighted
        experts = self._experts(weighted)
        if flush and self.flusher is None:
            self.flusher = L2Flusher(self.world.torch_device)
        ev = lambda: torch.cuda.Event(enable_timing=True)  # noqa: E731
        d_ms, c_ms = [], []
        for it in range(steps + 3):
            i = self.counter % self.copies
            self.counter += 1
            if flush:
                self.flusher()
            sync_ranks(distributed)
            e0, e1, e2, e3 = ev(), ev(), ev(), ev()
            # Keep the GPU busy (about 200 us) while the host enqueues the alignment kernel, the events
            # and the phase, so that the bracket measures the kernel and not the host: a host that
            # enqueues the phase after the alignment kernel has ended lets the ranks start apart.
            torch.cuda._sleep(400_000)
            self.align()   # the ranks leave this kernel together: launch skew stays out of the bracket
            e0.record()
            res = slot.dispatch(self.x[i], logits=self.logits[i])
            e1.record()
            staged = experts(res, slot.expert_output)
            offsets, rows = staged if isinstance(staged, tuple) else (None, slot.expert_output)
            if flush:
                self.flusher()
            sync_ranks(distributed)
            torch.cuda._sleep(400_000)
            self.align()
            e2.record()
            slot.combine(rows, expert_offsets=offsets)
            e3.record()
            torch.cuda.synchronize()
            if it >= 3:
                d_ms.append(e0.elapsed_time(e1))
                c_ms.append(e2.elapsed_time(e3))
        d = statistics.median(device_max_vector(d_ms, distributed)) * 1e3
        c = statistics.median(device_max_vector(c_ms, distributed)) * 1e3
        self.check()
        # The kernels' own phase stamps for one more step (this rank's view).
        slot.enable_trace()
        sync_ranks(distributed)
        res = slot.dispatch(self.x[0], logits=self.logits[0])
        torch.cuda.synchronize()
        kernel_trace = {"dispatch": slot.trace()}
        staged = experts(res, slot.expert_output)
        offsets, rows = staged if isinstance(staged, tuple) else (None, slot.expert_output)
        slot.trace_buffer.zero_()
        sync_ranks(distributed)
        slot.combine(rows, expert_offsets=offsets)
        torch.cuda.synchronize()
        kernel_trace["combine"] = slot.trace()
        slot.trace_buffer = None
        traffic = self._traffic()
        peaks = measured_peaks()
        roof = {"traffic": traffic, "denominators": peaks["source"]}
        if self.world.world_size > 1:
            td = traffic["dispatch_remote_bytes"] / (NVLINK_GBS * 1e3)  # us
            tc = traffic["combine_remote_bytes"] / (NVLINK_GBS * 1e3)
            nominal = NVLINK_GBS / NVLINK_NOMINAL_GBS
            roof.update({"bound": "nvlink egress per direction: 770 GB/s measured peer copy (900 nominal)",
                         "dispatch_roof_us": td, "combine_roof_us": tc,
                         "dispatch_frac": td / d if d else None, "combine_frac": tc / c if c else None,
                         "dispatch_frac_of_900": td * nominal / d if d else None,
                         "combine_frac_of_900": tc * nominal / c if c else None})
        else:
            td = traffic["dispatch_local_hbm_bytes"] / (peaks["hbm_gbs"] * 1e3)
            tc = traffic["combine_local_hbm_bytes"] / (peaks["hbm_gbs"] * 1e3)
            roof.update({"bound": f"hbm {peaks['hbm_gbs']} GB/s ({peaks['source']} copy)",
                         "dispatch_roof_us": td, "combine_roof_us": tc,
                         "dispatch_frac": td / d if d else None, "combine_frac": tc / c if c else None})
        return {"dispatch_us": d, "combine_us": c, "tokens_per_rank": self.tokens, "roofline": roof,
                "combine": "bf16 gate-weighted in kernel" if weighted else "bf16 unweighted sum of partials",
                "kernel_trace_us": kernel_trace,
                "dispatch_us_min": min(device_max_vector(d_ms, distributed)) * 1e3,
                "combine_us_min": min(device_max_vector(c_ms, distributed)) * 1e3,
                "l2": "flushed before each bracket" if flush else self.l2_policy}

    def end_to_end(self, *, steps: int, distributed: bool) -> dict:
        s = self.spec
        hosts = [(x.cpu().pin_memory(), l.cpu().pin_memory()) for x, l in zip(self.x, self.logits)]
        for k in range(3):
            self.layer.forward_from_host(*hosts[k % len(hosts)], self._experts(self.weighted),
                                         prefetch=hosts[(k + 1) % len(hosts)])
        torch.cuda.synchronize()
        sync_ranks(distributed)
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for k in range(steps):
            # Step k's inputs were copied under step k-1's kernels; step k+1's copy starts now.
            result = self.layer.forward_from_host(*hosts[k % len(hosts)], self._experts(self.weighted),
                                                  prefetch=hosts[(k + 1) % len(hosts)])
            torch.cuda.current_stream().synchronize()  # the caller reads the result every step
            if int(result[0]) != 0:
                raise RuntimeError(f"transport status {result.tolist()}")
        stop.record()
        torch.cuda.synchronize()
        ms = device_max(start.elapsed_time(stop), distributed) / steps
        value = self.world.world_size * self.tokens / (ms * 1e-3)
        return {"value": value, "unit": "tokens/s", "ms_per_step": ms,
                "h2d_bytes_per_step": self.tokens * s.hidden * 2 + self.tokens * s.experts * 4,
                "d2h_bytes_per_step": 32,
                "overlap": "each step's inputs are copied from pinned host memory on a side stream under "
                           "the previous step's kernels; the result is read back after every step"}


def alltoall_sweep(world: World, distributed: bool, sizes=None, *, rounds: int = 20,
                   chains=(1, 8, 64), chain_sizes=(1 << 10, 1 << 16, 1 << 20)) -> list[dict]:
    """Bus bandwidth of the all-to-all kernel over every power-of-two message size from 1 KiB to
    256 MiB per peer, and of put/signal chains (``chain`` puts closed by one signal) at
    ``chain_sizes``; ``busbw = (n-1) * S / t`` with t the mean round time of the slowest rank
    (definition: experiments/bench/README.md:111-131 of the reference)."""
    from .ops import alltoall, check_payload, fill_payload

    n, rank, dev = world.world_size, world.rank, world.torch_device
    sizes = list(sizes or [1 << e for e in range(10, 29)])
    top = max(sizes)
    max_lanes = 64   # 32 lanes per peer up to 32 MiB, 64 beyond (messages that no longer fit L2)
    arena = world.runtime.allocate(2 * n * top + n * max_lanes * 8)
    reg = world.register(arena, network=False)
    recv = world.region("a2a_recv", reg, offset=n * top, length=n * top)
    flags = world.region("a2a_flags", reg, offset=2 * n * top, length=n * max_lanes * 8)
    table = world.exchange_regions([recv, flags], tag="a2a")
    send = arena[: n * top]
    my_flags = arena[2 * n * top:].view(torch.int64)
    status = torch.zeros(2, dtype=torch.int64, device=dev)
    errors = torch.zeros(1, dtype=torch.int64, device=dev)
    tabs = (table.addresses("a2a_recv"), table.addresses("a2a_flags"))
    out = []
    for size in sizes:
        for p in range(n):
            fill_payload(send[p * top:], size, 4242, rank, p)
        # Keep a sweep short: fewer rounds once a round moves hundreds of megabytes.
        r = max(3, min(rounds, (4 << 30) // max(size * max(n - 1, 1), 1)))
        cases = [("vector", 1)] if size < (1 << 20) else [("bulk", 1)]
        if size in (1 << 22, 1 << 26):
            cases = [("vector", 1), ("bulk", 1)]
        cases += [("vector", c) for c in chains if c > 1 and size in chain_sizes]
        for mode, chain in cases:
            # 64 lanes only help the bulk-copy mode; the vector mode loses with them (384 against 617 GB/s)
            lanes = max(1, min(max_lanes if (size >= (64 << 20) and mode == "bulk") else 32, size // 16384))
            if size // lanes // chain < 16:
                continue
            my_flags.zero_()
            errors.zero_()
            sync_ranks(distributed)
            kwargs = dict(stride=top, nbytes=size, rank=rank, world=n, lanes=lanes, mode=mode,
                          chain=chain)
            alltoall(send, *tabs, my_flags, status, epoch0=0, rounds=3, **kwargs)
            sync_ranks(distributed)
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            alltoall(send, *tabs, my_flags, status, epoch0=3, rounds=r, **kwargs)
            stop.record()
            torch.cuda.synchronize()
            t = device_max(start.elapsed_time(stop), distributed) / r * 1e-3
            for s in range(n):
                if s != rank:
                    check_payload(arena[n * top + s * top:], size, 4242, s, rank, errors)
            sync_ranks(distributed)
            bus = (n - 1) * size / t / 1e9
            out.append({"bytes_per_peer": size, "mode": mode, "chain": chain, "lanes": lanes,
                        "rounds": r, "round_us": t * 1e6, "busbw_gbs": bus,
                        "frac_of_770": bus / NVLINK_GBS, "frac_of_900": bus / NVLINK_NOMINAL_GBS,
                        "wrong_words": int(errors.item()), "status": status.tolist()})
    del arena
    return out
