// Planning passes (C++ core; the Python layer only builds requests and reads plans).
//
// Arithmetic follows the reference passes:
//   plan-shapes     compiler/lib/Transforms/PlanShapes.cpp:28-116
//   plan-endpoints  compiler/lib/Transforms/PlanEndpoints.cpp:128-300
//   plan-storage    compiler/lib/Transforms/PlanStorage.cpp:34-312
//   plan-transport  compiler/lib/Transforms/PlanTransport.cpp:31-747
//   simplify-communication-dataflow
//                   compiler/lib/Transforms/SimplifyCommunicationDataflow.cpp:117-360
#include "planning.hpp"

#include <algorithm>
#include <cstring>
#include <limits>

#include "aboleth/abi/transport_plan.h"
#include "ir.hpp"

namespace spec {

namespace {

long long ceil_pow2(long long v) {
    long long b = 1;
    while (b < v && b < (1ll << 62))
        b *= 2;
    return b;
}

long long floor_pow2(long long v) {
    long long b = 1;
    while (b * 2 <= v)
        b *= 2;
    return v < 1 ? 1 : b;
}

// Every quantity a planner reads (bytes, rows, lanes, iterations) is far below this; refusing
// anything larger keeps sums and small products of them inside 64 bits.
constexpr long long kLargestQuantity = 1ll << 40;
constexpr long long kLargestWalk = 4096;  // iterations of one access walk that the planners enumerate

long long quantity(const std::string &text) {
    const long long value = to_integer(text);
    if (value > kLargestQuantity || value < -kLargestQuantity)
        throw Error("'" + text + "' is outside the range a plan can use");
    return value;
}

long long num(const Op &op, const std::string &key, long long fallback = 0) {
    if (!op.has(key))
        return fallback;
    const long long value = to_integer(op.get(key));
    if (value > kLargestQuantity || value < -kLargestQuantity)
        throw Error(op.kind + " " + key + "=" + op.get(key) + " is outside the range a plan can use");
    return value;
}

std::vector<std::string> list(const std::string &text) {
    std::vector<std::string> out;
    std::size_t start = 0;
    while (start <= text.size() && !text.empty()) {
        const std::size_t comma = text.find(',', start);
        out.push_back(text.substr(start, comma == std::string::npos ? comma : comma - start));
        if (comma == std::string::npos)
            break;
        start = comma + 1;
    }
    return out;
}

std::set<std::string> switches(const Program &p) {
    std::set<std::string> on;
    for (const auto &name : list(p.get("enable")))
        on.insert(name);
    return on;
}

// ---- plan-shapes ---------------------------------------------------------------------------

void plan_shapes(const Program &p, Json &j) {
    const bool specialize = switches(p).count("shape-specialization") != 0;
    j.key("families").begin_array();
    for (const Op &f : p.body) {
        if (f.kind != "shape_family")
            continue;
        const long long maximum = num(f, "maximum"), minimum = num(f, "minimum", 1),
                        slots = num(f, "slots", 1);
        if (maximum < 1 || minimum < 1 || minimum > maximum || slots < 1)
            throw Error("shape_family " + f.get("name") + ": need 1 <= minimum <= maximum and slots >= 1");
        const long long largest = ceil_pow2(maximum);
        std::vector<long long> bounds;
        if (specialize && num(f, "uniform", 0) != 0) {
            long long limit = maximum;
            if (f.has("iteration"))
                limit = std::min(limit, num(f, "iteration"));
            const long long specialized = ceil_pow2(limit);
            for (long long b = ceil_pow2(minimum);; b *= 2) {
                bounds.push_back(b);
                if (b >= specialized)
                    break;
            }
            if (bounds.back() != largest)
                bounds.push_back(largest);
        } else {
            bounds.push_back(largest);
        }
        j.begin_object();
        j.key("name").value(f.get("name"));
        j.key("maximum_bound").value(maximum);
        j.key("slots").value(slots);
        j.key("selector").value("first_capacity_at_least_runtime_bound");
        if (f.has("iteration"))
            j.key("iteration_bound").value(num(f, "iteration"));
        j.key("uniform_required").value(bounds.size() > 1);
        j.key("private_control").value("per_variant_slot");
        j.key("mutually_exclusive_within_slot").value(true);
        j.key("payload_aliases_proven").value(false);
        j.key("control_domains").value(static_cast<long long>(bounds.size()) * slots);
        j.key("variants").begin_array();
        for (std::size_t i = 0; i < bounds.size(); ++i) {
            j.begin_object();
            j.key("capacity").value(bounds[i]);
            j.key("control_base").value(static_cast<long long>(i) * slots);
            j.key("control_count").value(slots);
            j.end_object();
        }
        j.end_array();
        j.end_object();
    }
    j.end_array();
}

// ---- plan-endpoints -------------------------------------------------------------------------

void plan_endpoints(const Program &p, Json &j) {
    const auto on = switches(p);
    const bool fanout = on.count("endpoint-fanout") != 0;
    const bool coalesce = on.count("coalesce-receives") != 0;
    j.key("programs").begin_array();
    for (const Op &work : p.body) {
        if (work.kind != "endpoint_work")
            continue;
        const long long max_items = num(work, "max_items"), payload = num(work, "payload_bytes");
        if (max_items < 1 || payload < 0)
            throw Error("endpoint_work " + work.get("name") + ": max_items >= 1 and payload_bytes >= 0");
        std::vector<const Op *> partitions, profiles;
        for (const Op &child : work.body)
            (child.kind == "partition" ? partitions : profiles).push_back(&child);
        long long ready_stride = 1, world_lanes = max_items;
        const bool ranked = work.has("rank_count");
        if (ranked && !partitions.empty()) {
            for (const auto &lanes : list(partitions[0]->get("participantLanes")))
                world_lanes = std::min(world_lanes, quantity(lanes));
            world_lanes = floor_pow2(world_lanes);
            ready_stride = fanout ? world_lanes : 1;
        }
        struct Launch {
            const Op *partition;
            long long lanes, sender_warps, receiver_lanes;
            std::string identity;
        };
        std::vector<Launch> launches;
        for (const Op *part : partitions) {
            if (ranked && num(*part, "availableLanes", 1) < world_lanes)
                throw Error("partition cannot supply the participant image's common endpoint budget");
            Launch l{part, 1, 1, 1, ""};
            for (const Op *profile : profiles) {
                if (!fanout || profile->get("backend") != part->get("backend") ||
                    profile->get("platform") != part->get("platform") ||
                    profile->get("queueMemory") != part->get("queueMemory"))
                    continue;
                const std::string link = profile->get("peerLink");
                if (!link.empty()) {
                    bool all = part->get("peerLink") == link;
                    for (const auto &other : list(part->get("participantLinks")))
                        all = all && other == link;
                    if (!all)
                        continue;
                }
                l.identity = profile->get("identity");
                l.sender_warps = num(*profile, "senderWarps", 1);
                const long long budget = std::max(num(*profile, "bytesPerEndpoint", 1), 1LL);
                const long long needed = payload / budget + (payload % budget != 0);
                const long long cap = floor_pow2(std::min({world_lanes, max_items,
                                                           num(*part, "availableLanes", 1),
                                                           num(*profile, "maxLanes", 1)}));
                l.lanes = 1;
                while (l.lanes < needed && l.lanes < cap)
                    l.lanes *= 2;
            }
            ready_stride = std::max(ready_stride, l.lanes);
            const bool grouped = coalesce && num(work, "grouped_receiver", 0) != 0;
            l.receiver_lanes = grouped ? l.lanes : 1;
            launches.push_back(l);
        }
        j.begin_object();
        j.key("name").value(work.get("name"));
        j.key("payload_bytes").value(payload);
        j.key("max_items").value(max_items);
        j.key("launches").begin_array();
        for (const Launch &l : launches) {
            const auto peers = list(l.partition->get("peers"));
            j.begin_object();
            j.key("backend").value(l.partition->get("backend"));
            j.key("peers").begin_array();
            for (const auto &peer : peers)
                j.value(to_integer(peer));
            j.end_array();
            j.key("lanes").value(l.lanes);
            j.key("slices").begin_array();
            long long previous = 0;
            for (long long lane = 1; lane <= l.lanes; ++lane) {
                // quotient / remainder split: no max_items * lane overflow
                const long long boundary = (max_items / l.lanes) * lane + ((max_items % l.lanes) * lane) / l.lanes;
                j.begin_array().value(previous).value(boundary).end_array();
                previous = boundary;
            }
            j.end_array();
            j.key("slice_quotient").value(max_items / l.lanes);
            j.key("slice_remainder").value(max_items % l.lanes);
            j.key("count_lane").value(0);
            const long long slots = ranked ? num(work, "rank_count") * ready_stride
                                           : static_cast<long long>(peers.size()) * l.lanes;
            j.key("signal_slots").value(slots);
            j.key("sender_grid").begin_array().value(static_cast<long long>(peers.size())).value(l.lanes).end_array();
            j.key("receiver_grid").begin_array().value(static_cast<long long>(peers.size()))
                .value(l.lanes / l.receiver_lanes).end_array();
            j.key("receiver_lanes_per_program").value(l.receiver_lanes);
            j.key("sender_warps").value(l.sender_warps);
            j.key("receiver_warps").value(1);
            j.key("profile_identity").value(l.identity);
            j.key("ready_stride").value(ready_stride);
            j.end_object();
        }
        j.end_array();
        j.end_object();
    }
    j.end_array();
}

// ---- plan-storage -----------------------------------------------------------------------------

void plan_storage(const Program &p, Json &j) {
    const bool enabled = switches(p).count("plan-storage") != 0;
    j.key("regions").begin_array();
    for (const Op &region : p.body) {
        if (region.kind != "region")
            continue;
        const long long declared = num(region, "rows");
        long long reached = 0;
        bool written = false, all_prefix = true, any_read = false;
        std::string last_reader;
        for (const Op &access : region.body) {
            // rows=<begin>:<end>, end exclusive; through=<view rows> bounds an indexed view
            const std::string rows = access.get("rows", "0:" + std::to_string(declared));
            const std::size_t colon = rows.find(':');
            long long end = quantity(rows.substr(colon + 1));
            if (access.has("through"))
                end = std::min(end, num(access, "through"));
            reached = std::max(reached, std::min(end, declared));
            if (access.get("kind") == "write") {
                written = true;
            } else {
                any_read = true;
                last_reader = access.get("stage");
                all_prefix = all_prefix && num(access, "prefix", 0) != 0;
            }
        }
        const bool escapes = num(region, "escapes", 0) != 0;
        if (escapes || region.body.empty())
            reached = declared;
        const long long physical = enabled ? reached : declared;
        // An immutable input whose every reader stays inside the valid prefix can be
        // borrowed from the caller in place instead of being copied.
        const bool prefix_binding = enabled && num(region, "immutable", 0) != 0 &&
                                    region.has("valid_count") && !written && any_read && all_prefix;
        j.begin_object();
        j.key("name").value(region.get("name"));
        j.key("declared_rows").value(declared);
        j.key("reached_rows").value(reached);
        j.key("physical_rows").value(physical);
        j.key("row_bytes").value(num(region, "row_bytes", 0));
        j.key("bytes").value(physical * num(region, "row_bytes", 0));
        j.key("last_reader").value(last_reader);
        j.key("event_ordered").value(num(region, "event_ordered", 0) != 0);
        j.key("max_inflight").value(num(region, "max_inflight", 1));
        j.key("prefix_binding").value(prefix_binding);
        j.key("allocated").value(physical > 0);
        j.end_object();
    }
    j.end_array();
}

// ---- plan-transport ---------------------------------------------------------------------------

std::string hex(const void *data, std::size_t bytes) {
    static const char *digits = "0123456789abcdef";
    std::string out;
    const auto *b = static_cast<const unsigned char *>(data);
    for (std::size_t i = 0; i < bytes; ++i) {
        out += digits[b[i] >> 4];
        out += digits[b[i] & 15];
    }
    return out;
}

void plan_transport(const Program &p, Json &j) {
    using namespace aboleth::abi;
    // Launch partitions: peers grouped by transport, in first-seen order.
    std::vector<std::pair<std::string, std::vector<long long>>> partitions;
    for (const Op &op : p.body) {
        if (op.kind != "peer")
            continue;
        const std::string backend = op.get("backend");
        if (lookup_transport_caps(backend.c_str()) == nullptr)
            throw Error("unknown transport '" + backend + "'");
        auto it = std::find_if(partitions.begin(), partitions.end(),
                               [&](const auto &entry) { return entry.first == backend; });
        if (it == partitions.end()) {
            partitions.emplace_back(backend, std::vector<long long>{});
            it = partitions.end() - 1;
        }
        it->second.push_back(num(op, "rank"));
    }
    j.key("launch_partitions").begin_array();
    bool any_queue = false, any_p2p = false;
    for (const auto &part : partitions) {
        j.begin_object();
        j.key("backend").value(part.first);
        j.key("peers").begin_array();
        for (long long peer : part.second)
            j.value(peer);
        j.end_array();
        j.end_object();
        (lookup_transport_caps(part.first.c_str())->load_store_addressable ? any_p2p : any_queue) = true;
    }
    j.end_array();
    const TransportTopologyKind topology = any_queue && any_p2p ? TransportTopologyKind::Mixed
                                           : any_p2p ? TransportTopologyKind::AllP2P
                                                     : TransportTopologyKind::AllNIC;
    j.key("topology").value(topology == TransportTopologyKind::Mixed ? "mixed"
                            : topology == TransportTopologyKind::AllP2P ? "all_p2p" : "all_nic");
    static const char *mode_names[] = {"SameQueueStrong", "P2PRelease", "GinSignal",
                                       "FenceThenSignal", "ImmCounting", "SameQueueFencedWrite"};
    static const std::map<std::string, unsigned> phase_ids = {
        {"dispatch", 0}, {"experts", 1}, {"combine", 2}, {"next_pack", 3}};
    j.key("phases").begin_array();
    for (const Op &phase : p.body) {
        if (phase.kind != "phase")
            continue;
        const std::string backend = phase.get("backend", partitions.empty() ? "p2p" : partitions[0].first);
        const TransportCaps *caps = lookup_transport_caps(backend.c_str());
        if (caps == nullptr)
            throw Error("unknown transport '" + backend + "'");
        // Reuse distance: iterations until the phase's source storage is written again.
        const long long slots = std::max(num(phase, "buffer_slots", 1), 1LL);
        const long long reuse = std::max(num(phase, "reuse", slots), 1LL);
        const long long commands = std::max(num(phase, "commands", 1), 1LL);
        const long long capacity = num(phase, "queue_capacity", 0);
        const bool optimistic_inline = num(phase, "optimistic_inline_window", 0) != 0;
        if (optimistic_inline)
            throw Error("phase " + phase.get("name") + ": an optimistic inline window is refused; "
                        "inline payloads count against the queue like any command");
        long long interval = reuse;
        if (caps->default_completion_interval)
            interval = std::min<long long>(interval, caps->default_completion_interval);
        if (phase.has("policy_interval"))
            interval = std::min(interval, std::max(num(phase, "policy_interval"), 1LL));
        if (caps->queue_capacity_limited && capacity > 1)
            interval = std::min(interval, std::max((capacity - 1) / commands, 1LL));
        interval = floor_pow2(interval);
        if (caps->load_store_addressable)
            interval = 0;  // nothing to retire: the whole phase completes by program order
        const bool defers = interval > 1;
        const TransportPublicationMode mode = legal_strong_publication(
            *caps, num(phase, "prefer_imm", 0) != 0, num(phase, "strict_registrations", 0) != 0);
        TransportPhasePlan plan{};
        plan.abi_version = kTransportPhasePlanVersion;
        plan.byte_size = sizeof(TransportPhasePlan);
        plan.active_qps = static_cast<std::uint32_t>(num(phase, "lanes", 1));
        plan.data_qps = plan.active_qps;
        plan.data_wqe_bound = static_cast<std::uint32_t>(commands * std::max(interval, 1LL));
        plan.data_reclaim_interval = static_cast<std::uint32_t>(interval);
        plan.topology_kind = static_cast<std::uint32_t>(topology);
        plan.publication_mode = static_cast<std::uint32_t>(mode);
        plan.prologue_barrier_kind = static_cast<std::uint32_t>(TransportBarrierKind::None);
        plan.epilogue_barrier_kind = static_cast<std::uint32_t>(
            caps->load_store_addressable ? TransportBarrierKind::NativeP2P : TransportBarrierKind::Transport);
        plan.flags = kTransportPlanReuseSafe | (defers ? kTransportPlanDrainAtEpilogue : 0u) |
                     (num(phase, "exclusive", 0) ? kTransportPlanQpExclusive : 0u);
        auto phase_id = [&](const std::string &key) {
            auto it = phase_ids.find(phase.get(key));
            return it == phase_ids.end() ? kTransportNoPhase : it->second;
        };
        plan.publication_before_phase = phase_id("publication_before");
        plan.publication_iteration_delta = static_cast<std::uint32_t>(num(phase, "publication_delta", 0));
        plan.completion_before_phase = phase_id("completion_before");
        plan.completion_iteration_delta = static_cast<std::uint32_t>(num(phase, "completion_delta", reuse - 1));
        plan.first_overwrite_phase = phase_id("first_overwrite");
        plan.first_overwrite_iteration_delta = static_cast<std::uint32_t>(reuse);
        plan.reclaim_before_phase = plan.completion_before_phase;
        plan.reclaim_iteration_delta = plan.completion_iteration_delta;
        plan.payload_bytes = static_cast<std::uint32_t>(num(phase, "payload_bytes", 0));
        plan.path_mtu = caps->path_mtu;
        plan.completion_interval = static_cast<std::uint32_t>(interval);
        plan.buffer_slots = static_cast<std::uint32_t>(slots);
        j.begin_object();
        j.key("name").value(phase.get("name"));
        j.key("backend").value(backend);
        j.key("reuse_distance").value(reuse);
        j.key("completion_interval").value(interval);
        j.key("publication_mode").value(mode_names[static_cast<int>(mode)]);
        j.key("checked_publication").value(publication_is_checked(*caps));
        j.key("requires_final_drain").value(defers);
        j.key("output_pool_depth").value(slots);
        j.key("completion_before").value(phase.get("completion_before", ""));
        j.key("plan_blob").value(hex(&plan, sizeof(plan)));
        j.end_object();
    }
    j.end_array();
}

// ---- plan-transport-program ---------------------------------------------------------------------
//
// An ordered list of phases (transfers) and kernels with the memory each one reads and
// writes.  An access is an arithmetic walk over one allocation:
//   allocation, generation, offset, length, stride, period, count [, unknown]
// iteration i touches [offset + (i*stride mod period), +length).  From the overlaps the
// planner derives, per phase: how many iterations pass before the source is touched again
// (reuse distance), the completion interval that lifetime, the queue and the policy allow,
// the first later operation that overwrites the source (completion deadline) and the first
// that reads the destination (publication deadline), wrapping once when the program is
// cyclic; per kernel: who consumes its output last, who overwrites it first, and whether the
// output buffer may be pooled.  (reference: compiler/lib/Transforms/PlanTransport.cpp:61-198
// for the walk, 203-316 for the interval, 318-422 deadlines, 424-563 output lifetimes.)

struct Walk {
    long long allocation = 0, generation = 0, offset = 0, length = 0, stride = 0, period = 0, count = 1;
    bool unknown = false;
};

bool interval_at(const Walk &w, long long iteration, long long &begin, long long &end) {
    if (w.unknown || iteration < 0 || iteration >= w.count)
        return false;
    // Checked arithmetic: a walk whose addresses leave 64 bits touches nothing we can reason about.
    long long displacement;
    if (__builtin_mul_overflow(iteration, w.stride, &displacement))
        return false;
    if (w.period > 0)
        displacement %= w.period;
    if (__builtin_add_overflow(w.offset, displacement, &begin) || __builtin_add_overflow(begin, w.length, &end))
        return false;
    return true;
}

bool walks_overlap_at(const Walk &a, long long ia, const Walk &b, long long ib) {
    if (a.unknown || b.unknown)
        return true;
    if (a.allocation != b.allocation || a.generation != b.generation)
        return false;
    long long a0, a1, b0, b1;
    if (!interval_at(a, ia, a0, a1) || !interval_at(b, ib, b0, b1))
        return true;  // cannot be bounded: assume they meet
    return a0 < b1 && b0 < a1;
}

bool any_overlap(const std::vector<Walk> &first, const std::vector<Walk> &second) {
    for (const Walk &a : first)
        for (const Walk &b : second)
            for (long long i = 0; i < std::max(a.count, 1LL); ++i)
                for (long long k = 0; k < std::max(b.count, 1LL); ++k)
                    if (walks_overlap_at(a, i, b, k))
                        return true;
    return false;
}

struct Step {
    const Op *op;
    bool is_phase;
    std::string name;
    std::vector<Walk> reads, writes;
    bool unknown_access = false;
};

Step read_step(const Op &op) {
    Step s{&op, op.kind == "phase", op.get("name"), {}, {}, false};
    if (s.name.empty())
        throw Error(op.kind + " needs a name");
    for (const Op &access : op.body) {
        if (access.kind != "read" && access.kind != "write")
            throw Error(op.kind + " " + s.name + ": unknown access '" + access.kind + "'");
        Walk w;
        w.allocation = num(access, "allocation");
        w.generation = num(access, "generation");
        w.offset = num(access, "offset");
        w.length = num(access, "length");
        w.stride = num(access, "stride");
        w.period = num(access, "period");
        w.count = num(access, "count", 1);
        w.unknown = num(access, "unknown", 0) != 0;
        if (w.length < 0 || w.count < 1 || w.period < 0)
            throw Error(op.kind + " " + s.name + ": access needs length >= 0, count >= 1, period >= 0");
        if (w.count > kLargestWalk)  // overlaps are found by enumerating pairs of iterations
            throw Error(op.kind + " " + s.name + ": an access of more than " + std::to_string(kLargestWalk) +
                        " iterations is not enumerated; mark it unknown=1");
        s.unknown_access = s.unknown_access || w.unknown;
        (access.kind == "read" ? s.reads : s.writes).push_back(w);
    }
    return s;
}

void plan_transport_program(const Program &p, Json &j) {
    using namespace aboleth::abi;
    const bool cyclic = to_integer(p.get("cyclic", "0")) != 0;
    std::vector<Step> steps;
    for (const Op &op : p.body)
        if (op.kind == "phase" || op.kind == "kernel")
            steps.push_back(read_step(op));
    for (std::size_t i = 0; i < steps.size(); ++i)
        for (std::size_t k = i + 1; k < steps.size(); ++k)
            if (steps[i].name == steps[k].name)
                throw Error("operation name '" + steps[i].name + "' is used twice");

    // First operation after `index` (wrapping once when cyclic) for which `test` holds.
    auto first_after = [&](std::size_t index, auto test, std::string &name, long long &delta) {
        name = "program_end";
        delta = 0;
        for (std::size_t k = index + 1; k < steps.size(); ++k)
            if (test(steps[k])) {
                name = steps[k].name;
                return;
            }
        if (!cyclic)
            return;
        for (std::size_t k = 0; k <= index; ++k)
            if (test(steps[k])) {
                name = steps[k].name;
                delta = 1;
                return;
            }
    };

    j.key("cyclic").value(cyclic);
    j.key("phases").begin_array();
    for (std::size_t index = 0; index < steps.size(); ++index) {
        const Step &s = steps[index];
        if (!s.is_phase)
            continue;
        const Op &phase = *s.op;
        const long long commands = num(phase, "commands", 1), iterations = num(phase, "iterations", 1),
                        payload = num(phase, "payload_bytes", 0);
        if (commands <= 0 || iterations <= 0 || payload < 0 || iterations > kLargestWalk)
            throw Error("phase " + s.name + " has invalid transport planning facts");
        // Reuse distance: the smallest d such that iteration i and i + d touch the same source bytes.
        long long reuse = s.reads.empty() ? 1 : iterations;
        for (const Walk &read : s.reads) {
            if (read.count != iterations)
                throw Error("phase " + s.name + ": read effect count must equal iterations");
            long long mine = iterations;
            for (long long d = 1; d < iterations && mine == iterations; ++d)
                for (long long i = 0; i + d < iterations; ++i)
                    if (walks_overlap_at(read, i, read, i + d)) {
                        mine = d;
                        break;
                    }
            reuse = std::min(reuse, mine);
        }
        const std::vector<std::string> transports = list(phase.get("transports"));
        const std::vector<std::string> capacities = list(phase.get("capacities"));
        const std::vector<std::string> peer_intervals = list(phase.get("intervals"));
        if (transports.size() != capacities.size())
            throw Error("phase " + s.name + " requires one endpoint capacity per peer transport");
        if (!peer_intervals.empty() && peer_intervals.size() != transports.size())
            throw Error("phase " + s.name + " requires one completion interval per peer transport");
        const bool explicit_interval = phase.has("interval");
        const long long tiny = num(phase, "tiny", 4096);
        long long policy = iterations, capacity_limit = iterations;
        bool queued = false;
        for (std::size_t t = 0; t < transports.size(); ++t) {
            const TransportCaps *caps = lookup_transport_caps(transports[t].c_str());
            if (caps == nullptr)
                throw Error("unknown peer transport '" + transports[t] + "'");
            if (!explicit_interval) {
                const long long configured = peer_intervals.empty() ? 0 : quantity(peer_intervals[t]);
                const long long preferred =
                    configured > 0 ? configured
                    : (payload <= tiny || caps->load_store_addressable) ? iterations
                    : caps->default_completion_interval > 0
                        ? static_cast<long long>(caps->default_completion_interval) : iterations;
                policy = std::min(policy, std::min(preferred, iterations));
            }
            if (caps->queue_capacity_limited) {
                queued = true;
                const long long capacity = quantity(capacities[t]);
                if (capacity < commands)
                    throw Error("phase " + s.name + ": endpoint capacity cannot hold one iteration");
                capacity_limit = std::min(capacity_limit,
                                          std::min(std::max(1LL, (capacity - 1) / commands), iterations));
            }
        }
        const long long legal = std::min(reuse, capacity_limit);
        long long interval;
        if (explicit_interval) {
            interval = num(phase, "interval");
            if (interval < 1 || interval > legal)
                throw Error("phase " + s.name + ": explicit completion interval exceeds region lifetime "
                            "or endpoint capacity");
        } else {
            if (transports.empty())
                throw Error("phase " + s.name + ": automatic completion planning requires endpoint capabilities");
            interval = std::min(legal, policy);
        }
        std::string completion_before, publication_before;
        long long completion_delta = 0, publication_delta = 0;
        first_after(index, [&](const Step &later) { return any_overlap(s.reads, later.writes); },
                    completion_before, completion_delta);
        first_after(index, [&](const Step &later) { return any_overlap(later.reads, s.writes); },
                    publication_before, publication_delta);
        j.begin_object();
        j.key("name").value(s.name);
        j.key("resolvedCompletionInterval").value(interval);
        j.key("reuseDistance").value(reuse);
        j.key("completionBefore").value(completion_before);
        j.key("completionIterationDelta").value(completion_delta);
        j.key("publicationBefore").value(publication_before);
        j.key("publicationIterationDelta").value(publication_delta);
        j.key("requiresFinalDrain").value(queued && interval > 1);
        j.end_object();
    }
    j.end_array();

    j.key("kernels").begin_array();
    for (std::size_t index = 0; index < steps.size(); ++index) {
        const Step &s = steps[index];
        if (s.is_phase)
            continue;
        const Op &kernel = *s.op;
        j.begin_object();
        j.key("name").value(s.name);
        j.key("opaque").value(num(kernel, "opaque", 0) != 0);
        bool reusable = false;
        std::string last_consumer = "none", reuse_before = "program_end";
        long long consumer_delta = 0, reuse_delta = 0;
        if (!s.writes.empty() && !s.unknown_access) {
            bool unknown_interference = false;
            auto inspect = [&](const Step &later, long long delta) {
                if (later.unknown_access) {
                    unknown_interference = true;
                    return;
                }
                if (any_overlap(later.reads, s.writes)) {
                    last_consumer = later.name;
                    consumer_delta = delta;
                }
                if (any_overlap(s.writes, later.writes)) {
                    reuse_before = later.name;
                    reuse_delta = delta;
                }
            };
            for (std::size_t k = index + 1; k < steps.size() && reuse_before == "program_end"; ++k)
                inspect(steps[k], 0);
            if (reuse_before == "program_end" && cyclic)
                for (std::size_t k = 0; k <= index && reuse_before == "program_end"; ++k)
                    inspect(steps[k], 1);
            const bool asynchronous = num(kernel, "asynchronous", 0) != 0;
            const bool async_ok = !asynchronous || num(kernel, "event_ordered", 0) != 0;
            reusable = !unknown_interference && async_ok && last_consumer != "none" &&
                       reuse_before != "program_end" && consumer_delta <= reuse_delta;
            if (reusable) {
                j.key("outputLastConsumer").value(last_consumer);
                j.key("outputLastConsumerIterationDelta").value(consumer_delta);
                j.key("outputReuseBefore").value(reuse_before);
                j.key("outputReuseIterationDelta").value(reuse_delta);
                j.key("outputPoolDepth").value(asynchronous ? std::max(num(kernel, "max_inflight", 1), 1LL) : 1LL);
            }
        }
        j.key("outputReusable").value(reusable);
        j.end_object();
    }
    j.end_array();
}

// ---- simplify-communication-dataflow --------------------------------------------------------------

void simplify_dataflow(const Program &p, Json &j) {
    const auto on = switches(p);
    const bool dead = on.count("dead-communication") != 0;
    const bool storage = on.count("plan-storage") != 0;
    struct Region {
        bool escapes = false, registered = false, donated = false, immutable = false;
    };
    std::map<std::string, Region> regions;
    struct Node {
        Op op;
        bool alive = true;
        std::string note;
    };
    std::vector<Node> nodes;
    for (const Op &op : p.body) {
        if (op.kind == "region") {
            Region r;
            r.escapes = num(op, "escapes", 0) != 0;
            r.registered = num(op, "registered", 0) != 0;
            r.donated = num(op, "donated", 0) != 0;
            r.immutable = num(op, "immutable", 0) != 0;
            regions[op.get("name")] = r;
        } else {
            nodes.push_back({op, true, ""});
        }
    }
    std::vector<std::pair<std::string, std::string>> rewrites;
    // 1. A reduction over a single source is a transfer.
    for (Node &n : nodes)
        if (n.op.kind == "reduction" && list(n.op.get("src")).size() == 1) {
            n.op.kind = "transfer";
            rewrites.emplace_back(n.op.get("name"), "singleton reduction became a transfer");
        }
    // 2. Forward a producer into a donated, registered final destination: the copy
    //    (or the staging output of an opaque stage) disappears and the producer
    //    writes the destination directly.
    if (storage) {
        for (Node &copy : nodes) {
            if (!copy.alive || copy.op.kind != "copy")
                continue;
            const Region &dst = regions[copy.op.get("dst")];
            if (!dst.donated || !dst.registered)
                continue;
            const std::string staging = copy.op.get("src");
            int readers = 0;
            Node *producer = nullptr;
            for (Node &other : nodes) {
                if (!other.alive || &other == &copy)
                    continue;
                for (const auto &src : list(other.op.get("src")))
                    readers += src == staging;
                for (const auto &src : list(other.op.get("reads")))
                    readers += src == staging;
                if (other.op.get("dst") == staging || other.op.get("writes") == staging)
                    producer = &other;
            }
            const bool bindable = producer != nullptr &&
                                  (producer->op.kind != "opaque_stage" || num(producer->op, "bindable_outputs", 0));
            if (readers != 0 || !bindable || regions[staging].escapes)
                continue;
            producer->op.attrs[producer->op.has("writes") ? "writes" : "dst"] = copy.op.get("dst");
            copy.alive = false;
            copy.note = "forwarded into donated destination " + copy.op.get("dst");
            rewrites.emplace_back(copy.op.get("name"), copy.note);
        }
    }
    // 3. A copy of an immutable region is an alias.
    std::map<std::string, std::string> aliases;
    for (Node &copy : nodes)
        if (copy.alive && copy.op.kind == "copy" && regions[copy.op.get("src")].immutable &&
            !regions[copy.op.get("dst")].escapes && storage) {
            aliases[copy.op.get("dst")] = copy.op.get("src");
            copy.alive = false;
            copy.note = "immutable copy aliased";
            rewrites.emplace_back(copy.op.get("name"), copy.note);
        }
    // 4. Dead communication: drop transfers/copies whose destination nobody observes,
    //    to a fixed point.
    bool changed = dead;
    while (changed) {
        changed = false;
        for (Node &n : nodes) {
            if (!n.alive || !(n.op.kind == "transfer" || n.op.kind == "copy" || n.op.kind == "reduction" ||
                              n.op.kind == "transform"))
                continue;
            const std::string dst = n.op.get("dst");
            if (regions[dst].escapes)
                continue;
            bool observed = false;
            for (const Node &other : nodes) {
                if (!other.alive || &other == &n)
                    continue;
                for (const char *key : {"src", "reads"})
                    for (const auto &name : list(other.op.get(key))) {
                        auto it = aliases.find(name);
                        observed = observed || name == dst || (it != aliases.end() && it->second == dst);
                    }
            }
            if (!observed) {
                n.alive = false;
                n.note = "dead: nothing reads " + dst;
                rewrites.emplace_back(n.op.get("name"), n.note);
                changed = true;
            }
        }
    }
    std::set<std::string> live_regions;
    for (const Node &n : nodes)
        if (n.alive)
            for (const char *key : {"src", "dst", "reads", "writes"})
                for (const auto &name : list(n.op.get(key)))
                    live_regions.insert(name);
    j.key("operations").begin_array();
    for (const Node &n : nodes)
        if (n.alive) {
            j.begin_object();
            j.key("kind").value(n.op.kind);
            for (const auto &kv : n.op.attrs)
                j.key(kv.first).value(kv.second);
            j.end_object();
        }
    j.end_array();
    j.key("removed").begin_array();
    for (const auto &r : rewrites)
        j.begin_object().key("name").value(r.first).key("why").value(r.second).end_object();
    j.end_array();
    j.key("aliases").begin_object();
    for (const auto &kv : aliases)
        j.key(kv.first).value(kv.second);
    j.end_object();
    j.key("unallocated_regions").begin_array();
    for (const auto &kv : regions)
        if (!live_regions.count(kv.first) && !kv.second.escapes)
            j.value(kv.first);
    j.end_array();
}

}  // namespace

std::string run_planner(const std::string &kind, const std::string &request) {
    const Program program = parse(request);
    Json j;
    j.begin_object();
    j.key("ok").value(true);
    j.key("planner").value(kind);
    if (kind == "plan-shapes")
        plan_shapes(program, j);
    else if (kind == "plan-endpoints")
        plan_endpoints(program, j);
    else if (kind == "plan-storage")
        plan_storage(program, j);
    else if (kind == "plan-transport")
        plan_transport(program, j);
    else if (kind == "plan-transport-program")
        plan_transport_program(program, j);
    else if (kind == "simplify-dataflow")
        simplify_dataflow(program, j);
    else
        throw Error("unknown planner '" + kind + "'");
    j.end_object();
    return j.str();
}

}  // namespace spec
