// Expert-parallel dispatch and combine as two launches per MoE layer.
//
// DISPATCH (one launch): each CTA takes tokens round-robin.  For one token it
// runs the router (softmax + top-k in one warp, or takes given ids/weights),
// reserves one slot per destination rank that owns at least one chosen expert
// (rank-deduplicated records, reference python/aboleth/moe/kernels.py:43-70),
// quantises the row to e4m3 with one fp32 scale per `scale_group` columns, and
// stores the payload row and the metadata row STRAIGHT into every destination
// rank's receive segment over NVLink - there is no send staging buffer and no
// separate put kernel.  The last CTA to finish writes each peer's record count
// and publishes with ONE `st.release.sys` per peer.  The same CTAs then turn
// receiver: they wait (bounded) for every peer's flag and unpack the records
// that arrived (expert ids, gate weights, per-expert positions, scales).
//
// COMBINE (one launch): for every record it received, a CTA forms
// sum_j gate_j * expert_out[j] in fp32 (the gate-weighted reduction happens
// here, not on the expert side), rounds to bf16 and stores the partial row
// into the source rank's return segment; one release flag per peer; then the
// CTAs wait for the peers' flags and sum each token's partials over ranks.
//
// The reference runs this as >= 9 launches (pack, three self copies, send,
// await, unpack, send, await, gather: python/aboleth/moe/native.py:433-615).
//
// Sender work never waits on a peer, so the two halves can also be launched
// separately (`phases` mask); that is how a single GPU emulates several ranks.
#include "moe_common.cuh"

namespace {

using namespace ab::moe;
using aboleth::Status;

constexpr int kThreads = 256;
constexpr int kPhaseSend = 1;
constexpr int kPhaseRecv = 2;

struct EpGeometry {
    int rank, world, experts, top_k, hidden, scale_group, capacity;
    int value_fp8, round_scale, placeholder_expert;
    float amax_floor;
};

struct DispatchParams {
    EpGeometry g;
    int num_tokens, routing, renormalize, phases;
    int by_warp;                   // 1: one warp per token (throughput), 0: one CTA per token (latency)
    const std::uint32_t *x;        // [T, hidden] bf16
    const float *logits;           // [T, experts]       (routing == 1)
    const int *ids_in;             // [T, k]             (routing == 0)
    const float *weights_in;       // [T, k]
    int *ids_out;                  // optional [T, k]
    float *weights_out;            // optional [T, k]
    const int *owners;             // [experts] -> rank
    // sender state (local)
    int *source_slots;             // [capacity, world]
    unsigned long long *send_counts;  // [world]
    unsigned *done;                // [4] phase counters
    int *overflow;                 // [1]
    const unsigned long long *epoch;  // device epoch (starts at 1)
    unsigned long long *status;    // [2]
    // peers (device arrays of addresses, [world])
    const std::uint64_t *peer_payload, *peer_meta, *peer_counts, *peer_flags;
    // receiver side (local)
    const int *recv_meta;
    const unsigned long long *recv_counts;  // [world]
    const std::uint64_t *flags;             // [world]
    int *expert_ids;               // [world*capacity, k]
    float *expert_weights;         // [world*capacity, k]
    int *expert_pos;               // [world*capacity, k]
    int *expert_counts;            // [experts]
    float *expert_scales;          // [world*capacity, cols]   (fp8 only)
    unsigned long long *trace;     // optional [8]: %globaltimer stamps of CTA 0 and of the last CTA
};

__device__ __forceinline__ int meta_words(const EpGeometry &g) {
    return 2 + 2 * g.top_k + (g.value_fp8 ? g.hidden / g.scale_group : 0);
}

// Phase stamps for the tracing buffer: slot i <- %globaltimer (ns).
__device__ __forceinline__ void stamp(unsigned long long *trace, int slot, bool who) {
    if (trace != nullptr && who)
        trace[slot] = aboleth::detail::globaltimer_ns();
}

// Thread 0 of every CTA calls this after a CTA barrier.  Returns true in the
// CTA that arrived last; that CTA has then acquired every other CTA's stores.
__device__ __forceinline__ bool arrive_last(unsigned *counter) {
    aboleth::detail::fence_acq_rel_sys();
    const unsigned old = atomicAdd(counter, 1u);
    if (old != gridDim.x - 1)
        return false;
    aboleth::detail::fence_acq_rel_sys();
    return true;
}

// All CTAs: wait until every peer published `epoch`.  Returns false on timeout.
__device__ __forceinline__ bool wait_all_peers(const std::uint64_t *flags, int world,
                                               std::uint64_t epoch, unsigned long long *status,
                                               int *s_fail, unsigned detail_base) {
    if (threadIdx.x == 0)
        *s_fail = 0;
    __syncthreads();
    if (threadIdx.x < world) {
        const Status s = aboleth::wait_signal_status(flags + threadIdx.x, epoch);
        if (s != Status::Ok) {
            ab::set_status(status, s, detail_base + threadIdx.x);
            *s_fail = 1;
        }
    }
    __syncthreads();
    return *s_fail == 0;
}

// Per-warp scratch of the warp-per-token path.
struct alignas(16) WarpScratch {
    int meta[2 + 2 * kMaxTopK + 128 + 2];
    float scale[128];
};

__device__ __forceinline__ std::uint64_t shfl_u64(std::uint64_t v, int src) {
    const unsigned lo = __shfl_sync(0xffffffffu, static_cast<unsigned>(v), src);
    const unsigned hi = __shfl_sync(0xffffffffu, static_cast<unsigned>(v >> 32), src);
    return (static_cast<std::uint64_t>(hi) << 32) | lo;
}

// One warp sends one token: route, reserve slots, quantise, store payload and
// metadata rows to every destination.  No CTA-level synchronisation.
__device__ __forceinline__ void send_token_by_warp(const DispatchParams &p, int t, WarpScratch &ws) {
    const EpGeometry &g = p.g;
    const int lane = threadIdx.x & 31;
    const int cols = g.value_fp8 ? g.hidden / g.scale_group : 0;
    const int words = meta_words(g);
    const int row_bytes = g.value_fp8 ? g.hidden : g.hidden * 2;

    int id = -1;
    float w = 0.f;
    if (p.routing == 1) {
        warp_softmax_topk(p.logits + static_cast<std::size_t>(t) * g.experts, g.experts, g.top_k,
                          p.renormalize, id, w);
    } else if (lane < g.top_k) {
        id = p.ids_in[t * g.top_k + lane];
        w = p.weights_in[t * g.top_k + lane];
    }
    const bool valid = lane < g.top_k && id >= 0 && id < g.experts;
    const int owner = valid ? p.owners[id] : -1;
    if (lane < g.top_k) {
        if (p.ids_out != nullptr)
            p.ids_out[t * g.top_k + lane] = id;
        if (p.weights_out != nullptr)
            p.weights_out[t * g.top_k + lane] = w;
    }
    // Lane d decides for destination rank d.
    int nsel = 0;
    for (int j = 0; j < g.top_k; ++j)
        nsel += __shfl_sync(0xffffffffu, owner, j) == lane;
    int slot = -1;
    std::uint64_t my_row = 0, my_meta = 0;
    if (lane < g.world) {
        if (nsel > 0) {
            const unsigned long long got = atomicAdd(p.send_counts + lane, 1ull);
            if (got < static_cast<unsigned long long>(g.capacity))
                slot = static_cast<int>(got);
            else
                *p.overflow = 1;
        }
        p.source_slots[t * g.world + lane] = slot;
        if (slot >= 0) {
            const std::size_t row = static_cast<std::size_t>(g.rank) * g.capacity + slot;
            my_row = p.peer_payload[lane] + row * row_bytes;
            my_meta = p.peer_meta[lane] + row * words * 4;
        }
    }
    const unsigned live = __ballot_sync(0xffffffffu, slot >= 0);

    // ---- payload: four 512-element steps (128 bytes per lane) in flight ----
    const std::uint32_t *xrow = p.x + static_cast<std::size_t>(t) * (g.hidden / 2);
    const int chunks = g.hidden / 16;
    const int lanes_per_group = g.scale_group / 16;
    constexpr int kDepth = 4;
    for (int base = 0; base < chunks; base += 32 * kDepth) {
        uint4 a[kDepth], b[kDepth];
#pragma unroll
        for (int u = 0; u < kDepth; ++u) {
            const int c = base + u * 32 + lane;
            a[u] = make_uint4(0, 0, 0, 0);
            b[u] = a[u];
            if (c < chunks) {
                a[u] = aboleth::detail::ld_stream16(xrow + c * 8);
                b[u] = aboleth::detail::ld_stream16(xrow + c * 8 + 4);
            }
        }
#pragma unroll
        for (int u = 0; u < kDepth; ++u) {
            const int c = base + u * 32 + lane;
            const bool ok = c < chunks;
            if (base + u * 32 >= chunks)
                break;
            if (g.value_fp8) {
                const float amax = group_max(amax16(a[u], b[u]), lanes_per_group);
                const float scale = quant_scale(amax, g.amax_floor, g.round_scale);
                const uint4 q = quant16(a[u], b[u], scale);
                if (ok && c % lanes_per_group == 0)
                    ws.scale[c / lanes_per_group] = scale;
                for (unsigned m = live; m; m &= m - 1) {
                    const std::uint64_t row = shfl_u64(my_row, __ffs(m) - 1);
                    if (ok)
                        aboleth::detail::st_stream16(reinterpret_cast<void *>(row + c * 16), q);
                }
            } else {
                for (unsigned m = live; m; m &= m - 1) {
                    const std::uint64_t row = shfl_u64(my_row, __ffs(m) - 1);
                    if (ok) {
                        aboleth::detail::st_stream16(reinterpret_cast<void *>(row + c * 32), a[u]);
                        aboleth::detail::st_stream16(reinterpret_cast<void *>(row + c * 32 + 16), b[u]);
                    }
                }
            }
        }
    }

    // ---- metadata rows ----
    __syncwarp();
    if (lane == 0)
        ws.meta[0] = t;
    for (int c = lane; c < cols; c += 32)
        ws.meta[2 + 2 * g.top_k + c] = __float_as_int(ws.scale[c]);
    for (unsigned m = live; m; m &= m - 1) {
        const int d = __ffs(m) - 1;
        const bool mine = lane < g.top_k && owner == d;
        const unsigned sel = __ballot_sync(0xffffffffu, mine);
        const int n = __popc(sel);
        if (lane == 0)
            ws.meta[1] = n;
        if (mine) {
            const int idx = __popc(sel & ((1u << lane) - 1));
            ws.meta[2 + idx] = id;
            ws.meta[2 + g.top_k + idx] = __float_as_int(w);
        }
        if (lane >= n && lane < g.top_k) {
            ws.meta[2 + lane] = -1;
            ws.meta[2 + g.top_k + lane] = 0;
        }
        __syncwarp();
        const std::uint64_t dst = shfl_u64(my_meta, d);
        if ((words & 1) == 0) {
            for (int i = lane; i < words / 2; i += 32)
                reinterpret_cast<std::uint64_t *>(dst)[i] =
                    reinterpret_cast<const std::uint64_t *>(ws.meta)[i];
        } else {
            for (int i = lane; i < words; i += 32)
                reinterpret_cast<int *>(dst)[i] = ws.meta[i];
        }
        __syncwarp();
    }
}

__global__ void __launch_bounds__(kThreads, 4) ep_dispatch_kernel(DispatchParams p) {
    const EpGeometry &g = p.g;
    __shared__ int s_id[kMaxTopK];
    __shared__ float s_w[kMaxTopK];
    __shared__ int s_owner[kMaxTopK];
    __shared__ int s_slot[kMaxWorld];
    __shared__ int s_dest[kMaxWorld];
    __shared__ int s_ndest;
    __shared__ float s_scale[128];  // hidden / scale_group <= 128
    __shared__ int s_flag;

    const int tid = threadIdx.x;
    const int lane = tid & 31;
    const int warp = tid >> 5;
    const std::uint64_t epoch = *p.epoch;
    const int cols = g.value_fp8 ? g.hidden / g.scale_group : 0;
    const int words = meta_words(g);
    const int row_bytes = g.value_fp8 ? g.hidden : g.hidden * 2;
    const bool tracer = blockIdx.x == 0 && tid == 0;
    stamp(p.trace, 0, tracer);

    if ((p.phases & kPhaseSend) && p.by_warp) {
        __shared__ WarpScratch scratch[kThreads / 32];
        const int warps = gridDim.x * (kThreads / 32);
        for (int t = blockIdx.x * (kThreads / 32) + warp; t < p.num_tokens; t += warps)
            send_token_by_warp(p, t, scratch[warp]);
    }
    if (p.phases & kPhaseSend) {
        for (int t = blockIdx.x; t < p.num_tokens && !p.by_warp; t += gridDim.x) {
            // ---- routing and slot reservation (warp 0) ----
            if (warp == 0) {
                int id = -1;
                float w = 0.f;
                if (p.routing == 1) {
                    warp_softmax_topk(p.logits + static_cast<std::size_t>(t) * g.experts,
                                      g.experts, g.top_k, p.renormalize, id, w);
                } else if (lane < g.top_k) {
                    id = p.ids_in[t * g.top_k + lane];
                    w = p.weights_in[t * g.top_k + lane];
                }
                const bool valid = lane < g.top_k && id >= 0 && id < g.experts;
                const int owner = valid ? p.owners[id] : -1;
                if (lane < g.top_k) {
                    s_id[lane] = id;
                    s_w[lane] = w;
                    s_owner[lane] = owner;
                    if (p.ids_out != nullptr)
                        p.ids_out[t * g.top_k + lane] = id;
                    if (p.weights_out != nullptr)
                        p.weights_out[t * g.top_k + lane] = w;
                }
                __syncwarp();
                int slot = -1, nsel = 0;
                if (lane < g.world) {
                    for (int j = 0; j < g.top_k; ++j)
                        nsel += s_owner[j] == lane;
                    if (nsel > 0) {
                        const unsigned long long got = atomicAdd(p.send_counts + lane, 1ull);
                        if (got < static_cast<unsigned long long>(g.capacity))
                            slot = static_cast<int>(got);
                        else
                            *p.overflow = 1;
                    }
                    p.source_slots[t * g.world + lane] = slot;
                    s_slot[lane] = slot;
                }
                const unsigned live = __ballot_sync(0xffffffffu, slot >= 0);
                if (slot >= 0)
                    s_dest[__popc(live & ((1u << lane) - 1))] = lane;
                if (lane == 0)
                    s_ndest = __popc(live);
            }
            __syncthreads();
            const int ndest = s_ndest;

            // ---- payload: quantise once, store to every destination ----
            const std::uint32_t *xrow = p.x + static_cast<std::size_t>(t) * (g.hidden / 2);
            const int chunks = g.hidden / 16;  // 16 elements per thread-step
            const int lanes_per_group = g.scale_group / 16;
            for (int base = 0; base < chunks; base += kThreads) {
                const int c = base + tid;
                const bool live = c < chunks;
                uint4 a = make_uint4(0, 0, 0, 0), b = a;
                if (live) {
                    a = aboleth::detail::ld_stream16(xrow + c * 8);
                    b = aboleth::detail::ld_stream16(xrow + c * 8 + 4);
                }
                if (g.value_fp8) {
                    const float amax = group_max(amax16(a, b), lanes_per_group);
                    const float scale = quant_scale(amax, g.amax_floor, g.round_scale);
                    if (live) {
                        const uint4 q = quant16(a, b, scale);
                        if (c % lanes_per_group == 0)
                            s_scale[c / lanes_per_group] = scale;
                        for (int i = 0; i < ndest; ++i) {
                            const int d = s_dest[i];
                            std::uint8_t *row = reinterpret_cast<std::uint8_t *>(p.peer_payload[d]) +
                                (static_cast<std::size_t>(g.rank) * g.capacity + s_slot[d]) * row_bytes;
                            aboleth::detail::st_stream16(row + c * 16, q);
                        }
                    }
                } else if (live) {
                    for (int i = 0; i < ndest; ++i) {
                        const int d = s_dest[i];
                        std::uint8_t *row = reinterpret_cast<std::uint8_t *>(p.peer_payload[d]) +
                            (static_cast<std::size_t>(g.rank) * g.capacity + s_slot[d]) * row_bytes;
                        aboleth::detail::st_stream16(row + c * 32, a);
                        aboleth::detail::st_stream16(row + c * 32 + 16, b);
                    }
                }
            }
            __syncthreads();

            // ---- metadata rows: one warp per destination ----
            for (int i = warp; i < ndest; i += kThreads / 32) {
                const int d = s_dest[i];
                int *meta = reinterpret_cast<int *>(p.peer_meta[d]) +
                    (static_cast<std::size_t>(g.rank) * g.capacity + s_slot[d]) * words;
                const bool mine = lane < g.top_k && s_owner[lane] == d;
                const unsigned sel = __ballot_sync(0xffffffffu, mine);
                const int nsel = __popc(sel);
                if (lane == 0) {
                    meta[0] = t;
                    meta[1] = nsel;
                }
                if (mine) {
                    const int idx = __popc(sel & ((1u << lane) - 1));
                    meta[2 + idx] = s_id[lane];
                    meta[2 + g.top_k + idx] = __float_as_int(s_w[lane]);
                }
                if (lane >= nsel && lane < g.top_k) {
                    meta[2 + lane] = -1;
                    meta[2 + g.top_k + lane] = 0;
                }
                for (int c = lane; c < cols; c += 32)
                    meta[2 + 2 * g.top_k + c] = __float_as_int(s_scale[c]);
            }
            __syncthreads();
        }

        // ---- publication: the last CTA writes counts and one flag per peer ----
        __syncthreads();
        stamp(p.trace, 1, tracer);
        if (tid == 0)
            s_flag = arrive_last(p.done + 0) ? 1 : 0;
        __syncthreads();
        stamp(p.trace, 2, tracer);
        stamp(p.trace, 5, s_flag && tid == 0);
        if (s_flag && tid < g.world) {
            const unsigned long long n = ab::min64(
                aboleth::detail::ld_relaxed_sys(reinterpret_cast<const std::uint64_t *>(p.send_counts + tid)),
                static_cast<std::uint64_t>(g.capacity));
            std::uint64_t *cnt = reinterpret_cast<std::uint64_t *>(p.peer_counts[tid]) + g.rank;
            std::uint64_t *flag = reinterpret_cast<std::uint64_t *>(p.peer_flags[tid]) + g.rank;
            aboleth::detail::st_relaxed_sys(cnt, n);
            aboleth::detail::st_release_sys(flag, epoch);
            p.send_counts[tid] = 0;
            if (tid == 0)
                p.done[0] = 0;
        }
    }

    if (p.phases & kPhaseRecv) {
        if (!wait_all_peers(p.flags, g.world, epoch, p.status, &s_flag, 0x1000))
            return;
        stamp(p.trace, 3, tracer);
        // One warp per received record.
        const int warps = gridDim.x * (kThreads / 32);
        const int total = g.world * g.capacity;
        for (int row = blockIdx.x * (kThreads / 32) + warp; row < total; row += warps) {
            const int src = row / g.capacity;
            const int slot = row - src * g.capacity;
            const unsigned long long count = p.recv_counts[src];
            if (count > static_cast<unsigned long long>(g.capacity)) {
                if (lane == 0 && slot == 0)
                    ab::set_status(p.status, Status::Malformed, 0x1100 + src);
                continue;
            }
            if (static_cast<unsigned long long>(slot) >= count)
                continue;
            const int *meta = p.recv_meta + static_cast<std::size_t>(row) * words;
            int nsel = meta[1];
            if (nsel < 1 || nsel > g.top_k) {
                if (lane == 0)
                    ab::set_status(p.status, Status::Malformed, 0x1200 + src);
                nsel = 0;
            }
            if (lane < g.top_k) {
                int id = g.placeholder_expert;
                float w = 0.f;
                int pos = -1;
                if (lane < nsel) {
                    id = meta[2 + lane];
                    w = __int_as_float(meta[2 + g.top_k + lane]);
                    if (id >= 0 && id < g.experts) {
                        pos = atomicAdd(p.expert_counts + id, 1);
                    } else {
                        id = g.placeholder_expert;
                        w = 0.f;
                    }
                }
                p.expert_ids[row * g.top_k + lane] = id;
                p.expert_weights[row * g.top_k + lane] = w;
                p.expert_pos[row * g.top_k + lane] = pos;
            }
            if (p.expert_scales != nullptr)
                for (int c = lane; c < cols; c += 32)
                    p.expert_scales[static_cast<std::size_t>(row) * cols + c] =
                        __int_as_float(meta[2 + 2 * g.top_k + c]);
        }
        stamp(p.trace, 4, tracer);
    }
}

struct CombineParams {
    EpGeometry g;
    int num_tokens, phases, weighted, by_warp;
    // expert side
    const std::uint32_t *expert_out;   // bf16 rows: weighted ? [pairs, hidden] : [world*capacity, hidden]
    const int *expert_ids, *expert_pos;
    const float *expert_weights;
    const int *expert_offsets;         // [experts] start row of each expert's group (weighted)
    const int *recv_meta;
    const unsigned long long *recv_counts;
    // transport
    const std::uint64_t *peer_return, *peer_return_flags;
    const std::uint64_t *return_flags;  // local [world]
    const std::uint32_t *returned;      // local [world*capacity, hidden] bf16
    // source side
    const int *source_slots;
    std::uint32_t *out;                 // [T, hidden] bf16
    unsigned *done;
    int *expert_counts;                 // zeroed at the end (self-cleaning)
    unsigned long long *epoch;
    unsigned long long *status;
    unsigned long long *trace;          // optional [8]
};

__device__ __forceinline__ void add_bf16x8(float (&acc)[8], const uint4 &y, float w) {
    acc[0] += w * bf16_lo(y.x); acc[1] += w * bf16_hi(y.x);
    acc[2] += w * bf16_lo(y.y); acc[3] += w * bf16_hi(y.y);
    acc[4] += w * bf16_lo(y.z); acc[5] += w * bf16_hi(y.z);
    acc[6] += w * bf16_lo(y.w); acc[7] += w * bf16_hi(y.w);
}

__device__ __forceinline__ uint4 pack_bf16x8(const float (&acc)[8]) {
    uint4 o;
    o.x = pack_bf16x2(acc[0], acc[1]);
    o.y = pack_bf16x2(acc[2], acc[3]);
    o.z = pack_bf16x2(acc[4], acc[5]);
    o.w = pack_bf16x2(acc[6], acc[7]);
    return o;
}

// One warp returns one received record to its source rank.
__device__ __forceinline__ void return_row_by_warp(const CombineParams &p, int row, int src, int slot) {
    const EpGeometry &g = p.g;
    const int lane = threadIdx.x & 31;
    const int vecs = g.hidden / 8;
    std::uint8_t *dst = reinterpret_cast<std::uint8_t *>(p.peer_return[src]) +
        (static_cast<std::size_t>(g.rank) * g.capacity + slot) * g.hidden * 2;
    if (!p.weighted) {
        const std::uint32_t *y = p.expert_out + static_cast<std::size_t>(row) * (g.hidden / 2);
        int v = lane;
        for (; v + 96 < vecs; v += 128) {
            const uint4 a = aboleth::detail::ld_stream16(y + v * 4);
            const uint4 b = aboleth::detail::ld_stream16(y + (v + 32) * 4);
            const uint4 c = aboleth::detail::ld_stream16(y + (v + 64) * 4);
            const uint4 d = aboleth::detail::ld_stream16(y + (v + 96) * 4);
            aboleth::detail::st_stream16(dst + v * 16, a);
            aboleth::detail::st_stream16(dst + (v + 32) * 16, b);
            aboleth::detail::st_stream16(dst + (v + 64) * 16, c);
            aboleth::detail::st_stream16(dst + (v + 96) * 16, d);
        }
        for (; v < vecs; v += 32)
            aboleth::detail::st_stream16(dst + v * 16, aboleth::detail::ld_stream16(y + v * 4));
        return;
    }
    int n = p.recv_meta[static_cast<std::size_t>(row) * meta_words(g) + 1];
    n = n < 0 ? 0 : (n > g.top_k ? g.top_k : n);
    int my_row = -1;
    float my_gate = 0.f;
    if (lane < n) {
        const int pos = p.expert_pos[row * g.top_k + lane];
        if (pos >= 0)
            my_row = p.expert_offsets[p.expert_ids[row * g.top_k + lane]] + pos;
        my_gate = p.expert_weights[row * g.top_k + lane];
    }
    for (int base = 0; base < vecs; base += 64) {
        float acc[2][8] = {};
        for (int j = 0; j < n; ++j) {
            const int r = __shfl_sync(0xffffffffu, my_row, j);
            const float w = __shfl_sync(0xffffffffu, my_gate, j);
            if (r < 0)
                continue;
            const std::uint32_t *y = p.expert_out + static_cast<std::size_t>(r) * (g.hidden / 2);
#pragma unroll
            for (int u = 0; u < 2; ++u) {
                const int v = base + u * 32 + lane;
                if (v < vecs)
                    add_bf16x8(acc[u], aboleth::detail::ld_stream16(y + v * 4), w);
            }
        }
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            const int v = base + u * 32 + lane;
            if (v < vecs)
                aboleth::detail::st_stream16(dst + v * 16, pack_bf16x8(acc[u]));
        }
    }
}

// One warp reduces one token's partial rows over the ranks that hold one.
__device__ __forceinline__ void reduce_token_by_warp(const CombineParams &p, int t) {
    const EpGeometry &g = p.g;
    const int lane = threadIdx.x & 31;
    const int vecs = g.hidden / 8;
    int slot = -1;
    if (lane < g.world)
        slot = p.source_slots[t * g.world + lane];
    const unsigned live = __ballot_sync(0xffffffffu, slot >= 0);
    const std::uint32_t *my_src = p.returned +
        (static_cast<std::size_t>(lane < g.world ? lane : 0) * g.capacity + (slot < 0 ? 0 : slot)) * (g.hidden / 2);
    std::uint32_t *out = p.out + static_cast<std::size_t>(t) * (g.hidden / 2);
    for (int base = 0; base < vecs; base += 64) {
        float acc[2][8] = {};
        for (unsigned m = live; m; m &= m - 1) {
            const std::uint32_t *y = reinterpret_cast<const std::uint32_t *>(
                shfl_u64(reinterpret_cast<std::uint64_t>(my_src), __ffs(m) - 1));
#pragma unroll
            for (int u = 0; u < 2; ++u) {
                const int v = base + u * 32 + lane;
                if (v < vecs)
                    add_bf16x8(acc[u], aboleth::detail::ld_stream16(y + v * 4), 1.0f);
            }
        }
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            const int v = base + u * 32 + lane;
            if (v < vecs)
                *reinterpret_cast<uint4 *>(out + v * 4) = pack_bf16x8(acc[u]);
        }
    }
}

__global__ void __launch_bounds__(kThreads) ep_combine_kernel(CombineParams p) {
    const EpGeometry &g = p.g;
    __shared__ int s_flag;
    __shared__ int s_rows[kMaxTopK];
    __shared__ float s_gate[kMaxTopK];
    const int tid = threadIdx.x;
    const std::uint64_t epoch = *p.epoch;
    const int vecs = g.hidden / 8;  // 16-byte vectors per bf16 row
    const int words = meta_words(g);
    const bool tracer = blockIdx.x == 0 && tid == 0;
    stamp(p.trace, 0, tracer);

    // Records are visited round-robin over the source ranks, starting at rank + 1: at any moment
    // the CTAs of one rank write to every peer, and no two ranks start on the same peer.  (Walking
    // source 0, then source 1, ... makes all ranks converge on one receiver at a time.)
    int most = 0;
    for (int src = 0; src < g.world; ++src)
        most = max(most, static_cast<int>(ab::min64(p.recv_counts[src], g.capacity)));
    const int spread = most * g.world;
    if ((p.phases & kPhaseSend) && p.by_warp) {
        const int warps = gridDim.x * (kThreads / 32);
        const int gw = blockIdx.x * (kThreads / 32) + (tid >> 5);
        for (int i = gw; i < spread; i += warps) {
            const int slot = i / g.world;
            const int src = (g.rank + 1 + (i - slot * g.world)) % g.world;
            if (static_cast<unsigned long long>(slot) < p.recv_counts[src])
                return_row_by_warp(p, src * g.capacity + slot, src, slot);
        }
    }
    if (p.phases & kPhaseSend) {
        const int total = p.by_warp ? 0 : spread;
        for (int i = blockIdx.x; i < total; i += gridDim.x) {
            const int slot = i / g.world;
            const int src = (g.rank + 1 + (i - slot * g.world)) % g.world;
            if (static_cast<unsigned long long>(slot) >= p.recv_counts[src])
                continue;  // the same for every thread of the CTA
            const int row = src * g.capacity + slot;
            int n = 1;
            if (p.weighted) {
                n = p.recv_meta[static_cast<std::size_t>(row) * words + 1];
                n = n < 0 ? 0 : (n > g.top_k ? g.top_k : n);
                if (tid < n) {
                    const int id = p.expert_ids[row * g.top_k + tid];
                    const int pos = p.expert_pos[row * g.top_k + tid];
                    s_rows[tid] = pos >= 0 ? p.expert_offsets[id] + pos : -1;
                    s_gate[tid] = p.expert_weights[row * g.top_k + tid];
                }
                __syncthreads();
            }
            std::uint8_t *dst = reinterpret_cast<std::uint8_t *>(p.peer_return[src]) +
                (static_cast<std::size_t>(g.rank) * g.capacity + slot) * g.hidden * 2;
            for (int v = tid; v < vecs; v += kThreads) {
                uint4 o;
                if (!p.weighted) {
                    o = aboleth::detail::ld_stream16(p.expert_out + static_cast<std::size_t>(row) * (g.hidden / 2) + v * 4);
                } else {
                    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
                    for (int j = 0; j < n; ++j) {
                        if (s_rows[j] < 0)
                            continue;
                        const uint4 y = aboleth::detail::ld_stream16(
                            p.expert_out + static_cast<std::size_t>(s_rows[j]) * (g.hidden / 2) + v * 4);
                        const float w = s_gate[j];
                        acc[0] += w * bf16_lo(y.x); acc[1] += w * bf16_hi(y.x);
                        acc[2] += w * bf16_lo(y.y); acc[3] += w * bf16_hi(y.y);
                        acc[4] += w * bf16_lo(y.z); acc[5] += w * bf16_hi(y.z);
                        acc[6] += w * bf16_lo(y.w); acc[7] += w * bf16_hi(y.w);
                    }
                    o.x = pack_bf16x2(acc[0], acc[1]);
                    o.y = pack_bf16x2(acc[2], acc[3]);
                    o.z = pack_bf16x2(acc[4], acc[5]);
                    o.w = pack_bf16x2(acc[6], acc[7]);
                }
                aboleth::detail::st_stream16(dst + v * 16, o);
            }
            if (p.weighted)
                __syncthreads();
        }
        __syncthreads();
        stamp(p.trace, 1, tracer);
        if (tid == 0)
            s_flag = arrive_last(p.done + 1) ? 1 : 0;
        __syncthreads();
        stamp(p.trace, 2, tracer);
        if (s_flag && tid < g.world) {
            std::uint64_t *flag = reinterpret_cast<std::uint64_t *>(p.peer_return_flags[tid]) + g.rank;
            aboleth::detail::st_release_sys(flag, epoch);
            if (tid == 0)
                p.done[1] = 0;
        }
    }

    if (p.phases & kPhaseRecv) {
        if (!wait_all_peers(p.return_flags, g.world, epoch, p.status, &s_flag, 0x2000))
            return;
        stamp(p.trace, 3, tracer);
        if (p.by_warp) {
            const int warps = gridDim.x * (kThreads / 32);
            for (int t = blockIdx.x * (kThreads / 32) + (tid >> 5); t < p.num_tokens; t += warps)
                reduce_token_by_warp(p, t);
        }
        for (int t = blockIdx.x; t < p.num_tokens && !p.by_warp; t += gridDim.x) {
            for (int v = tid; v < vecs; v += kThreads) {
                float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
                for (int d = 0; d < g.world; ++d) {
                    const int slot = p.source_slots[t * g.world + d];
                    if (slot < 0)
                        continue;
                    const uint4 y = aboleth::detail::ld_stream16(
                        p.returned + (static_cast<std::size_t>(d) * g.capacity + slot) * (g.hidden / 2) + v * 4);
                    acc[0] += bf16_lo(y.x); acc[1] += bf16_hi(y.x);
                    acc[2] += bf16_lo(y.y); acc[3] += bf16_hi(y.y);
                    acc[4] += bf16_lo(y.z); acc[5] += bf16_hi(y.z);
                    acc[6] += bf16_lo(y.w); acc[7] += bf16_hi(y.w);
                }
                uint4 o;
                o.x = pack_bf16x2(acc[0], acc[1]);
                o.y = pack_bf16x2(acc[2], acc[3]);
                o.z = pack_bf16x2(acc[4], acc[5]);
                o.w = pack_bf16x2(acc[6], acc[7]);
                *reinterpret_cast<uint4 *>(p.out + static_cast<std::size_t>(t) * (g.hidden / 2) + v * 4) = o;
            }
        }
        // Close the layer: the last CTA clears the expert counters and
        // advances the epoch for the next dispatch.
        __syncthreads();
        stamp(p.trace, 4, tracer);
        if (tid == 0)
            s_flag = arrive_last(p.done + 2) ? 1 : 0;
        __syncthreads();
        if (s_flag) {
            for (int e = tid; e < g.experts; e += kThreads)
                p.expert_counts[e] = 0;
            if (tid == 0) {
                p.done[2] = 0;
                *p.epoch = epoch + 1;
            }
        }
    }
}

// ---- standalone pieces ------------------------------------------------------------

// x [rows, hidden] bf16 -> q [rows, hidden] e4m3, scales [rows, hidden/group] fp32.
__global__ void __launch_bounds__(kThreads) quant_fp8_kernel(
    const std::uint32_t *x, std::uint8_t *q, float *scales, int rows, int hidden, int group,
    float amax_floor, int round_scale) {
    const int chunks = hidden / 16;
    const int lanes_per_group = group / 16;
    for (int r = blockIdx.x; r < rows; r += gridDim.x) {
        const std::uint32_t *xrow = x + static_cast<std::size_t>(r) * (hidden / 2);
        for (int base = 0; base < chunks; base += kThreads) {
            const int c = base + threadIdx.x;
            const bool live = c < chunks;
            uint4 a = make_uint4(0, 0, 0, 0), b = a;
            if (live) {
                a = aboleth::detail::ld_stream16(xrow + c * 8);
                b = aboleth::detail::ld_stream16(xrow + c * 8 + 4);
            }
            const float amax = group_max(amax16(a, b), lanes_per_group);
            const float scale = quant_scale(amax, amax_floor, round_scale);
            if (live) {
                *reinterpret_cast<uint4 *>(q + static_cast<std::size_t>(r) * hidden + c * 16) =
                    quant16(a, b, scale);
                if (c % lanes_per_group == 0)
                    scales[static_cast<std::size_t>(r) * (hidden / group) + c / lanes_per_group] = scale;
            }
        }
    }
}

// logits [T, experts] -> ids [T, k], weights [T, k]; one warp per token.
__global__ void __launch_bounds__(kThreads) router_topk_kernel(
    const float *logits, int *ids, float *weights, int tokens, int experts, int top_k,
    int renormalize) {
    const int warp = (blockIdx.x * kThreads + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (warp >= tokens)
        return;
    int id;
    float w;
    warp_softmax_topk(logits + static_cast<std::size_t>(warp) * experts, experts, top_k,
                      renormalize, id, w);
    if (lane < top_k) {
        ids[warp * top_k + lane] = id;
        weights[warp * top_k + lane] = w;
    }
}

// Exclusive scan of expert_counts -> offsets (one CTA; experts <= 1024 * 4).
__global__ void __launch_bounds__(1024) expert_offsets_kernel(
    const int *counts, int *offsets, int *total, int experts, int align) {
    __shared__ int s[1024];
    int carry = 0;
    for (int base = 0; base < experts; base += 1024) {
        const int e = base + threadIdx.x;
        int v = e < experts ? counts[e] : 0;
        if (align > 1)
            v = (v + align - 1) / align * align;
        s[threadIdx.x] = v;
        __syncthreads();
        for (int off = 1; off < 1024; off <<= 1) {
            const int add = threadIdx.x >= off ? s[threadIdx.x - off] : 0;
            __syncthreads();
            s[threadIdx.x] += add;
            __syncthreads();
        }
        if (e < experts)
            offsets[e] = carry + s[threadIdx.x] - v;
        carry += s[1023];
        __syncthreads();
    }
    if (threadIdx.x == 0 && total != nullptr)
        *total = carry;
}

// Gather received rows into expert-contiguous order:
//   dst[offsets[id] + pos] = src[row]   for every live (row, choice).
// Also writes the inverse map perm_row[offsets[id] + pos] = row * k + j.
__global__ void __launch_bounds__(kThreads) permute_kernel(
    const std::uint8_t *src, std::uint8_t *dst, const float *src_scales, float *dst_scales,
    const int *expert_ids, const int *expert_pos, const int *offsets,
    const unsigned long long *recv_counts, int *perm_row, int world, int capacity, int top_k,
    int row_bytes, int cols) {
    const int total = world * capacity;
    for (int row = blockIdx.x; row < total; row += gridDim.x) {
        const int srcr = row / capacity;
        if (static_cast<unsigned long long>(row - srcr * capacity) >= recv_counts[srcr])
            continue;
        for (int j = 0; j < top_k; ++j) {
            const int pos = expert_pos[row * top_k + j];
            if (pos < 0)
                continue;
            const int out = offsets[expert_ids[row * top_k + j]] + pos;
            const uint4 *s = reinterpret_cast<const uint4 *>(src + static_cast<std::size_t>(row) * row_bytes);
            uint4 *d = reinterpret_cast<uint4 *>(dst + static_cast<std::size_t>(out) * row_bytes);
            for (int v = threadIdx.x; v < row_bytes / 16; v += kThreads)
                d[v] = s[v];
            if (src_scales != nullptr)
                for (int c = threadIdx.x; c < cols; c += kThreads)
                    dst_scales[static_cast<std::size_t>(out) * cols + c] =
                        src_scales[static_cast<std::size_t>(row) * cols + c];
            if (threadIdx.x == 0 && perm_row != nullptr)
                perm_row[out] = row * top_k + j;
        }
    }
}

// out[row] = sum_j weights[row, j] * y[offsets[id] + pos]  (bf16, fp32 accumulate).
__global__ void __launch_bounds__(kThreads) unpermute_kernel(
    const std::uint32_t *y, std::uint32_t *out, const int *expert_ids, const int *expert_pos,
    const float *expert_weights, const int *offsets, const unsigned long long *recv_counts,
    int world, int capacity, int top_k, int hidden) {
    const int total = world * capacity;
    const int vecs = hidden / 8;
    for (int row = blockIdx.x; row < total; row += gridDim.x) {
        const int srcr = row / capacity;
        if (static_cast<unsigned long long>(row - srcr * capacity) >= recv_counts[srcr])
            continue;
        for (int v = threadIdx.x; v < vecs; v += kThreads) {
            float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
            for (int j = 0; j < top_k; ++j) {
                const int pos = expert_pos[row * top_k + j];
                if (pos < 0)
                    continue;
                const float w = expert_weights[row * top_k + j];
                const uint4 r = *reinterpret_cast<const uint4 *>(
                    y + static_cast<std::size_t>(offsets[expert_ids[row * top_k + j]] + pos) * (hidden / 2) + v * 4);
                acc[0] += w * bf16_lo(r.x); acc[1] += w * bf16_hi(r.x);
                acc[2] += w * bf16_lo(r.y); acc[3] += w * bf16_hi(r.y);
                acc[4] += w * bf16_lo(r.z); acc[5] += w * bf16_hi(r.z);
                acc[6] += w * bf16_lo(r.w); acc[7] += w * bf16_hi(r.w);
            }
            uint4 o;
            o.x = pack_bf16x2(acc[0], acc[1]);
            o.y = pack_bf16x2(acc[2], acc[3]);
            o.z = pack_bf16x2(acc[4], acc[5]);
            o.w = pack_bf16x2(acc[6], acc[7]);
            *reinterpret_cast<uint4 *>(out + static_cast<std::size_t>(row) * (hidden / 2) + v * 4) = o;
        }
    }
}

// The benchmark's stand-in expert, applied to every live (record, choice):
//   y[row] = sum_j w_j * dequant(x[row]) * (1 + (id_j mod 7) / 8)      (bf16 out)
// (reference oracle: experiments/dsl/moe/moe_common.py:72-140).  It writes in
// record layout so the combine can run unweighted, as in the reference.
__global__ void __launch_bounds__(kThreads) standin_expert_kernel(
    const std::uint8_t *payload, const float *scales, std::uint32_t *y, const int *expert_ids,
    const float *expert_weights, const int *expert_pos, const unsigned long long *recv_counts,
    int world, int capacity, int top_k, int hidden, int group, int value_fp8) {
    const int total = world * capacity;
    const int cols = hidden / group;
    for (int row = blockIdx.x; row < total; row += gridDim.x) {
        const int srcr = row / capacity;
        if (static_cast<unsigned long long>(row - srcr * capacity) >= recv_counts[srcr])
            continue;
        float coef = 0.f;
        for (int j = 0; j < top_k; ++j)
            if (expert_pos[row * top_k + j] >= 0)
                coef += expert_weights[row * top_k + j] *
                        (1.0f + static_cast<float>(expert_ids[row * top_k + j] % 7) * 0.125f);
        for (int v = threadIdx.x; v < hidden / 8; v += kThreads) {
            float f[8];
            if (value_fp8) {
                const uint2 q = *reinterpret_cast<const uint2 *>(payload + static_cast<std::size_t>(row) * hidden + v * 8);
                const float s = scales[static_cast<std::size_t>(row) * cols + (v * 8) / group];
                const std::uint32_t w[2] = {q.x, q.y};
#pragma unroll
                for (int i = 0; i < 2; ++i) {
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        const __half2_raw h2 = __nv_cvt_fp8x2_to_halfraw2(
                            static_cast<__nv_fp8x2_storage_t>((w[i] >> (16 * h)) & 0xffffu), __NV_E4M3);
                        const float2 ff = __half22float2(*reinterpret_cast<const __half2 *>(&h2));
                        f[i * 4 + h * 2] = ff.x * s;
                        f[i * 4 + h * 2 + 1] = ff.y * s;
                    }
                }
            } else {
                const uint4 r = *reinterpret_cast<const uint4 *>(payload + static_cast<std::size_t>(row) * hidden * 2 + v * 16);
                f[0] = bf16_lo(r.x); f[1] = bf16_hi(r.x); f[2] = bf16_lo(r.y); f[3] = bf16_hi(r.y);
                f[4] = bf16_lo(r.z); f[5] = bf16_hi(r.z); f[6] = bf16_lo(r.w); f[7] = bf16_hi(r.w);
            }
            uint4 o;
            o.x = pack_bf16x2(f[0] * coef, f[1] * coef);
            o.y = pack_bf16x2(f[2] * coef, f[3] * coef);
            o.z = pack_bf16x2(f[4] * coef, f[5] * coef);
            o.w = pack_bf16x2(f[6] * coef, f[7] * coef);
            *reinterpret_cast<uint4 *>(y + static_cast<std::size_t>(row) * (hidden / 2) + v * 4) = o;
        }
    }
}

// A CTA that has finished sending spins (bounded) on its peers' flags, and a
// peer's flag needs ALL of that peer's CTAs to have run.  Every CTA of the grid
// must therefore be resident at once: clamp the grid to what the device holds.
template <typename Kernel>
int resident_grid(Kernel kernel, int requested) {
    int device = 0, sms = 0, per_sm = 0;
    cudaGetDevice(&device);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
    cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, kThreads, 0);
    const int limit = sms * (per_sm > 0 ? per_sm : 1);
    return requested < limit ? requested : limit;
}

bool geometry_ok(const EpGeometry &g) {
    return g.world >= 1 && g.world <= kMaxWorld && g.top_k >= 1 && g.top_k <= kMaxTopK &&
           g.experts >= 1 && g.experts <= 32 * kMaxExpertsPerLane && g.hidden % 16 == 0 &&
           g.scale_group % 16 == 0 && g.scale_group <= 512 &&
           (g.scale_group & (g.scale_group - 1)) == 0 && g.hidden % g.scale_group == 0 &&
           g.hidden / g.scale_group <= 128 && g.capacity >= 1 && g.rank >= 0 && g.rank < g.world;
}

}  // namespace

// Argument blocks are passed as arrays of 64-bit words so the Python side needs
// no struct mirror: ints[] carries the integer geometry, ptrs[] the addresses.
AB_EXPORT int ab_ep_dispatch(const int *ints, float amax_floor, const std::uint64_t *ptrs,
                             int grid, cudaStream_t stream) {
    DispatchParams p{};
    p.g = EpGeometry{ints[0], ints[1], ints[2], ints[3], ints[4], ints[5], ints[6],
                     ints[7], ints[8], ints[9], amax_floor};
    p.num_tokens = ints[10];
    p.routing = ints[11];
    p.renormalize = ints[12];
    p.phases = ints[13];
    p.by_warp = ints[15];
    if (!geometry_ok(p.g) || p.num_tokens < 0 || p.num_tokens > p.g.capacity || grid < 0)
        return -1;
    if (grid == 0)  // auto: enough CTAs for the tokens, never fewer than 32 for the unpack
        grid = p.by_warp ? (p.num_tokens + kThreads / 32 - 1) / (kThreads / 32) : p.num_tokens;
    if (grid < 32)
        grid = 32;
    int i = 0;
    p.x = reinterpret_cast<const std::uint32_t *>(ptrs[i++]);
    p.logits = reinterpret_cast<const float *>(ptrs[i++]);
    p.ids_in = reinterpret_cast<const int *>(ptrs[i++]);
    p.weights_in = reinterpret_cast<const float *>(ptrs[i++]);
    p.ids_out = reinterpret_cast<int *>(ptrs[i++]);
    p.weights_out = reinterpret_cast<float *>(ptrs[i++]);
    p.owners = reinterpret_cast<const int *>(ptrs[i++]);
    p.source_slots = reinterpret_cast<int *>(ptrs[i++]);
    p.send_counts = reinterpret_cast<unsigned long long *>(ptrs[i++]);
    p.done = reinterpret_cast<unsigned *>(ptrs[i++]);
    p.overflow = reinterpret_cast<int *>(ptrs[i++]);
    p.epoch = reinterpret_cast<const unsigned long long *>(ptrs[i++]);
    p.status = reinterpret_cast<unsigned long long *>(ptrs[i++]);
    p.peer_payload = reinterpret_cast<const std::uint64_t *>(ptrs[i++]);
    p.peer_meta = reinterpret_cast<const std::uint64_t *>(ptrs[i++]);
    p.peer_counts = reinterpret_cast<const std::uint64_t *>(ptrs[i++]);
    p.peer_flags = reinterpret_cast<const std::uint64_t *>(ptrs[i++]);
    p.recv_meta = reinterpret_cast<const int *>(ptrs[i++]);
    p.recv_counts = reinterpret_cast<const unsigned long long *>(ptrs[i++]);
    p.flags = reinterpret_cast<const std::uint64_t *>(ptrs[i++]);
    p.expert_ids = reinterpret_cast<int *>(ptrs[i++]);
    p.expert_weights = reinterpret_cast<float *>(ptrs[i++]);
    p.expert_pos = reinterpret_cast<int *>(ptrs[i++]);
    p.expert_counts = reinterpret_cast<int *>(ptrs[i++]);
    p.expert_scales = reinterpret_cast<float *>(ptrs[i++]);
    p.trace = reinterpret_cast<unsigned long long *>(ptrs[i++]);
    ep_dispatch_kernel<<<resident_grid(ep_dispatch_kernel, grid), kThreads, 0, stream>>>(p);
    return ab::launch_result("ep_dispatch");
}

AB_EXPORT int ab_ep_combine(const int *ints, float amax_floor, const std::uint64_t *ptrs, int grid,
                            cudaStream_t stream) {
    CombineParams p{};
    p.g = EpGeometry{ints[0], ints[1], ints[2], ints[3], ints[4], ints[5], ints[6],
                     ints[7], ints[8], ints[9], amax_floor};
    p.num_tokens = ints[10];
    p.phases = ints[13];
    p.weighted = ints[14];
    p.by_warp = ints[15];
    if (!geometry_ok(p.g) || p.num_tokens < 0 || p.num_tokens > p.g.capacity || grid < 0)
        return -1;
    if (grid == 0)
        grid = p.by_warp ? 1 << 20 : (p.num_tokens * 8 < 32 ? 32 : p.num_tokens * 8);
    int i = 0;
    p.expert_out = reinterpret_cast<const std::uint32_t *>(ptrs[i++]);
    p.expert_ids = reinterpret_cast<const int *>(ptrs[i++]);
    p.expert_pos = reinterpret_cast<const int *>(ptrs[i++]);
    p.expert_weights = reinterpret_cast<const float *>(ptrs[i++]);
    p.expert_offsets = reinterpret_cast<const int *>(ptrs[i++]);
    p.recv_meta = reinterpret_cast<const int *>(ptrs[i++]);
    p.recv_counts = reinterpret_cast<const unsigned long long *>(ptrs[i++]);
    p.peer_return = reinterpret_cast<const std::uint64_t *>(ptrs[i++]);
    p.peer_return_flags = reinterpret_cast<const std::uint64_t *>(ptrs[i++]);
    p.return_flags = reinterpret_cast<const std::uint64_t *>(ptrs[i++]);
    p.returned = reinterpret_cast<const std::uint32_t *>(ptrs[i++]);
    p.source_slots = reinterpret_cast<const int *>(ptrs[i++]);
    p.out = reinterpret_cast<std::uint32_t *>(ptrs[i++]);
    p.done = reinterpret_cast<unsigned *>(ptrs[i++]);
    p.expert_counts = reinterpret_cast<int *>(ptrs[i++]);
    p.epoch = reinterpret_cast<unsigned long long *>(ptrs[i++]);
    p.status = reinterpret_cast<unsigned long long *>(ptrs[i++]);
    p.trace = reinterpret_cast<unsigned long long *>(ptrs[i++]);
    ep_combine_kernel<<<resident_grid(ep_combine_kernel, grid), kThreads, 0, stream>>>(p);
    return ab::launch_result("ep_combine");
}

AB_EXPORT int ab_quant_fp8(const void *x, void *q, float *scales, int rows, int hidden, int group,
                           float amax_floor, int round_scale, cudaStream_t stream) {
    if (rows < 1 || hidden % 16 || group % 16 || hidden % group || (group & (group - 1)) || group > 512)
        return -1;
    const int grid = rows < 148 * 8 ? rows : 148 * 8;
    quant_fp8_kernel<<<grid, kThreads, 0, stream>>>(static_cast<const std::uint32_t *>(x),
                                                    static_cast<std::uint8_t *>(q), scales, rows,
                                                    hidden, group, amax_floor, round_scale);
    return ab::launch_result("quant_fp8");
}

AB_EXPORT int ab_router_topk(const float *logits, int *ids, float *weights, int tokens, int experts,
                             int top_k, int renormalize, cudaStream_t stream) {
    if (tokens < 1 || experts < 1 || experts > 32 * kMaxExpertsPerLane || top_k < 1 ||
        top_k > kMaxTopK || top_k > experts)
        return -1;
    const int grid = (tokens * 32 + kThreads - 1) / kThreads;
    router_topk_kernel<<<grid, kThreads, 0, stream>>>(logits, ids, weights, tokens, experts, top_k,
                                                      renormalize);
    return ab::launch_result("router_topk");
}

AB_EXPORT int ab_expert_offsets(const int *counts, int *offsets, int *total, int experts, int align,
                                cudaStream_t stream) {
    if (experts < 1)
        return -1;
    expert_offsets_kernel<<<1, 1024, 0, stream>>>(counts, offsets, total, experts, align);
    return ab::launch_result("expert_offsets");
}

AB_EXPORT int ab_permute(const void *src, void *dst, const float *src_scales, float *dst_scales,
                         const int *expert_ids, const int *expert_pos, const int *offsets,
                         const unsigned long long *recv_counts, int *perm_row, int world,
                         int capacity, int top_k, int row_bytes, int cols, cudaStream_t stream) {
    if (row_bytes % 16 || world < 1 || capacity < 1)
        return -1;
    const int total = world * capacity;
    const int grid = total < 148 * 8 ? total : 148 * 8;
    permute_kernel<<<grid, kThreads, 0, stream>>>(
        static_cast<const std::uint8_t *>(src), static_cast<std::uint8_t *>(dst), src_scales,
        dst_scales, expert_ids, expert_pos, offsets, recv_counts, perm_row, world, capacity, top_k,
        row_bytes, cols);
    return ab::launch_result("permute");
}

AB_EXPORT int ab_unpermute(const void *y, void *out, const int *expert_ids, const int *expert_pos,
                           const float *expert_weights, const int *offsets,
                           const unsigned long long *recv_counts, int world, int capacity, int top_k,
                           int hidden, cudaStream_t stream) {
    if (hidden % 8 || world < 1 || capacity < 1)
        return -1;
    const int total = world * capacity;
    const int grid = total < 148 * 8 ? total : 148 * 8;
    unpermute_kernel<<<grid, kThreads, 0, stream>>>(
        static_cast<const std::uint32_t *>(y), static_cast<std::uint32_t *>(out), expert_ids,
        expert_pos, expert_weights, offsets, recv_counts, world, capacity, top_k, hidden);
    return ab::launch_result("unpermute");
}

AB_EXPORT int ab_standin_expert(const void *payload, const float *scales, void *y,
                                const int *expert_ids, const float *expert_weights,
                                const int *expert_pos, const unsigned long long *recv_counts,
                                int world, int capacity, int top_k, int hidden, int group,
                                int value_fp8, cudaStream_t stream) {
    if (hidden % 8 || world < 1 || capacity < 1)
        return -1;
    const int total = world * capacity;
    const int grid = total < 148 * 8 ? total : 148 * 8;
    standin_expert_kernel<<<grid, kThreads, 0, stream>>>(
        static_cast<const std::uint8_t *>(payload), scales, static_cast<std::uint32_t *>(y),
        expert_ids, expert_weights, expert_pos, recv_counts, world, capacity, top_k, hidden, group,
        value_fp8);
    return ab::launch_result("standin_expert");
}
