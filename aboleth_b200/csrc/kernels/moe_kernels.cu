// Expert-parallel dispatch and combine as two launches per MoE layer.
//
// DISPATCH (one launch).  The sender does ALL the per-record work; a receiver only waits.
//   * route: softmax + top-k in one warp (or given ids / weights);
//   * slots: one record per (token, destination rank that owns a chosen expert)
//     (rank-deduplicated records, reference python/aboleth/moe/kernels.py:43-70).  Above the
//     latency threshold the slots are handed out in TOKEN ORDER: every CTA counts its tokens'
//     records per destination, one bounded grid barrier, a scan of the CTA counts.  The combine
//     of the same layer returns records in slot order, so a token-ordered segment lets the
//     source rank reduce token t while later records are still in flight;
//   * position inside the expert: one LOCAL `atom.add` per chosen expert gives the record's
//     position among THIS rank's records for that expert; the per-expert totals travel with the
//     record counts, and the receiver's offset table places source s after sources < s.  (A
//     position taken from the owner's counter over NVLink was tried first: its round trip queues
//     behind the payload in both directions and lengthened the send by a fifth at 8 GPUs.)
//   * payload: the row is quantised once to e4m3 with one fp32 scale per `scale_group` columns
//     and stored straight into every destination's receive segment (no send staging);
//   * metadata row (wire format) and the unpacked view the expert stage reads (expert ids,
//     gate weights, positions) are written by the sender too;
//   * the last CTA to arrive writes each peer's record count and ONE `st.release.sys` flag per
//     peer, then waits (bounded) for the peers' flags and totals the per-source expert counts.
// Every other CTA exits after its stores: no CTA polls while another still sends.
//
// COMBINE (one launch).  Sender warps walk the received records in slot order, round-robin over
// the source ranks; one record = sum_j gate_j * expert_out[row_j] in fp32 (the gate-weighted
// reduction happens here), rounded to bf16, stored into the source rank's return segment.
// Records complete in blocks of `block` rows: the warp that completes a block publishes that
// block's flag on the source rank.  Reducer warps of the same launch walk this rank's tokens in
// order, wait (bounded) only for the blocks that hold the token's partial rows, and sum them.
// The reduction therefore runs under the transfer instead of after it.  The kernel ends when
// every peer has said that it finished sending (its reads of this layer's records are over), so
// the next dispatch may overwrite the receive segments.
//
// The reference runs this as >= 9 launches (pack, three self copies, send, await, unpack, send,
// await, gather: python/aboleth/moe/native.py:433-615).
//
// Sender work never waits on a peer, so the two halves can also be launched separately
// (`phases` mask); that is how a single GPU emulates several ranks.
#include "moe_common.cuh"

namespace {

using namespace ab::moe;
using aboleth::Status;

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;
constexpr int kPhaseSend = 1;
constexpr int kPhaseRecv = 2;
constexpr int kMaxTokensPerCta = 64;  // ordered slots: tokens one CTA may own
constexpr unsigned kFull = 0xffffffffu;

// Counter words in `done`.
constexpr int kDoneDispatch = 0, kDoneCombine = 1, kBarrierCount = 2, kBarrierGen = 3, kDoneSenders = 4,
              kNextToken = 5, kNextRecord = 8;  // kNextRecord + d: next unclaimed record of destination d

struct EpGeometry {
    int rank, world, experts, top_k, hidden, scale_group, capacity;
    int value_fp8, round_scale;
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
    int *ids_out;                  // [T, k]  (required with routing == 1)
    float *weights_out;            // [T, k]
    const int *owners;             // [experts] -> rank
    const int *placeholders;       // [world]: an expert rank d does not own (-1 if none)
    // sender state (local)
    int *source_slots;             // [capacity, world]
    unsigned long long *send_counts;  // [world]   (unordered slots)
    unsigned *done;                // [8] arrival counters, see kDone*
    int *overflow;                 // [1]
    const unsigned long long *epoch;  // device epoch (starts at 1)
    unsigned long long *status;    // [2]
    int *block_counts;             // [grid, world] records per CTA and destination (ordered slots)
    // peers (device arrays of addresses, [world])
    const std::uint64_t *peer_payload, *peer_meta, *peer_counts, *peer_flags;
    const std::uint64_t *peer_ids, *peer_weights, *peer_pos, *peer_expert_counts;
    int *send_expert_counts;       // [experts] (record, choice) pairs this rank sent per expert
    // receiver side (local)
    const unsigned long long *recv_counts;  // [world]
    const std::uint64_t *flags;             // [world]
    const int *recv_expert_counts; // [world, experts]: row s written by rank s
    int *expert_counts;            // [experts] totals handed to the expert stage
    unsigned long long *trace;     // optional [8] %globaltimer stamps
};

__device__ __forceinline__ int meta_words(const EpGeometry &g) {
    return 2 + 2 * g.top_k + (g.value_fp8 ? g.hidden / g.scale_group : 0);
}

// Phase stamps for the tracing buffer: slot i <- %globaltimer (ns).
__device__ __forceinline__ void stamp(unsigned long long *trace, int slot, bool who) {
    if (trace != nullptr && who)
        trace[slot] = aboleth::detail::globaltimer_ns();
}

__device__ __forceinline__ unsigned atom_add_acq_rel_gpu(unsigned *p, unsigned v) {
    unsigned old;
    asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], %2;" : "=r"(old) : "l"(p), "r"(v) : "memory");
    return old;
}

__device__ __forceinline__ unsigned ld_acquire_gpu(const unsigned *p) {
    unsigned v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

__device__ __forceinline__ void st_release_gpu(unsigned *p, unsigned v) {
    asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

__device__ __forceinline__ void st_relaxed_gpu(unsigned *p, unsigned v) {
    asm volatile("st.relaxed.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

__device__ __forceinline__ int ld_volatile_int(const int *p) {
    int v;
    asm volatile("ld.volatile.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// Thread 0 of every CTA calls this after a CTA barrier.  The system fence makes the CTA's peer
// stores visible before the arrival is; the CTA that arrives last has acquired every arrival.
__device__ __forceinline__ bool arrive_last(unsigned *counter, unsigned expected) {
    aboleth::detail::fence_acq_rel_sys();
    return atom_add_acq_rel_gpu(counter, 1u) == expected - 1;
}

// All CTAs of the grid (co-resident: see resident_grid).  Bounded: false after the timeout.
__device__ __forceinline__ bool grid_barrier(unsigned *done, unsigned long long *status, int *s_fail) {
    __syncthreads();
    if (threadIdx.x == 0) {
        *s_fail = 0;
        const unsigned gen = ld_acquire_gpu(done + kBarrierGen);
        if (atom_add_acq_rel_gpu(done + kBarrierCount, 1u) == gridDim.x - 1) {
            st_relaxed_gpu(done + kBarrierCount, 0u);
            st_release_gpu(done + kBarrierGen, gen + 1);
        } else {
            const std::uint64_t start = aboleth::detail::globaltimer_ns();
            unsigned spins = 0;
            while (ld_acquire_gpu(done + kBarrierGen) == gen) {
                if ((++spins & 63) == 0 &&
                    aboleth::detail::globaltimer_ns() - start > ABOLETH_WAIT_TIMEOUT_NS) {
                    ab::set_status(status, Status::Timeout, 0x1300);
                    *s_fail = 1;
                    break;
                }
            }
        }
    }
    __syncthreads();
    return *s_fail == 0;
}

// Threads d < world wait for flag d.  Returns false on timeout (status recorded).
__device__ __forceinline__ bool wait_all_peers(const std::uint64_t *flags, int world, int stride,
                                               std::uint64_t epoch, unsigned long long *status,
                                               int *s_fail, unsigned detail_base) {
    if (threadIdx.x == 0)
        *s_fail = 0;
    __syncthreads();
    if (threadIdx.x < world) {
        const Status s = aboleth::wait_signal_status(flags + static_cast<std::size_t>(threadIdx.x) * stride, epoch);
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
    const unsigned lo = __shfl_sync(kFull, static_cast<unsigned>(v), src);
    const unsigned hi = __shfl_sync(kFull, static_cast<unsigned>(v >> 32), src);
    return (static_cast<std::uint64_t>(hi) << 32) | lo;
}

// Lanes < top_k: (id, weight) of choice `lane` of token t, from the router or from the caller.
__device__ __forceinline__ void route_token(const DispatchParams &p, int t, int &id, float &w) {
    const EpGeometry &g = p.g;
    const int lane = threadIdx.x & 31;
    id = -1;
    w = 0.f;
    if (p.routing == 1) {
        warp_softmax_topk(p.logits + static_cast<std::size_t>(t) * g.experts, g.experts, g.top_k,
                          p.renormalize, id, w);
    } else if (lane < g.top_k) {
        id = p.ids_in[t * g.top_k + lane];
        w = p.weights_in[t * g.top_k + lane];
    }
    if (lane < g.top_k) {
        if (p.ids_out != nullptr)
            p.ids_out[t * g.top_k + lane] = id;
        if (p.weights_out != nullptr)
            p.weights_out[t * g.top_k + lane] = w;
    }
}

__device__ __forceinline__ int owner_of(const DispatchParams &p, int id) {
    const int lane = threadIdx.x & 31;
    return (lane < p.g.top_k && id >= 0 && id < p.g.experts) ? p.owners[id] : -1;
}

// The record's position among this rank's records for expert `id` (a local atomic).
__device__ __forceinline__ int reserve_position(const DispatchParams &p, int owner, int id) {
    (void)owner;
    return atomicAdd(p.send_expert_counts + id, 1);
}

// One warp sends one token whose routing is (id, w, owner) in lanes < top_k and whose slot at
// destination `lane` is `slot` (-1: no record there).  No CTA-level synchronisation.
__device__ __forceinline__ void send_token_by_warp(const DispatchParams &p, int t, WarpScratch &ws,
                                                   int id, float w, int owner, int slot) {
    const EpGeometry &g = p.g;
    const int lane = threadIdx.x & 31;
    const int cols = g.value_fp8 ? g.hidden / g.scale_group : 0;
    const int words = meta_words(g);
    const int row_bytes = g.value_fp8 ? g.hidden : g.hidden * 2;

    std::uint64_t my_row = 0, my_meta = 0;
    if (lane < g.world) {
        p.source_slots[t * g.world + lane] = slot;
        if (slot >= 0) {
            const std::size_t row = static_cast<std::size_t>(g.rank) * g.capacity + slot;
            my_row = p.peer_payload[lane] + row * row_bytes;
            my_meta = p.peer_meta[lane] + row * words * 4;
        }
    }
    const unsigned live = __ballot_sync(kFull, slot >= 0);
    // Position inside the expert's group of this source; needed after the payload.
    const int owner_slot = __shfl_sync(kFull, slot, owner >= 0 ? owner : 0);
    int pos = -1;
    if (owner >= 0 && owner_slot >= 0)
        pos = reserve_position(p, owner, id);

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

    // ---- metadata rows (wire format) and the unpacked view ----
    __syncwarp();
    if (lane == 0)
        ws.meta[0] = t;
    for (int c = lane; c < cols; c += 32)
        ws.meta[2 + 2 * g.top_k + c] = __float_as_int(ws.scale[c]);
    for (unsigned m = live; m; m &= m - 1) {
        const int d = __ffs(m) - 1;
        const bool mine = lane < g.top_k && owner == d;
        const unsigned sel = __ballot_sync(kFull, mine);
        const int n = __popc(sel);
        const int idx = __popc(sel & ((1u << lane) - 1));
        const std::size_t row = static_cast<std::size_t>(g.rank) * g.capacity + __shfl_sync(kFull, slot, d);
        int *ids = reinterpret_cast<int *>(p.peer_ids[d]) + row * g.top_k;
        float *wts = reinterpret_cast<float *>(p.peer_weights[d]) + row * g.top_k;
        int *poss = reinterpret_cast<int *>(p.peer_pos[d]) + row * g.top_k;
        if (lane == 0)
            ws.meta[1] = n;
        if (mine) {
            ws.meta[2 + idx] = id;
            ws.meta[2 + g.top_k + idx] = __float_as_int(w);
            ids[idx] = id;
            wts[idx] = w;
            poss[idx] = pos;
        }
        if (lane >= n && lane < g.top_k) {
            ws.meta[2 + lane] = -1;
            ws.meta[2 + g.top_k + lane] = 0;
            // Unused choice slots name an expert the destination does not own, at weight 0.
            ids[lane] = p.placeholders[d];
            wts[lane] = 0.f;
            poss[lane] = -1;
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

// Lane d < world: take the next slot of destination d if this token has a record there.
__device__ __forceinline__ int take_slot(const DispatchParams &p, int owner) {
    const EpGeometry &g = p.g;
    const int lane = threadIdx.x & 31;
    int nsel = 0;
    for (int j = 0; j < g.top_k; ++j)
        nsel += __shfl_sync(kFull, owner, j) == lane;
    int slot = -1;
    if (lane < g.world && nsel > 0) {
        const unsigned long long got = atomicAdd(p.send_counts + lane, 1ull);
        if (got < static_cast<unsigned long long>(g.capacity))
            slot = static_cast<int>(got);
        else
            *p.overflow = 1;
    }
    return slot;
}

// The publishing CTA: wait for every peer's flag, check the counts, hand the expert counters over.
__device__ __forceinline__ void finish_dispatch(const DispatchParams &p, std::uint64_t epoch, int *s_fail) {
    const EpGeometry &g = p.g;
    const int tid = threadIdx.x;
    if (!wait_all_peers(p.flags, g.world, 1, epoch, p.status, s_fail, 0x1000))
        return;
    stamp(p.trace, 3, tid == 0);
    if (tid < g.world &&
        aboleth::detail::ld_relaxed_sys(reinterpret_cast<const std::uint64_t *>(p.recv_counts + tid)) >
            static_cast<std::uint64_t>(g.capacity))
        ab::set_status(p.status, Status::Malformed, 0x1100 + tid);
    // Row s of the table was written by rank s before it released its flag.
    for (int e = tid; e < g.experts; e += kThreads) {
        int total = 0;
        for (int src = 0; src < g.world; ++src)
            total += ld_volatile_int(p.recv_expert_counts + src * g.experts + e);
        p.expert_counts[e] = total;
    }
    stamp(p.trace, 4, tid == 0);
}

// BY_WARP: one warp per token (throughput, token-ordered slots) or one CTA per token (latency).
template <bool BY_WARP>
__global__ void __launch_bounds__(kThreads, 4) ep_dispatch_kernel(DispatchParams p) {
    const EpGeometry &g = p.g;
    __shared__ int s_id[kMaxTopK];
    __shared__ float s_w[kMaxTopK];
    __shared__ int s_owner[kMaxTopK];
    __shared__ int s_pos[kMaxTopK];
    __shared__ int s_slot[kMaxWorld];
    __shared__ int s_dest[kMaxWorld];
    __shared__ int s_base[kMaxWorld];
    __shared__ int s_ndest;
    __shared__ float s_scale[128];  // hidden / scale_group <= 128
    __shared__ int s_flag;
    __shared__ unsigned s_mask[kMaxTokensPerCta];
    __shared__ unsigned short s_local[kMaxTokensPerCta][kMaxWorld];

    const int tid = threadIdx.x;
    const int lane = tid & 31;
    const int warp = tid >> 5;
    const std::uint64_t epoch = *p.epoch;
    const int cols = g.value_fp8 ? g.hidden / g.scale_group : 0;
    const int words = meta_words(g);
    const int row_bytes = g.value_fp8 ? g.hidden : g.hidden * 2;
    const bool tracer = blockIdx.x == 0 && tid == 0;
    stamp(p.trace, 0, tracer);
    // Warp-per-token launches give CTA b the contiguous tokens [first, last); slots are handed out
    // in token order when a CTA's share fits the shared-memory tables.
    const int per_cta = (p.num_tokens + gridDim.x - 1) / gridDim.x;
    const bool ordered = BY_WARP && per_cta <= kMaxTokensPerCta;

    if constexpr (BY_WARP) if (p.phases & kPhaseSend) {
        __shared__ WarpScratch scratch[kWarps];
        const int first = blockIdx.x * per_cta;
        const int last = min(p.num_tokens, first + per_cta);
        if (ordered || p.routing == 1) {
            // Pass 1: route, and note which destinations every token has a record for.
            for (int t = first + warp; t < last; t += kWarps) {
                int id;
                float w;
                route_token(p, t, id, w);
                const int owner = owner_of(p, id);
                const unsigned mask = __reduce_or_sync(kFull, owner >= 0 ? 1u << owner : 0u);
                if (ordered && lane == 0)
                    s_mask[t - first] = mask;
            }
        }
        if (ordered) {
            __syncthreads();
            if (warp == 0 && lane < g.world) {
                int run = 0;
                for (int i = 0; i < last - first; ++i) {
                    s_local[i][lane] = static_cast<unsigned short>(run);
                    run += (s_mask[i] >> lane) & 1u;
                }
                p.block_counts[blockIdx.x * g.world + lane] = run;
            }
            if (!grid_barrier(p.done, p.status, &s_flag))
                return;
            // Slots of this CTA's records start after those of the CTAs before it.
            for (int d = warp; d < g.world; d += kWarps) {
                int sum = 0;
                for (int b = lane; b < static_cast<int>(blockIdx.x); b += 32)
                    sum += ld_volatile_int(p.block_counts + b * g.world + d);
                for (int off = 16; off > 0; off >>= 1)
                    sum += __shfl_xor_sync(kFull, sum, off);
                if (lane == 0)
                    s_base[d] = sum;
            }
            __syncthreads();
        }
        const int *ids_src = (p.routing == 1 || p.ids_in == nullptr) ? p.ids_out : p.ids_in;
        const float *w_src = (p.routing == 1 || p.weights_in == nullptr) ? p.weights_out : p.weights_in;
        for (int t = first + warp; t < last; t += kWarps) {
            int id = -1;
            float w = 0.f;
            if (ordered || p.routing == 1) {
                if (lane < g.top_k) {
                    id = ids_src[t * g.top_k + lane];
                    w = w_src[t * g.top_k + lane];
                }
            } else {
                route_token(p, t, id, w);
            }
            const int owner = owner_of(p, id);
            int slot;
            if (ordered) {
                slot = -1;
                if (lane < g.world && ((s_mask[t - first] >> lane) & 1u))
                    slot = s_base[lane] + s_local[t - first][lane];
            } else {
                slot = take_slot(p, owner);
            }
            send_token_by_warp(p, t, scratch[warp], id, w, owner, slot);
        }
    }
    if constexpr (!BY_WARP) if (p.phases & kPhaseSend) {
        const int chunks = g.hidden / 16;  // 16 elements per thread-step
        const int lanes_per_group = g.scale_group / 16;
        constexpr int kPayloadThreads = kThreads - 32;  // warps 1..7 move the row, warp 0 routes
        for (int t = blockIdx.x; t < p.num_tokens; t += gridDim.x) {
            const std::uint32_t *xrow = p.x + static_cast<std::size_t>(t) * (g.hidden / 2);
            int pos = -1;
            for (int base = 0; base < chunks; base += 2 * kPayloadThreads) {
                // Quantisation needs no routing: the payload warps load and quantise two steps each
                // while warp 0 routes the token; only the stores wait for the destinations.
                uint4 a[2], b[2];
                const int pt = tid - 32;
                if (warp > 0) {
#pragma unroll
                    for (int u = 0; u < 2; ++u) {
                        const int c = base + u * kPayloadThreads + pt;
                        a[u] = make_uint4(0, 0, 0, 0);
                        b[u] = a[u];
                        if (c < chunks) {
                            a[u] = aboleth::detail::ld_stream16(xrow + c * 8);
                            b[u] = aboleth::detail::ld_stream16(xrow + c * 8 + 4);
                        }
                    }
                    if (g.value_fp8) {
#pragma unroll
                        for (int u = 0; u < 2; ++u) {
                            const int c = base + u * kPayloadThreads + pt;
                            const float amax = group_max(amax16(a[u], b[u]), lanes_per_group);
                            const float scale = quant_scale(amax, g.amax_floor, g.round_scale);
                            a[u] = quant16(a[u], b[u], scale);
                            if (c < chunks && c % lanes_per_group == 0)
                                s_scale[c / lanes_per_group] = scale;
                        }
                    }
                } else if (base == 0) {
                    int id;
                    float w;
                    route_token(p, t, id, w);
                    const int owner = owner_of(p, id);
                    if (lane < g.top_k) {
                        s_id[lane] = id;
                        s_w[lane] = w;
                        s_owner[lane] = owner;
                    }
                    const int slot = take_slot(p, owner);
                    if (lane < g.world) {
                        p.source_slots[t * g.world + lane] = slot;
                        s_slot[lane] = slot;
                    }
                    const unsigned live = __ballot_sync(kFull, slot >= 0);
                    if (slot >= 0)
                        s_dest[__popc(live & ((1u << lane) - 1))] = lane;
                    if (lane == 0)
                        s_ndest = __popc(live);
                    // Position inside the expert's group: asked for now, read after the payload went out.
                    const int owner_slot = __shfl_sync(kFull, slot, owner >= 0 ? owner : 0);
                    if (owner >= 0 && owner_slot >= 0)
                        pos = reserve_position(p, owner, id);
                }
                if (base == 0)
                    __syncthreads();
                if (warp > 0) {
                    const int ndest = s_ndest;
#pragma unroll
                    for (int u = 0; u < 2; ++u) {
                        const int c = base + u * kPayloadThreads + pt;
                        if (c >= chunks)
                            continue;
                        for (int i = 0; i < ndest; ++i) {
                            const int d = s_dest[i];
                            std::uint8_t *row = reinterpret_cast<std::uint8_t *>(p.peer_payload[d]) +
                                (static_cast<std::size_t>(g.rank) * g.capacity + s_slot[d]) * row_bytes;
                            if (g.value_fp8) {
                                aboleth::detail::st_stream16(row + c * 16, a[u]);
                            } else {
                                aboleth::detail::st_stream16(row + c * 32, a[u]);
                                aboleth::detail::st_stream16(row + c * 32 + 16, b[u]);
                            }
                        }
                    }
                }
            }
            const int ndest = s_ndest;
            if (warp == 0 && lane < g.top_k)
                s_pos[lane] = pos;
            __syncthreads();

            // ---- metadata rows and the unpacked view: one warp per destination ----
            for (int i = warp; i < ndest; i += kWarps) {
                const int d = s_dest[i];
                const std::size_t row = static_cast<std::size_t>(g.rank) * g.capacity + s_slot[d];
                int *meta = reinterpret_cast<int *>(p.peer_meta[d]) + row * words;
                int *ids = reinterpret_cast<int *>(p.peer_ids[d]) + row * g.top_k;
                float *wts = reinterpret_cast<float *>(p.peer_weights[d]) + row * g.top_k;
                int *poss = reinterpret_cast<int *>(p.peer_pos[d]) + row * g.top_k;
                const bool mine = lane < g.top_k && s_owner[lane] == d;
                const unsigned sel = __ballot_sync(kFull, mine);
                const int nsel = __popc(sel);
                if (lane == 0) {
                    meta[0] = t;
                    meta[1] = nsel;
                }
                if (mine) {
                    const int idx = __popc(sel & ((1u << lane) - 1));
                    meta[2 + idx] = s_id[lane];
                    meta[2 + g.top_k + idx] = __float_as_int(s_w[lane]);
                    ids[idx] = s_id[lane];
                    wts[idx] = s_w[lane];
                    poss[idx] = s_pos[lane];
                }
                if (lane >= nsel && lane < g.top_k) {
                    meta[2 + lane] = -1;
                    meta[2 + g.top_k + lane] = 0;
                    ids[lane] = p.placeholders[d];
                    wts[lane] = 0.f;
                    poss[lane] = -1;
                }
                for (int c = lane; c < cols; c += 32)
                    meta[2 + 2 * g.top_k + c] = __float_as_int(s_scale[c]);
            }
            __syncthreads();
        }
    }

    bool publisher = false;
    if (p.phases & kPhaseSend) {
        // ---- publication: the last CTA writes counts and one flag per peer ----
        __syncthreads();
        stamp(p.trace, 1, tracer);
        if (tid == 0)
            s_flag = arrive_last(p.done + kDoneDispatch, gridDim.x) ? 1 : 0;
        __syncthreads();
        publisher = s_flag != 0;
        if (publisher) {
            stamp(p.trace, 2, tid == 0);
            if (ordered) {
                for (int d = warp; d < g.world; d += kWarps) {
                    int sum = 0;
                    for (int b = lane; b < static_cast<int>(gridDim.x); b += 32)
                        sum += ld_volatile_int(p.block_counts + b * g.world + d);
                    for (int off = 16; off > 0; off >>= 1)
                        sum += __shfl_xor_sync(kFull, sum, off);
                    if (lane == 0)
                        s_base[d] = sum;
                }
            } else if (tid < g.world) {
                s_base[tid] = static_cast<int>(ab::min64(
                    aboleth::detail::ld_relaxed_sys(reinterpret_cast<const std::uint64_t *>(p.send_counts + tid)),
                    static_cast<std::uint64_t>(g.capacity)));
            }
            // Every expert's pair count goes to its owner (row `rank` of the owner's table).
            for (int e = tid; e < g.experts; e += kThreads) {
                const int owner = p.owners[e];
                int *row = reinterpret_cast<int *>(p.peer_expert_counts[owner]) +
                           static_cast<std::size_t>(g.rank) * g.experts;
                asm volatile("st.relaxed.sys.global.s32 [%0], %1;" ::"l"(row + e),
                             "r"(ld_volatile_int(p.send_expert_counts + e)) : "memory");
                p.send_expert_counts[e] = 0;
            }
            __syncthreads();
            if (tid < g.world) {
                std::uint64_t *cnt = reinterpret_cast<std::uint64_t *>(p.peer_counts[tid]) + g.rank;
                std::uint64_t *flag = reinterpret_cast<std::uint64_t *>(p.peer_flags[tid]) + g.rank;
                aboleth::detail::st_relaxed_sys(cnt, static_cast<std::uint64_t>(s_base[tid]));
                aboleth::detail::st_release_sys(flag, epoch);
                p.send_counts[tid] = 0;
                if (tid == 0)
                    p.done[kDoneDispatch] = 0;
            }
        }
    }
    if (p.phases & kPhaseRecv) {
        // Fused launch: the publishing CTA finishes.  Receive-only launch: CTA 0 does.
        if ((p.phases & kPhaseSend) ? publisher : blockIdx.x == 0)
            finish_dispatch(p, epoch, &s_flag);
    }
}

struct CombineParams {
    EpGeometry g;
    int num_tokens, phases, weighted, by_warp;
    int block, nblk;                   // records per readiness block, blocks per source segment
    int send_warps;                    // warps per CTA that send in a fused by-warp launch
    // expert side
    const std::uint32_t *expert_out;   // bf16 rows: weighted ? [pairs, hidden] : [world*capacity, hidden]
    const int *expert_ids, *expert_pos;
    const float *expert_weights;
    const int *expert_offsets;         // [world, experts] first row of (source, expert) in expert_out (weighted)
    const int *recv_meta;
    const unsigned long long *recv_counts;
    // transport
    const std::uint64_t *peer_return, *peer_return_flags;
    const std::uint64_t *return_flags;  // local [world, nblk + 1]; the last word: that peer finished sending
    const std::uint32_t *returned;      // local [world*capacity, hidden] bf16
    // source side
    const int *source_slots;
    std::uint32_t *out;                 // [T, hidden] bf16
    unsigned *done;
    unsigned *block_done;               // [world, nblk] records completed per block
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

// One thread, after the stores of record (src, slot) were ordered before it (warp or CTA
// barrier): count the record; whoever completes a block publishes it on the source rank.
__device__ __forceinline__ void complete_record(const CombineParams &p, int src, int slot, int count,
                                                std::uint64_t epoch) {
    const int blk = slot / p.block;
    const int expected = min(p.block, count - blk * p.block);
    unsigned *counter = p.block_done + src * p.nblk + blk;
    if (atom_add_acq_rel_gpu(counter, 1u) + 1 == static_cast<unsigned>(expected)) {
        st_relaxed_gpu(counter, 0u);
        std::uint64_t *flag = reinterpret_cast<std::uint64_t *>(p.peer_return_flags[src]) +
            static_cast<std::size_t>(p.g.rank) * (p.nblk + 1) + blk;
        aboleth::detail::st_release_sys(flag, epoch);
    }
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
    // Choices are packed to the front of a record by its sender; unused ones carry position -1.
    int my_row = -1;
    float my_gate = 0.f;
    if (lane < g.top_k) {
        const int pos = p.expert_pos[row * g.top_k + lane];
        const int id = p.expert_ids[row * g.top_k + lane];
        my_gate = p.expert_weights[row * g.top_k + lane];
        if (pos >= 0 && id >= 0 && id < g.experts)
            my_row = p.expert_offsets[src * g.experts + id] + pos;
    }
    const int n = __popc(__ballot_sync(kFull, my_row >= 0));
    // Four consecutive 512-byte pieces (2 KiB) of a row per pass, two rows in flight: long
    // contiguous reads keep DRAM pages open, eight 16-byte loads per lane hide the latency.
    constexpr int kPieces = 4;
    for (int base = 0; base < vecs; base += 32 * kPieces) {
        float acc[kPieces][8] = {};
        for (int j0 = 0; j0 < n; j0 += 2) {
            uint4 y[2][kPieces];
            float w[2];
#pragma unroll
            for (int r2 = 0; r2 < 2; ++r2) {
                const int r = __shfl_sync(kFull, my_row, (j0 + r2) & 31);
                w[r2] = __shfl_sync(kFull, my_gate, (j0 + r2) & 31);
                const bool live = j0 + r2 < n && r >= 0;
                if (!live)
                    w[r2] = 0.f;
                const std::uint32_t *row = p.expert_out + static_cast<std::size_t>(live ? r : 0) * (g.hidden / 2);
#pragma unroll
                for (int u = 0; u < kPieces; ++u) {
                    const int v = base + u * 32 + lane;
                    y[r2][u] = make_uint4(0, 0, 0, 0);
                    if (live && v < vecs)
                        y[r2][u] = aboleth::detail::ld_stream16(row + v * 4);
                }
            }
#pragma unroll
            for (int r2 = 0; r2 < 2; ++r2)
#pragma unroll
                for (int u = 0; u < kPieces; ++u)
                    add_bf16x8(acc[u], y[r2][u], w[r2]);
        }
#pragma unroll
        for (int u = 0; u < kPieces; ++u) {
            const int v = base + u * 32 + lane;
            if (v < vecs)
                aboleth::detail::st_stream16(dst + v * 16, pack_bf16x8(acc[u]));
        }
    }
}

// One warp reduces one token's partial rows over the ranks that hold one, once the blocks that
// hold them are published.  Returns false when a wait ran out (status recorded).
// Part `part` of `parts` of token `t`: a token's row is cut into parts that different warps reduce, so the
// chain of dependent loads behind the LAST records to arrive is a quarter as long.
__device__ __forceinline__ bool reduce_token_by_warp(const CombineParams &p, int t, std::uint64_t epoch, int part,
                                                     int parts) {
    const EpGeometry &g = p.g;
    const int lane = threadIdx.x & 31;
    const int vecs = g.hidden / 8;
    int slot = -1;
    if (lane < g.world)
        slot = p.source_slots[t * g.world + lane];
    bool ok = true;
    if (slot >= 0) {
        const Status s = aboleth::wait_signal_status(
            p.return_flags + static_cast<std::size_t>(lane) * (p.nblk + 1) + slot / p.block, epoch);
        if (s != Status::Ok) {
            ab::set_status(p.status, s, 0x2000 + lane);
            ok = false;
        }
    }
    if (__any_sync(kFull, !ok))
        return false;
    const unsigned live = __ballot_sync(kFull, slot >= 0);
    const std::uint32_t *my_src = p.returned +
        (static_cast<std::size_t>(lane < g.world ? lane : 0) * g.capacity + (slot < 0 ? 0 : slot)) * (g.hidden / 2);
    std::uint32_t *out = p.out + static_cast<std::size_t>(t) * (g.hidden / 2);
    // Two 16-byte vectors per lane from each of up to four sources are in flight together (eight loads per
    // lane): a token has five to six partials on eight ranks, so a group of 1 KiB costs two round trips to
    // memory instead of one per source.
    constexpr int kChunks = 2, kSources = 4;
    const int groups = (vecs + 32 * kChunks - 1) / (32 * kChunks);
    const int first = part * groups / parts * (32 * kChunks), last = (part + 1) * groups / parts * (32 * kChunks);
    for (int base = first; base < min(last, vecs); base += 32 * kChunks) {
        float acc[kChunks][8] = {};
        unsigned m = live;
        while (m) {
            uint4 r[kSources][kChunks];
#pragma unroll
            for (int q = 0; q < kSources; ++q) {
                const bool more = m != 0;
                // every lane takes part in the shuffle; an exhausted mask names lane 0 and loads nothing
                const int from = more ? __ffs(m) - 1 : 0;
                const std::uint32_t *y = reinterpret_cast<const std::uint32_t *>(
                    shfl_u64(reinterpret_cast<std::uint64_t>(my_src), from));
                m &= m - 1;
#pragma unroll
                for (int u = 0; u < kChunks; ++u) {
                    const int v = base + u * 32 + lane;
                    r[q][u] = make_uint4(0, 0, 0, 0);
                    if (v < vecs && more)
                        r[q][u] = aboleth::detail::ld_stream16(y + v * 4);
                }
            }
#pragma unroll
            for (int q = 0; q < kSources; ++q)
#pragma unroll
                for (int u = 0; u < kChunks; ++u)
                    add_bf16x8(acc[u], r[q][u], 1.0f);
        }
#pragma unroll
        for (int u = 0; u < kChunks; ++u) {
            const int v = base + u * 32 + lane;
            if (v < vecs)
                *reinterpret_cast<uint4 *>(out + v * 4) = pack_bf16x8(acc[u]);
        }
    }
    return true;
}

__global__ void __launch_bounds__(kThreads, 3) ep_combine_kernel(CombineParams p) {
    const EpGeometry &g = p.g;
    __shared__ int s_flag;
    __shared__ int s_rows[kMaxTopK];
    __shared__ float s_gate[kMaxTopK];
    __shared__ int s_count[kMaxWorld];
    __shared__ int s_src_row[kMaxWorld];
    __shared__ int s_nsrc;
    const int tid = threadIdx.x;
    const int lane = tid & 31;
    const int warp = tid >> 5;
    const std::uint64_t epoch = *p.epoch;
    const int vecs = g.hidden / 8;  // 16-byte vectors per bf16 row
    const bool tracer = blockIdx.x == 0 && tid == 0;
    stamp(p.trace, 0, tracer);

    // The record counts are read once: a peer may publish the next layer's counts as soon as this
    // rank has said that it finished sending.
    if (tid < g.world)
        s_count[tid] = static_cast<int>(ab::min64(p.recv_counts[tid], g.capacity));
    __syncthreads();
    // Records are visited round-robin over the source ranks, starting at rank + 1: at any moment
    // the warps of one rank write to every peer, and no two ranks start on the same peer.  (Walking
    // source 0, then source 1, ... makes all ranks converge on one receiver at a time.)
    int most = 0;
    for (int src = 0; src < g.world; ++src)
        most = max(most, s_count[src]);
    const int spread = most * g.world;
    const bool fused = p.phases == (kPhaseSend | kPhaseRecv);

    if (p.by_warp) {
        const int senders = fused ? p.send_warps : ((p.phases & kPhaseSend) ? kWarps : 0);
        if (warp < senders) {
            const int stride = gridDim.x * senders;
            // A sender warp serves ONE destination (warps are dealt round-robin over the destinations,
            // starting at rank + 1, so every link is busy all the time and the warps of the local
            // destination, which finish early, turn into reducers) and claims that destination's records
            // one at a time from a counter: warps that drew records with few expert rows take more, and
            // the warps of a destination end together.  (A fixed stride left the slowest warps 40 % behind
            // the first; one counter for all destinations made every warp wait on the link.)
            // (With fewer sender warps than destinations a warp serves several, one after the other.)
            for (int turn = (blockIdx.x * senders + warp) % g.world; turn < g.world; turn += stride) {
                const int src = (g.rank + 1 + turn) % g.world;
                for (;;) {
                    int slot = 0;
                    if (lane == 0)
                        slot = static_cast<int>(atomicAdd(p.done + kNextRecord + src, 1u));
                    slot = __shfl_sync(kFull, slot, 0);
                    if (slot >= s_count[src])
                        break;
                    return_row_by_warp(p, src * g.capacity + slot, src, slot);
                    __syncwarp();
                    if (lane == 0)
                        complete_record(p, src, slot, s_count[src], epoch);
                }
            }
            stamp(p.trace, 1, tracer);
            // This warp has sent everything it will send.
            unsigned old = 0;
            if (lane == 0)
                old = atom_add_acq_rel_gpu(p.done + kDoneSenders, 1u);
            old = __shfl_sync(kFull, old, 0);
            if (old + 1 == static_cast<unsigned>(stride)) {
                if (lane == 0)
                    st_relaxed_gpu(p.done + kDoneSenders, 0u);
                if (lane < g.world)
                    aboleth::detail::st_release_sys(
                        reinterpret_cast<std::uint64_t *>(p.peer_return_flags[lane]) +
                            static_cast<std::size_t>(g.rank) * (p.nblk + 1) + p.nblk, epoch);
            }
        }
        if (p.phases & kPhaseRecv) {
            // Tokens are handed out in order through one counter: the dedicated reducer warps start at
            // once, the sender warps join when they have nothing left to send.
            const int parts = min(4, (vecs + 63) / 64);
            for (;;) {
                int item = 0;
                if (lane == 0)
                    item = static_cast<int>(atomicAdd(p.done + kNextToken, 1u));
                item = __shfl_sync(kFull, item, 0);
                const int t = item / parts;
                if (t >= p.num_tokens || !reduce_token_by_warp(p, t, epoch, item - t * parts, parts))
                    break;
            }
        }
    } else {
        if (p.phases & kPhaseSend) {
            for (int i = blockIdx.x; i < spread; i += gridDim.x) {
                const int slot = i / g.world;
                const int src = (g.rank + 1 + (i - slot * g.world)) % g.world;
                if (slot >= s_count[src])
                    continue;  // the same for every thread of the CTA
                const int row = src * g.capacity + slot;
                int n = 1;
                if (p.weighted) {
                    // ids, positions and gates are fetched together (no look at the record's choice
                    // count first): unused choice slots carry position -1 and are skipped.
                    n = g.top_k;
                    if (tid < n) {
                        const int id = p.expert_ids[row * g.top_k + tid];
                        const int pos = p.expert_pos[row * g.top_k + tid];
                        s_gate[tid] = p.expert_weights[row * g.top_k + tid];
                        s_rows[tid] = (pos >= 0 && id >= 0 && id < g.experts)
                                          ? p.expert_offsets[src * g.experts + id] + pos : -1;
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
                        for (int j0 = 0; j0 < n; j0 += 8) {
                            uint4 y[8];
#pragma unroll
                            for (int u = 0; u < 8; ++u) {
                                y[u] = make_uint4(0, 0, 0, 0);
                                if (j0 + u < n && s_rows[j0 + u] >= 0)
                                    y[u] = aboleth::detail::ld_stream16(
                                        p.expert_out + static_cast<std::size_t>(s_rows[j0 + u]) * (g.hidden / 2) + v * 4);
                            }
#pragma unroll
                            for (int u = 0; u < 8; ++u)
                                if (j0 + u < n)
                                    add_bf16x8(acc, y[u], s_gate[j0 + u]);
                        }
                        o = pack_bf16x8(acc);
                    }
                    aboleth::detail::st_stream16(dst + v * 16, o);
                }
                __syncthreads();
                if (tid == 0)
                    complete_record(p, src, slot, s_count[src], epoch);
            }
            // This CTA has sent everything it will send.
            __syncthreads();
            if (tid == 0)
                s_flag = atom_add_acq_rel_gpu(p.done + kDoneSenders, 1u) == gridDim.x - 1 ? 1 : 0;
            __syncthreads();
            if (s_flag) {
                if (tid == 0)
                    st_relaxed_gpu(p.done + kDoneSenders, 0u);
                if (tid < g.world)
                    aboleth::detail::st_release_sys(
                        reinterpret_cast<std::uint64_t *>(p.peer_return_flags[tid]) +
                            static_cast<std::size_t>(g.rank) * (p.nblk + 1) + p.nblk, epoch);
            }
            stamp(p.trace, 1, tracer);
        }
        if (p.phases & kPhaseRecv) {
            for (int t = blockIdx.x; t < p.num_tokens; t += gridDim.x) {
                // Threads d < world wait for the block that holds this token's partial from rank d.
                if (tid == 0)
                    s_flag = 0;
                __syncthreads();
                if (tid < 32) {
                    // Lane d < world waits for the block that holds this token's partial from rank d;
                    // the rows that exist are listed for the reduction.
                    const int slot = tid < g.world ? p.source_slots[t * g.world + tid] : -1;
                    if (slot >= 0) {
                        const Status s = aboleth::wait_signal_status(
                            p.return_flags + static_cast<std::size_t>(tid) * (p.nblk + 1) + slot / p.block, epoch);
                        if (s != Status::Ok) {
                            ab::set_status(p.status, s, 0x2000 + tid);
                            s_flag = 1;
                        }
                    }
                    const unsigned have = __ballot_sync(kFull, slot >= 0);
                    if (slot >= 0)
                        s_src_row[__popc(have & ((1u << tid) - 1))] = tid * g.capacity + slot;
                    if (tid == 0)
                        s_nsrc = __popc(have);
                }
                __syncthreads();
                if (s_flag)
                    break;
                const int nsrc = s_nsrc;
                for (int v = tid; v < vecs; v += kThreads) {
                    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
                    for (int i0 = 0; i0 < nsrc; i0 += 4) {
                        uint4 r[4];
#pragma unroll
                        for (int u = 0; u < 4; ++u) {
                            r[u] = make_uint4(0, 0, 0, 0);
                            if (i0 + u < nsrc)
                                r[u] = aboleth::detail::ld_stream16(
                                    p.returned + static_cast<std::size_t>(s_src_row[i0 + u]) * (g.hidden / 2) + v * 4);
                        }
#pragma unroll
                        for (int u = 0; u < 4; ++u)
                            add_bf16x8(acc, r[u], 1.0f);
                    }
                    *reinterpret_cast<uint4 *>(p.out + static_cast<std::size_t>(t) * (g.hidden / 2) + v * 4) =
                        pack_bf16x8(acc);
                }
                __syncthreads();
            }
        }
    }

    if (p.phases & kPhaseRecv) {
        // Close the layer: the last CTA waits until every peer finished sending (its reads of this
        // layer's records are over), then advances the epoch for the next dispatch.
        __syncthreads();
        stamp(p.trace, 2, tracer);
        if (tid == 0)
            s_flag = atom_add_acq_rel_gpu(p.done + kDoneCombine, 1u) == gridDim.x - 1 ? 1 : 0;
        __syncthreads();
        if (s_flag) {
            stamp(p.trace, 3, tid == 0);
            const bool ok = wait_all_peers(p.return_flags + p.nblk, g.world, p.nblk + 1, epoch, p.status,
                                           &s_flag, 0x2100);
            if (tid == 0) {
                p.done[kDoneCombine] = 0;
                p.done[kNextToken] = 0;
                for (int d = 0; d < g.world; ++d)
                    p.done[kNextRecord + d] = 0;
                (void)ok;  // a timeout is in the status word; the epoch still advances
                *p.epoch = epoch + 1;
                stamp(p.trace, 4, true);
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

// counts [sources, experts] -> offsets [sources, experts]: the rows of expert e start at the
// exclusive scan of the experts' totals (each rounded up to `align`), and inside an expert's
// group the rows of source s follow those of the sources before it.  One CTA; experts <= 1024.
__global__ void __launch_bounds__(1024) expert_offsets_kernel(
    const int *counts, int *offsets, int *total, int sources, int experts, int align) {
    __shared__ int s[1024];
    const int e = threadIdx.x;
    int sum = 0;
    if (e < experts)
        for (int src = 0; src < sources; ++src)
            sum += counts[src * experts + e];
    int v = sum;
    if (align > 1)
        v = (v + align - 1) / align * align;
    s[e] = e < experts ? v : 0;
    __syncthreads();
    for (int off = 1; off < 1024; off <<= 1) {
        const int add = e >= off ? s[e - off] : 0;
        __syncthreads();
        s[e] += add;
        __syncthreads();
    }
    if (e < experts) {
        int at = s[e] - v;
        for (int src = 0; src < sources; ++src) {
            offsets[src * experts + e] = at;
            at += counts[src * experts + e];
        }
    }
    if (e == 0 && total != nullptr)
        *total = s[1023];
}

// Gather received rows into expert-contiguous order:
//   dst[offsets[id] + pos] = src[row]   for every live (row, choice).
// Also writes the inverse map perm_row[offsets[id] + pos] = row * k + j.
__global__ void __launch_bounds__(kThreads) permute_kernel(
    const std::uint8_t *src, std::uint8_t *dst, const float *src_scales, float *dst_scales,
    const int *expert_ids, const int *expert_pos, const int *offsets,
    const unsigned long long *recv_counts, int *perm_row, int world, int capacity, int top_k,
    int row_bytes, int cols, int src_scale_stride, int offset_stride) {
    const int total = world * capacity;
    for (int row = blockIdx.x; row < total; row += gridDim.x) {
        const int srcr = row / capacity;
        if (static_cast<unsigned long long>(row - srcr * capacity) >= recv_counts[srcr])
            continue;
        for (int j = 0; j < top_k; ++j) {
            const int pos = expert_pos[row * top_k + j];
            if (pos < 0)
                continue;
            const int out = offsets[srcr * offset_stride + expert_ids[row * top_k + j]] + pos;
            const uint4 *s = reinterpret_cast<const uint4 *>(src + static_cast<std::size_t>(row) * row_bytes);
            uint4 *d = reinterpret_cast<uint4 *>(dst + static_cast<std::size_t>(out) * row_bytes);
            for (int v = threadIdx.x; v < row_bytes / 16; v += kThreads)
                d[v] = s[v];
            if (src_scales != nullptr)
                for (int c = threadIdx.x; c < cols; c += kThreads)
                    dst_scales[static_cast<std::size_t>(out) * cols + c] =
                        src_scales[static_cast<std::size_t>(row) * src_scale_stride + c];
            if (threadIdx.x == 0 && perm_row != nullptr)
                perm_row[out] = row * top_k + j;
        }
    }
}

// out[row] = sum_j weights[row, j] * y[offsets[id] + pos]  (bf16, fp32 accumulate).
__global__ void __launch_bounds__(kThreads) unpermute_kernel(
    const std::uint32_t *y, std::uint32_t *out, const int *expert_ids, const int *expert_pos,
    const float *expert_weights, const int *offsets, const unsigned long long *recv_counts,
    int world, int capacity, int top_k, int hidden, int offset_stride) {
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
                    y + static_cast<std::size_t>(offsets[srcr * offset_stride + expert_ids[row * top_k + j]] + pos) *
                            (hidden / 2) + v * 4);
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

// The benchmark's stand-in expert f_e(x) = dequant(x) * (1 + (e mod 7) / 8)
// (reference oracle: experiments/dsl/moe/moe_common.py:72-140), in two forms:
//  * record layout (offsets == nullptr): y[row] = sum_j w_j * f_{id_j}(x[row]), gate applied
//    here, so the combine sums unweighted partials as the reference does;
//  * expert-contiguous layout (offsets given): y[offsets[id_j] + pos_j] = f_{id_j}(x[row]) for
//    every live choice, no gate: what a grouped expert GEMM would leave behind, so the combine
//    kernel gathers the rows and applies the gates itself.
__global__ void __launch_bounds__(kThreads) standin_expert_kernel(
    const std::uint8_t *payload, const float *scales, int scale_stride, std::uint32_t *y,
    const int *expert_ids, const float *expert_weights, const int *expert_pos, const int *offsets,
    const unsigned long long *recv_counts, int world, int capacity, int top_k, int hidden, int group,
    int value_fp8, int offset_stride) {
    const int total = world * capacity;
    __shared__ float s_coef[kMaxTopK];
    __shared__ int s_out[kMaxTopK];
    for (int row = blockIdx.x; row < total; row += gridDim.x) {
        const int srcr = row / capacity;
        if (static_cast<unsigned long long>(row - srcr * capacity) >= recv_counts[srcr])
            continue;
        int outputs = 1;
        __syncthreads();
        if (offsets == nullptr) {
            if (threadIdx.x == 0) {
                float coef = 0.f;
                for (int j = 0; j < top_k; ++j)
                    if (expert_pos[row * top_k + j] >= 0)
                        coef += expert_weights[row * top_k + j] *
                                (1.0f + static_cast<float>(expert_ids[row * top_k + j] % 7) * 0.125f);
                s_coef[0] = coef;
                s_out[0] = row;
            }
        } else {
            outputs = top_k;
            if (threadIdx.x < top_k) {
                const int id = expert_ids[row * top_k + threadIdx.x];
                const int pos = expert_pos[row * top_k + threadIdx.x];
                s_out[threadIdx.x] = pos >= 0 ? offsets[srcr * offset_stride + id] + pos : -1;
                s_coef[threadIdx.x] = 1.0f + static_cast<float>(id % 7) * 0.125f;
            }
        }
        __syncthreads();
        for (int v = threadIdx.x; v < hidden / 8; v += kThreads) {
            float f[8];
            if (value_fp8) {
                const uint2 q = *reinterpret_cast<const uint2 *>(payload + static_cast<std::size_t>(row) * hidden + v * 8);
                const float s = scales[static_cast<std::size_t>(row) * scale_stride + (v * 8) / group];
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
            for (int j = 0; j < outputs; ++j) {
                if (s_out[j] < 0)
                    continue;
                const float coef = s_coef[j];
                uint4 o;
                o.x = pack_bf16x2(f[0] * coef, f[1] * coef);
                o.y = pack_bf16x2(f[2] * coef, f[3] * coef);
                o.z = pack_bf16x2(f[4] * coef, f[5] * coef);
                o.w = pack_bf16x2(f[6] * coef, f[7] * coef);
                *reinterpret_cast<uint4 *>(y + static_cast<std::size_t>(s_out[j]) * (hidden / 2) + v * 4) = o;
            }
        }
    }
}

// The dispatch kernel's CTAs meet at one grid barrier (token-ordered slots), and the combine
// kernel's reducer warps wait for sender warps of other ranks: every CTA of the grid must be
// resident at once, so the grid is clamped to what the device holds.
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

// CTAs of the last dispatch (0) / combine (1) launch made by the calling host thread.
static thread_local int g_last_grid[2] = {0, 0};
AB_EXPORT int ab_ep_last_grid(int which) { return which == 0 || which == 1 ? g_last_grid[which] : -1; }

// Argument blocks are passed as arrays of 64-bit words so the Python side needs
// no struct mirror: ints[] carries the integer geometry, ptrs[] the addresses.
//   ints: 0 rank, 1 world, 2 experts, 3 top_k, 4 hidden, 5 scale_group, 6 capacity, 7 value_fp8,
//         8 round_scale, 9 (unused), 10 num_tokens, 11 routing, 12 renormalize, 13 phases,
//         14 weighted, 15 by_warp, 16 block, 17 send_warps, 18 block_count_rows
AB_EXPORT int ab_ep_dispatch(const int *ints, float amax_floor, const std::uint64_t *ptrs,
                             int grid, cudaStream_t stream) {
    DispatchParams p{};
    p.g = EpGeometry{ints[0], ints[1], ints[2], ints[3], ints[4], ints[5], ints[6],
                     ints[7], ints[8], amax_floor};
    p.num_tokens = ints[10];
    p.routing = ints[11];
    p.renormalize = ints[12];
    p.phases = ints[13];
    p.by_warp = ints[15];
    if (!geometry_ok(p.g) || p.num_tokens < 0 || p.num_tokens > p.g.capacity || grid < 0)
        return -1;
    const int resident = p.by_warp ? resident_grid(ep_dispatch_kernel<true>, 1 << 30)
                                   : resident_grid(ep_dispatch_kernel<false>, 1 << 30);
    if (grid == 0) {
        if (p.by_warp) {
            // Every SM gets the same number of CTAs and every CTA the same number of tokens (one
            // per warp at most while the device has room): the slowest SM sets the time.
            int per_cta = (p.num_tokens + resident - 1) / (resident > 0 ? resident : 1);
            per_cta = per_cta < 1 ? 1 : per_cta;
            grid = (p.num_tokens + per_cta - 1) / per_cta;
        } else {
            grid = p.num_tokens;  // one CTA per token
        }
    }
    if (grid < 1 || !(p.phases & kPhaseSend))
        grid = 1;
    grid = grid < resident ? grid : resident;
    if (p.by_warp && grid > ints[18])
        grid = ints[18];  // rows of block_counts
    if (grid < 1)
        return -1;
    int i = 0;
    p.x = reinterpret_cast<const std::uint32_t *>(ptrs[i++]);
    p.logits = reinterpret_cast<const float *>(ptrs[i++]);
    p.ids_in = reinterpret_cast<const int *>(ptrs[i++]);
    p.weights_in = reinterpret_cast<const float *>(ptrs[i++]);
    p.ids_out = reinterpret_cast<int *>(ptrs[i++]);
    p.weights_out = reinterpret_cast<float *>(ptrs[i++]);
    p.owners = reinterpret_cast<const int *>(ptrs[i++]);
    p.placeholders = reinterpret_cast<const int *>(ptrs[i++]);
    p.source_slots = reinterpret_cast<int *>(ptrs[i++]);
    p.send_counts = reinterpret_cast<unsigned long long *>(ptrs[i++]);
    p.done = reinterpret_cast<unsigned *>(ptrs[i++]);
    p.overflow = reinterpret_cast<int *>(ptrs[i++]);
    p.epoch = reinterpret_cast<const unsigned long long *>(ptrs[i++]);
    p.status = reinterpret_cast<unsigned long long *>(ptrs[i++]);
    p.block_counts = reinterpret_cast<int *>(ptrs[i++]);
    p.peer_payload = reinterpret_cast<const std::uint64_t *>(ptrs[i++]);
    p.peer_meta = reinterpret_cast<const std::uint64_t *>(ptrs[i++]);
    p.peer_counts = reinterpret_cast<const std::uint64_t *>(ptrs[i++]);
    p.peer_flags = reinterpret_cast<const std::uint64_t *>(ptrs[i++]);
    p.peer_ids = reinterpret_cast<const std::uint64_t *>(ptrs[i++]);
    p.peer_weights = reinterpret_cast<const std::uint64_t *>(ptrs[i++]);
    p.peer_pos = reinterpret_cast<const std::uint64_t *>(ptrs[i++]);
    p.peer_expert_counts = reinterpret_cast<const std::uint64_t *>(ptrs[i++]);
    p.send_expert_counts = reinterpret_cast<int *>(ptrs[i++]);
    p.recv_counts = reinterpret_cast<const unsigned long long *>(ptrs[i++]);
    p.flags = reinterpret_cast<const std::uint64_t *>(ptrs[i++]);
    p.recv_expert_counts = reinterpret_cast<const int *>(ptrs[i++]);
    p.expert_counts = reinterpret_cast<int *>(ptrs[i++]);
    p.trace = reinterpret_cast<unsigned long long *>(ptrs[i++]);
    if (p.num_tokens > 0) {  // an empty batch may come with null (empty) tensors
        if (p.routing == 1 && (p.ids_out == nullptr || p.weights_out == nullptr || p.logits == nullptr))
            return -1;
        if (p.routing != 1 && (p.ids_in == nullptr || p.weights_in == nullptr))
            return -1;
    }
    g_last_grid[0] = grid;
    if (p.by_warp)
        ep_dispatch_kernel<true><<<grid, kThreads, 0, stream>>>(p);
    else
        ep_dispatch_kernel<false><<<grid, kThreads, 0, stream>>>(p);
    return ab::launch_result("ep_dispatch");
}

AB_EXPORT int ab_ep_combine(const int *ints, float amax_floor, const std::uint64_t *ptrs, int grid,
                            cudaStream_t stream) {
    CombineParams p{};
    p.g = EpGeometry{ints[0], ints[1], ints[2], ints[3], ints[4], ints[5], ints[6],
                     ints[7], ints[8], amax_floor};
    p.num_tokens = ints[10];
    p.phases = ints[13];
    p.weighted = ints[14];
    p.by_warp = ints[15];
    p.block = ints[16];
    p.send_warps = ints[17];
    if (!geometry_ok(p.g) || p.num_tokens < 0 || p.num_tokens > p.g.capacity || grid < 0 ||
        p.block < 1)
        return -1;
    p.nblk = (p.g.capacity + p.block - 1) / p.block;
    if (p.send_warps < 1 || p.send_warps >= kWarps)
        p.send_warps = kWarps - 2;
    if (grid == 0) {
        // by warp: fill the device; by CTA: one CTA per record the tokens can have produced.
        const int fan = p.g.world < p.g.top_k ? p.g.world : p.g.top_k;
        grid = p.by_warp ? 1 << 20 : (p.num_tokens * fan < 1 ? 1 : p.num_tokens * fan);
    }
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
    p.block_done = reinterpret_cast<unsigned *>(ptrs[i++]);
    p.epoch = reinterpret_cast<unsigned long long *>(ptrs[i++]);
    p.status = reinterpret_cast<unsigned long long *>(ptrs[i++]);
    p.trace = reinterpret_cast<unsigned long long *>(ptrs[i++]);
    if (p.weighted && p.expert_offsets == nullptr)
        return -1;
    g_last_grid[1] = resident_grid(ep_combine_kernel, grid);
    ep_combine_kernel<<<g_last_grid[1], kThreads, 0, stream>>>(p);
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

AB_EXPORT int ab_expert_offsets(const int *counts, int *offsets, int *total, int sources, int experts,
                                int align, cudaStream_t stream) {
    if (experts < 1 || experts > 1024 || sources < 1)
        return -1;
    expert_offsets_kernel<<<1, 1024, 0, stream>>>(counts, offsets, total, sources, experts, align);
    return ab::launch_result("expert_offsets");
}

AB_EXPORT int ab_permute(const void *src, void *dst, const float *src_scales, float *dst_scales,
                         const int *expert_ids, const int *expert_pos, const int *offsets,
                         const unsigned long long *recv_counts, int *perm_row, int world,
                         int capacity, int top_k, int row_bytes, int cols, int src_scale_stride,
                         int offset_stride, cudaStream_t stream) {
    if (row_bytes % 16 || world < 1 || capacity < 1)
        return -1;
    const int total = world * capacity;
    const int grid = total < 148 * 8 ? total : 148 * 8;
    permute_kernel<<<grid, kThreads, 0, stream>>>(
        static_cast<const std::uint8_t *>(src), static_cast<std::uint8_t *>(dst), src_scales,
        dst_scales, expert_ids, expert_pos, offsets, recv_counts, perm_row, world, capacity, top_k,
        row_bytes, cols, src_scale_stride > 0 ? src_scale_stride : cols, offset_stride);
    return ab::launch_result("permute");
}

AB_EXPORT int ab_unpermute(const void *y, void *out, const int *expert_ids, const int *expert_pos,
                           const float *expert_weights, const int *offsets,
                           const unsigned long long *recv_counts, int world, int capacity, int top_k,
                           int hidden, int offset_stride, cudaStream_t stream) {
    if (hidden % 8 || world < 1 || capacity < 1)
        return -1;
    const int total = world * capacity;
    const int grid = total < 148 * 8 ? total : 148 * 8;
    unpermute_kernel<<<grid, kThreads, 0, stream>>>(
        static_cast<const std::uint32_t *>(y), static_cast<std::uint32_t *>(out), expert_ids,
        expert_pos, expert_weights, offsets, recv_counts, world, capacity, top_k, hidden, offset_stride);
    return ab::launch_result("unpermute");
}

AB_EXPORT int ab_standin_expert(const void *payload, const float *scales, int scale_stride, void *y,
                                const int *expert_ids, const float *expert_weights,
                                const int *expert_pos, const int *offsets,
                                const unsigned long long *recv_counts, int world, int capacity,
                                int top_k, int hidden, int group, int value_fp8, int offset_stride,
                                cudaStream_t stream) {
    if (hidden % 8 || world < 1 || capacity < 1 || top_k < 1 || top_k > kMaxTopK)
        return -1;
    const int total = world * capacity;
    const int grid = total < 148 * 8 ? total : 148 * 8;
    standin_expert_kernel<<<grid, kThreads, 0, stream>>>(
        static_cast<const std::uint8_t *>(payload), scales,
        scale_stride > 0 ? scale_stride : hidden / group, static_cast<std::uint32_t *>(y),
        expert_ids, expert_weights, expert_pos, offsets, recv_counts, world, capacity, top_k, hidden,
        group, value_fp8, offset_stride);
    return ab::launch_result("standin_expert");
}
