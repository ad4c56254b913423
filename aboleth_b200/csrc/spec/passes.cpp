// Scheduling passes of the Tier-2 specializer (order and contracts: passes.hpp).
//
// Each pass restates, on this project's text IR, the analysis of the reference
// pass of the same name:
//   materialize-valid-extents   compiler/lib/Transforms/MaterializeValidExtents.cpp:11-65
//   materialize-completion      .../MaterializeCompletion.cpp:27-237
//   forward-inline-payloads     .../ForwardInlinePayloads.cpp:90-395
//   plan-publication            .../PlanPublication.cpp:21-66
//   form-batches                .../FormBatches.cpp:26-233
//   coalesce-submissions        .../CoalesceSubmissions.cpp:23-145
//   order-publications          .../OrderPublications.cpp:22-82
//   elide-epochs                .../ElideEpochs.cpp:22-174
//   defer-announcement          .../DeferAnnouncement.cpp:19-53
//   order-producers             .../OrderProducers.cpp:22-114
//   analyze-issuers             .../AnalyzeIssuers.cpp:30-310
#include "passes.hpp"

#include <algorithm>
#include <cctype>
#include <functional>

namespace spec {

namespace {

using Block = std::vector<Op>;

std::string endpoint_of(const Op &op) { return op.operands.empty() ? "" : op.operands[0]; }

unsigned bit_floor(unsigned v) {
    unsigned k = 1;
    while (k * 2 <= v && k * 2 != 0)
        k *= 2;
    return v == 0 ? 0 : k;
}

// Definition of a value visible from a block: search enclosing definitions.
struct Defs {
    std::map<std::string, const Op *> map;
    void collect(const Block &ops) {
        for (const auto &op : ops) {
            if (!op.result.empty())
                map[op.result] = &op;
            collect(op.body);
        }
    }
    const Op *find(const std::string &name) const {
        auto it = map.find(name);
        return it == map.end() ? nullptr : it->second;
    }
};

bool communicates(const Op &op) {
    static const std::set<std::string> kinds = {
        "put", "put_inline", "signal", "wait", "planned_wait", "wait_signal", "drain",
        "begin_group", "wait_group", "system_fence", "publish_head", "post_put", "post_inline",
        "post_signal", "post_nop", "submit", "poll"};
    return kinds.count(op.kind) != 0;
}

bool contains_if(const Block &ops, const std::function<bool(const Op &)> &pred) {
    bool found = false;
    walk(ops, [&](const Op &op) { found = found || pred(op); });
    return found;
}

// May a submission be placed after `op` although a chain member precedes it?
// Pure ops, bindings, loads and stores, and structured control flow made of
// those may be crossed; other chains' commands too.
bool crossable(const Op &op) {
    static const std::set<std::string> plain = {"endpoint", "local", "remote", "remote_at", "let", "load",
                                                "store", "tensor_store", "compute"};
    if (plain.count(op.kind) || is_command(op) || is_posted(op))
        return true;
    if (op.kind == "stmt")
        return true;  // frontend loads, arithmetic and stores
    if (op.kind == "for" || op.kind == "if")
        return !contains_if(op.body, [](const Op &o) { return !crossable(o) || communicates(o); });
    return false;
}

}  // namespace

Options parse_options(const std::string &text) {
    Options o;
    std::istringstream in(text);
    std::string tok;
    while (in >> tok) {
        const std::size_t eq = tok.find('=');
        const std::string key = tok.substr(0, eq);
        const std::string value = eq == std::string::npos ? "" : tok.substr(eq + 1);
        if (key == "backend")
            o.backend = value;
        else if (key == "enable") {
            std::size_t start = 0;
            while (start <= value.size()) {
                const std::size_t comma = value.find(',', start);
                const std::string name = value.substr(start, comma == std::string::npos ? comma : comma - start);
                if (!name.empty())
                    o.enabled.insert(name);
                if (comma == std::string::npos)
                    break;
                start = comma + 1;
            }
        } else if (key == "inline_bytes")
            o.inline_bytes = static_cast<unsigned>(std::stoul(value));
        else if (key == "queue_capacity")
            o.queue_capacity = static_cast<unsigned>(std::stoul(value));
        else if (key == "completion_interval")
            o.completion_interval = static_cast<unsigned>(std::stoul(value));
        else if (key == "strict_registrations")
            o.strict_registrations = value == "1";
        else if (key == "coop_min")
            o.coop_min = static_cast<unsigned>(std::stoul(value));
        else if (key == "coop_elements")
            o.coop_elements = static_cast<unsigned>(std::stoul(value));
        else if (key == "p2p_scalar")
            o.p2p_scalar = value == "1";
        else if (key == "stop_after")
            o.stop_after = value;
        else
            throw Error("unknown specializer option '" + key + "'");
    }
    o.caps = aboleth::abi::lookup_transport_caps(o.backend.c_str());
    if (o.caps == nullptr)
        throw Error("unknown transport '" + o.backend + "'");
    if (o.coop_elements < 32 || o.coop_elements > 4096 || (o.coop_elements & (o.coop_elements - 1)))
        throw Error("coop_elements must be a power of two in [32, 4096]");
    return o;
}

// ---- materialize-valid-extents ------------------------------------------------------------

int materialize_valid_extents(Program &p, const Options &o) {
    Defs defs;
    defs.collect(p.body);
    int changed = 0;
    walk(p.body, [&](Op &op) {
        if (op.kind != "put" || op.operands.size() != 3)
            return;
        const Op *src = defs.find(op.operands[2]);
        if (src == nullptr || src->kind != "local" || !src->has("valid") || op.has("extent"))
            return;
        // valid=<count>,<capacity>,<item_bytes>; `at` is the byte offset of the view.
        const std::string v = src->get("valid");
        const std::size_t c1 = v.find(','), c2 = v.find(',', c1 + 1);
        const std::string count = v.substr(0, c1), capacity = v.substr(c1 + 1, c2 - c1 - 1),
                          item = v.substr(c2 + 1), at = src->get("at", "0");
        // Counts are normalised to [0, capacity] either way.  With the switch on the
        // transfer is clamped to what remains of the valid prefix (64-bit math until
        // the final 32-bit length); with it off the padding travels too.
        const std::string fn = o.on("valid-extents") ? "ab_valid_bytes" : "ab_checked_bytes";
        op.attrs["bytes"] = fn + "(" + op.get("bytes") + "," + count + "," + capacity + "," + item +
                            "," + at + ")";
        op.attrs["extent"] = o.on("valid-extents") ? "trimmed" : "capacity";
        ++changed;
    });
    return changed;
}

// ---- materialize-completion ----------------------------------------------------------------

int materialize_completion(Program &p, const Options &o) {
    int changed = 0;
    Defs defs;
    defs.collect(p.body);
    for_each_block(p.body, [&](Block &block) {
        for (Op &op : block) {
            if (op.kind != "planned_wait")
                continue;
            const Op *token = defs.find(op.operands[0]);
            const std::string endpoint = token ? endpoint_of(*token) : "";
            // Every planned chain on this endpoint in this block counts against the queue.
            unsigned slots = 0;
            for (const Op &other : block)
                if ((is_command(other) || is_posted(other)) && endpoint_of(other) == endpoint)
                    ++slots;
            slots = std::max(slots, 1u);
            unsigned k = 1;
            if (o.on("completion-planning")) {
                // A wait spliced from a transport plan carries the plan's resolved interval (and
                // the smallest peer queue) instead of a reuse distance.
                unsigned bound = static_cast<unsigned>(
                    std::max(1ll, to_integer(op.has("reuse") ? op.get("reuse") : op.get("interval"))));
                const unsigned prefer = o.completion_interval ? o.completion_interval
                                                              : o.caps->default_completion_interval;
                if (prefer)
                    bound = std::min(bound, prefer);
                unsigned capacity = o.queue_capacity;
                if (op.has("queue_capacity") && is_integer(op.get("queue_capacity"))) {
                    const unsigned planned = static_cast<unsigned>(std::max(0ll, to_integer(op.get("queue_capacity"))));
                    capacity = capacity ? std::min(capacity, planned) : planned;
                }
                if (o.caps->queue_capacity_limited && capacity > 1)
                    bound = std::max(1u, std::min(bound, (capacity - 1) / slots));
                k = std::max(bit_floor(bound), 1u);
            }
            const std::string iter = op.get("iteration");
            std::string pred = k == 1 ? "1"
                                      : "(((" + iter + ") & " + std::to_string(k - 1) + ") == " +
                                            std::to_string(k - 1) + ")";
            if (k != 1 && op.has("final") && !op.get("final").empty())
                pred = "(" + pred + " || (" + op.get("final") + "))";
            op.kind = "wait";
            op.attrs.erase("reuse");
            op.attrs.erase("queue_capacity");
            op.attrs.erase("final");
            op.attrs["pred"] = pred;
            op.attrs["interval"] = std::to_string(k);
            op.attrs["planned"] = iter;
            op.attrs.erase("iteration");
            ++changed;
        }
    });
    return changed;
}

// ---- forward-inline-payloads ----------------------------------------------------------------

int forward_inline_payloads(Program &p, const Options &o) {
    if (!o.on("forward-inline-payloads") ||
        !(o.backend == "rdma" || o.backend == "p2p" || o.backend == "ionic"))
        return 0;
    int changed = 0;
    // How often is each staging base mentioned anywhere?  A base that anything
    // besides its stores and its one `local` can reach is left alone.
    std::map<std::string, int> mentions;
    walk(p.body, [&](const Op &op) {
        for (const auto &operand : op.operands)
            ++mentions[strip_parens(operand)];
    });
    for_each_block(p.body, [&](Block &block) {
        for (std::size_t i = 0; i < block.size(); ++i) {
            Op &put = block[i];
            if (put.kind != "put" || !is_integer(put.get("bytes")) || put.has("extent"))
                continue;
            const long long bytes = to_integer(put.get("bytes"));
            if (bytes <= 0 || bytes > static_cast<long long>(o.inline_bytes))
                continue;
            // Source must be a `local` in this block whose base is an identifiable name.
            std::size_t li = block.size();
            for (std::size_t j = 0; j < i; ++j)
                if (block[j].result == put.operands[2] && block[j].kind == "local")
                    li = j;
            if (li == block.size() || block[li].has("valid") || block[li].operands.size() != 1)
                continue;
            const std::string base = strip_parens(block[li].operands[0]);
            // Collect the scalar stores to `base` that precede the put.
            std::vector<std::size_t> stores;
            bool legal = true;
            std::size_t first = i;
            for (std::size_t j = 0; j < i; ++j)
                if (block[j].kind == "store" && strip_parens(block[j].operands[0]) == base) {
                    stores.push_back(j);
                    first = std::min(first, j);
                }
            if (stores.empty())
                continue;
            for (std::size_t j = first; j < i && legal; ++j) {
                const Op &between = block[j];
                const bool mine = between.kind == "store" && strip_parens(between.operands[0]) == base;
                if (mine || j == li)
                    continue;
                static const std::set<std::string> harmless = {"local", "remote", "endpoint", "let",
                                                               "load", "store", "compute"};
                legal = harmless.count(between.kind) != 0;
            }
            if (!legal || mentions[base] != static_cast<int>(stores.size()) + 1)
                continue;
            // The stores must tile [0, bytes) exactly, each at a constant offset.
            std::vector<std::pair<long long, std::size_t>> by_offset;
            for (std::size_t j : stores) {
                if (!is_integer(block[j].get("offset", "0")) || !is_integer(block[j].get("width"))) {
                    legal = false;
                    break;
                }
                by_offset.emplace_back(to_integer(block[j].get("offset", "0")), j);
            }
            if (!legal)
                continue;
            std::sort(by_offset.begin(), by_offset.end());
            long long cursor = 0;
            std::string values;
            for (const auto &entry : by_offset) {
                const Op &st = block[entry.second];
                const long long width = to_integer(st.get("width"));
                if (entry.first != cursor || width % 8 != 0) {
                    legal = false;
                    break;
                }
                if (!values.empty())
                    values += ",";
                values += st.get("value") + ":" + std::to_string(width);
                cursor += width / 8;
            }
            if (!legal || cursor != bytes)
                continue;
            put.kind = "put_inline";
            put.operands.pop_back();
            put.attrs.erase("bytes");
            put.attrs["values"] = values;
            put.attrs["forwarded"] = std::to_string(bytes);
            // Delete the stores and the now unused `local`, back to front.
            std::vector<std::size_t> dead = stores;
            dead.push_back(li);
            std::sort(dead.rbegin(), dead.rend());
            for (std::size_t j : dead)
                block.erase(block.begin() + static_cast<long>(j));
            i -= dead.size();
            ++changed;
        }
    });
    return changed;
}

// ---- plan-publication --------------------------------------------------------------------------

int plan_publication(Program &p, const Options &o) {
    using aboleth::abi::TransportPublicationMode;
    static const char *names[] = {"SameQueueStrong", "P2PRelease", "GinSignal",
                                  "FenceThenSignal", "ImmCounting", "SameQueueFencedWrite"};
    int changed = 0;
    walk(p.body, [&](Op &op) {
        if (op.kind != "signal" || op.has("expected") || op.has("weak") || op.has("strong"))
            return;
        const bool standalone = !op.has("after") && !op.has("group");
        if (standalone && o.on("plan-publication")) {
            op.attrs["weak"] = "";
        } else {
            op.attrs["strong"] = "";
            const TransportPublicationMode mode = aboleth::abi::legal_strong_publication(
                *o.caps, /*prefer_imm=*/false,
                o.on("plan-publication") && o.strict_registrations);
            op.attrs["mode"] = names[static_cast<int>(mode)];
        }
        ++changed;
    });
    return changed;
}

// ---- form-batches ---------------------------------------------------------------------------------

int form_batches(Program &p, const Options &) {
    int batches = 0;
    for_each_block(p.body, [&](Block &block) {
        // successor map: which command names `x` as its `after`
        std::map<std::string, std::size_t> index;
        std::set<std::string> has_successor;
        for (std::size_t i = 0; i < block.size(); ++i)
            if (is_command(block[i])) {
                index[block[i].result] = i;
                if (block[i].has("after") && index.count(block[i].get("after")))
                    has_successor.insert(block[i].get("after"));
            }
        if (index.empty())
            return;
        struct Batch {
            std::vector<std::string> tokens;
            std::size_t place_after;  // index (in the original block) the submit follows
            std::string name;
        };
        std::vector<Batch> formed;
        std::map<std::string, std::string> token_batch;
        for (std::size_t i = 0; i < block.size(); ++i) {
            const Op &tail = block[i];
            if (!is_command(tail) || has_successor.count(tail.result))
                continue;
            // Walk the `after` chain back from the tail.
            std::vector<std::size_t> members = {i};
            std::string cursor = tail.get("after");
            while (!cursor.empty() && index.count(cursor) &&
                   endpoint_of(block[index[cursor]]) == endpoint_of(tail)) {
                members.push_back(index[cursor]);
                cursor = block[index[cursor]].get("after");
            }
            std::reverse(members.begin(), members.end());
            // Cut the chain where something between two members may not be crossed.
            std::vector<std::vector<std::size_t>> pieces(1);
            for (std::size_t m = 0; m < members.size(); ++m) {
                if (m > 0) {
                    bool ok = true;
                    for (std::size_t j = members[m - 1] + 1; j < members[m]; ++j)
                        ok = ok && crossable(block[j]);
                    if (!ok)
                        pieces.emplace_back();
                }
                pieces.back().push_back(members[m]);
            }
            for (const auto &piece : pieces) {
                Batch b;
                for (std::size_t m : piece)
                    b.tokens.push_back(block[m].result);
                b.place_after = piece.back();
                b.name = "%b" + std::to_string(batches++);
                for (const auto &t : b.tokens)
                    token_batch[t] = b.name;
                formed.push_back(b);
            }
        }
        // Rewrite in place, then insert submits back to front.
        for (Op &op : block) {
            if (op.kind == "put")
                op.kind = "post_put";
            else if (op.kind == "put_inline")
                op.kind = "post_inline";
            else if (op.kind == "signal")
                op.kind = "post_signal";
            else if (op.kind == "wait" && token_batch.count(op.operands[0])) {
                op.kind = "poll";
                op.operands[0] = token_batch[op.operands[0]];
            }
        }
        std::sort(formed.begin(), formed.end(),
                  [](const Batch &a, const Batch &b) { return a.place_after > b.place_after; });
        for (const Batch &b : formed) {
            Op submit;
            submit.kind = "submit";
            submit.result = b.name;
            submit.operands = b.tokens;
            submit.attrs["batch"] = std::to_string(b.tokens.size());
            submit.line = block[b.place_after].line;
            block.insert(block.begin() + static_cast<long>(b.place_after) + 1, submit);
        }
    });
    // Waits on tokens defined in an enclosing block.
    Defs defs;
    defs.collect(p.body);
    std::map<std::string, std::string> owner;
    walk(p.body, [&](const Op &op) {
        if (op.kind == "submit")
            for (const auto &t : op.operands)
                owner[t] = op.result;
    });
    walk(p.body, [&](Op &op) {
        if (op.kind == "wait" && owner.count(op.operands[0])) {
            op.kind = "poll";
            op.operands[0] = owner[op.operands[0]];
        }
    });
    return batches;
}

// ---- coalesce-submissions ------------------------------------------------------------------------

namespace {

std::string submit_endpoint(const Block &block, const Op &submit) {
    for (const Op &op : block)
        if (op.result == submit.operands[0])
            return endpoint_of(op);
    return "";
}

std::string flag_signature(const Op &submit) {
    std::string sig;
    for (const auto &kv : submit.attrs)
        if (kv.first != "batch" && kv.first != "segments")
            sig += kv.first + "=" + kv.second + ";";
    return sig;
}

}  // namespace

int coalesce_submissions(Program &p, const Options &o) {
    if (!o.on("coalesce-submissions") || o.caps->load_store_addressable)
        return 0;
    int merged = 0;
    for_each_block(p.body, [&](Block &block) {
        bool again = true;
        while (again) {
            again = false;
            for (std::size_t i = 0; i < block.size() && !again; ++i) {
                if (block[i].kind != "submit")
                    continue;
                for (std::size_t j = i + 1; j < block.size(); ++j) {
                    const Op &between = block[j];
                    if (between.kind == "submit") {
                        Op &first = block[i];
                        Op &second = block[j];
                        if (submit_endpoint(block, first) != submit_endpoint(block, second) ||
                            flag_signature(first) != flag_signature(second))
                            break;
                        // Poll predicates must agree (both absent counts as agreeing).
                        auto poll_pred = [&](const Op &s) {
                            for (const Op &op : block)
                                if (op.kind == "poll" && op.operands[0] == s.result)
                                    return op.get("pred", "1");
                            return std::string("<none>");
                        };
                        if (poll_pred(first) != poll_pred(second))
                            break;
                        const std::string gone = first.result;
                        const std::size_t first_count = first.operands.size();
                        std::vector<std::string> tokens = first.operands;
                        tokens.insert(tokens.end(), second.operands.begin(), second.operands.end());
                        second.operands = tokens;
                        second.attrs["batch"] = std::to_string(tokens.size());
                        const std::string prior = first.get("segments", std::to_string(first_count));
                        second.attrs["segments"] =
                            prior + "+" + second.get("segments", std::to_string(tokens.size() - first_count));
                        const std::string kept = second.result;
                        block.erase(block.begin() + static_cast<long>(i));
                        // Retarget polls; a second poll of the same batch is redundant.
                        bool seen = false;
                        for (std::size_t k = 0; k < block.size();) {
                            Op &op = block[k];
                            if (op.kind == "poll" && (op.operands[0] == gone || op.operands[0] == kept)) {
                                op.operands[0] = kept;
                                if (seen) {
                                    block.erase(block.begin() + static_cast<long>(k));
                                    continue;
                                }
                                seen = true;
                            }
                            ++k;
                        }
                        // The surviving poll must come after the surviving submit.
                        ++merged;
                        again = true;
                        break;
                    }
                    if (!(is_posted(between) || crossable(between)))
                        break;
                }
            }
        }
        // A poll that now precedes its submit moves right behind it.
        for (std::size_t i = 0; i < block.size(); ++i) {
            if (block[i].kind != "poll")
                continue;
            for (std::size_t j = i + 1; j < block.size(); ++j)
                if (block[j].kind == "submit" && block[j].result == block[i].operands[0]) {
                    Op poll = block[i];
                    block.erase(block.begin() + static_cast<long>(i));
                    block.insert(block.begin() + static_cast<long>(j), poll);
                    break;
                }
        }
    });
    return merged;
}

// ---- order-publications ---------------------------------------------------------------------------

int order_publications(Program &p, const Options &o) {
    if (!o.on("order-publications") || o.caps->load_store_addressable)
        return 0;
    int changed = 0;
    for_each_block(p.body, [&](Block &block) {
        for (Op &submit : block) {
            if (submit.kind != "submit" || !submit.has("segments"))
                continue;
            std::map<std::string, Op *> by_name;
            for (Op &op : block)
                if (is_posted(op))
                    by_name[op.result] = &op;
            std::vector<std::string> payload, signals;
            for (const auto &t : submit.operands)
                (by_name[t]->kind == "post_signal" ? signals : payload).push_back(t);
            if (signals.size() < 2)
                continue;
            // Payload first; strong signals chained so only the first orders.
            bool first_strong = true;
            std::string previous;
            for (const auto &t : signals) {
                Op *s = by_name[t];
                if (!s->has("strong"))
                    continue;
                if (first_strong) {
                    s->attrs["ordering_point"] = "";
                    first_strong = false;
                } else {
                    s->attrs["chained"] = previous;
                }
                previous = t;
            }
            payload.insert(payload.end(), signals.begin(), signals.end());
            submit.operands = payload;
            submit.attrs["publicationsOrdered"] = "1";
            ++changed;
        }
    });
    return changed;
}

// ---- elide-epochs ------------------------------------------------------------------------------------

// `expr` with every occurrence of the identifier `var` replaced by `(value)`.
static std::string substitute_identifier(const std::string &expr, const std::string &var,
                                         const std::string &value) {
    std::string out;
    for (std::size_t at = 0; at < expr.size();) {
        const bool start = std::isalpha(static_cast<unsigned char>(expr[at])) || expr[at] == '_';
        if (!start) {
            out += expr[at++];
            continue;
        }
        std::size_t end = at;
        while (end < expr.size() && (std::isalnum(static_cast<unsigned char>(expr[end])) || expr[end] == '_'))
            ++end;
        const std::string word = expr.substr(at, end - at);
        out += word == var ? "(" + value + ")" : word;
        at = end;
    }
    return out;
}

// In a counted loop whose completion is polled only every k-th iteration, a signal published on
// those iterations (and on the last) delivers every payload no later than the completion already
// does; the other iterations' ordering points are dropped.  Receivers that wait for "at least
// epoch e" see the same epochs, only later.  A CHECKED publication (compare-and-swap against the
// epoch before it) then has to compare against the epoch LAST PUBLISHED rather than epoch - 1:
// that value is carried through the loop in a variable set up in front of it and advanced whenever
// the signal is published (reference: compiler/lib/Transforms/ElideEpochs.cpp:110-174, where the
// value rides on an scf.for iteration argument).  A signal with an explicit `expected` is left
// alone; so is a kernel that itself waits on a peer.
int elide_epochs(Program &p, const Options &o) {
    if (!o.on("elide-epochs") || o.caps->load_store_addressable)
        return 0;
    if (contains_if(p.body, [](const Op &op) { return op.kind == "wait_signal"; }))
        return 0;  // a kernel that waits on peers must not skip what they wait for
    int changed = 0, carried = 0;
    for_each_block(p.body, [&](Block &block) {
        for (std::size_t at = 0; at < block.size(); ++at) {
            if (block[at].kind != "for" || block[at].operands.size() != 3)
                continue;
            std::vector<Op> setups;
            {
                Op &loop = block[at];
                // A planned poll in the loop body gives the predicate.
                std::string pred;
                for (const Op &op : loop.body)
                    if (op.kind == "poll" && op.has("planned") && op.get("pred") != "1")
                        pred = op.get("pred");
                if (pred.empty())
                    continue;
                const std::string last = "((" + loop.operands[0] + ") == (" + loop.operands[2] + ") - 1)";
                const std::string due = "(" + pred + " || " + last + ")";
                for (std::size_t j = 0; j < loop.body.size(); ++j) {
                    if (loop.body[j].kind != "post_signal" || loop.body[j].has("pred") ||
                        loop.body[j].has("expected"))
                        continue;
                    loop.body[j].attrs["pred"] = due;
                    loop.body[j].attrs["elided"] = "";
                    ++changed;
                    if (loop.body[j].get("mode") != "SameQueueStrong")
                        continue;
                    // Checked: the epoch in the cell is the one this loop published last.
                    const std::string name = "ab_published_" + std::to_string(carried++);
                    const std::string epoch = loop.body[j].get("epoch");
                    loop.body[j].attrs["expected"] = name;
                    Op setup;
                    setup.kind = "stmt";
                    setup.line = loop.line;
                    setup.operands = {"\"long long " + name + " = (" +
                                      substitute_identifier(epoch, loop.operands[0], loop.operands[1]) +
                                      ") - 1; (void)" + name + ";\""};
                    setups.push_back(setup);
                    Op advance;
                    advance.kind = "stmt";
                    advance.line = loop.body[j].line;
                    advance.operands = {"\"if " + due + " " + name + " = (" + epoch + ");\""};
                    // The value advances after the submission that carries the signal has read it.
                    std::size_t where = j + 1;
                    for (std::size_t k = j + 1; k < loop.body.size(); ++k)
                        if (loop.body[k].kind == "submit" &&
                            std::find(loop.body[k].operands.begin(), loop.body[k].operands.end(),
                                      loop.body[j].result) != loop.body[k].operands.end()) {
                            where = k + 1;
                            break;
                        }
                    loop.body.insert(loop.body.begin() + where, advance);
                }
            }
            block.insert(block.begin() + at, setups.begin(), setups.end());
            at += setups.size();
        }
    });
    return changed;
}

// ---- defer-announcement -----------------------------------------------------------------------------

int defer_announcement(Program &p, const Options &o) {
    using aboleth::abi::TransportDoorbellModel;
    if (!o.on("defer-announcement") || o.caps->doorbell_model == TransportDoorbellModel::None)
        return 0;
    if (contains_if(p.body, [](const Op &op) { return op.kind == "wait_signal"; }))
        return 0;
    int changed = 0;
    for_each_block(p.body, [&](Block &block) {
        for (Op &submit : block) {
            if (submit.kind != "submit")
                continue;
            for (const Op &op : block)
                if (op.kind == "poll" && op.operands[0] == submit.result && op.has("planned") &&
                    op.get("pred") != "1") {
                    submit.attrs["deferredAnnouncement"] = "";
                    submit.attrs["poll_predicate"] = op.get("pred");
                    ++changed;
                }
        }
    });
    return changed;
}

// ---- self-reclaim ----------------------------------------------------------------------------------
//
// wait(token, predicate=p) with a predicate the USER wrote defers completion without a bound the
// planner knows (docs of the reference, COMPILER_SEMANTICS.md:344-359): the submission is marked
// selfReclaim (a producer that finds the queue full retires completions itself instead of assuming
// the planned window) and the kernel has to retire what it deferred - it must end, on that endpoint,
// with an unconditional completion or a drain.  Queue transports only; on peer memory completion is
// vacuous.
int mark_self_reclaim(Program &p, const Options &o) {
    if (o.caps->load_store_addressable)
        return 0;
    Defs defs;
    defs.collect(p.body);
    int changed = 0;
    // Endpoint of each user-predicated poll, and where it was seen (for the diagnostic).
    std::map<std::string, int> deferred;
    const auto endpoint_of_token = [&](const std::string &token) -> std::string {
        const Op *def = defs.find(token);
        if (def == nullptr)
            return "";
        if (def->kind == "submit" && !def->operands.empty())
            if (const Op *cmd = defs.find(def->operands[0]))
                return cmd->operands.empty() ? "" : cmd->operands[0];
        return def->operands.empty() ? "" : def->operands[0];
    };
    // Program order, outermost blocks flattened: a later unconditional completion or drain retires.
    std::function<void(Block &)> scan = [&](Block &block) {
        for (Op &op : block) {
            if ((op.kind == "poll" || op.kind == "wait") && !op.operands.empty()) {
                const std::string ep = endpoint_of_token(op.operands[0]);
                const bool user = op.has("pred") && op.get("pred") != "1" && !op.has("planned");
                if (user) {
                    deferred[ep] = op.line;
                    if (o.on("self-reclaim"))
                        for (Op &other : block)
                            if (other.kind == "submit" && other.result == op.operands[0] &&
                                !other.has("selfReclaim")) {
                                other.attrs["selfReclaim"] = "";
                                ++changed;
                            }
                } else if (!op.has("pred") || op.get("pred") == "1") {
                    deferred.erase(ep);
                }
            } else if (op.kind == "drain" && !op.operands.empty()) {
                deferred.erase(op.operands[0]);
            }
            if (!op.body.empty())
                scan(op.body);
        }
    };
    scan(p.body);
    if (!deferred.empty())
        throw Error("line " + std::to_string(deferred.begin()->second) +
                    ": wait: a completion deferred by a user-written predicate is never retired on " +
                    deferred.begin()->first + ": end the kernel with an unconditional wait or drain(" +
                    deferred.begin()->first + ")");
    return changed;
}

// ---- order-producers ---------------------------------------------------------------------------------

namespace {

// Returns the dirty state after the block; marks submits that need a barrier.
bool scan_producers(Block &block, bool dirty, const Defs &defs, int &marked) {
    for (Op &op : block) {
        if (op.kind == "tensor_store" || (op.kind == "stmt" && op.has("unknown_write"))) {
            dirty = true;
        } else if (op.kind == "barrier") {
            dirty = false;
        } else if (op.kind == "submit") {
            bool reads_region = false;
            for (const auto &t : op.operands) {
                const Op *cmd = defs.find(t);
                reads_region = reads_region || (cmd && cmd->kind == "post_put");
            }
            if (reads_region && dirty) {
                if (!op.has("producerBarrier")) {
                    op.attrs["producerBarrier"] = "";
                    ++marked;
                }
                dirty = false;
            }
        } else if (op.kind == "for") {
            const bool out = scan_producers(op.body, dirty, defs, marked);
            if (out && !dirty)  // the second iteration starts dirty
                scan_producers(op.body, true, defs, marked);
            dirty = dirty || out;
        } else if (op.kind == "if") {
            dirty = scan_producers(op.body, dirty, defs, marked) || dirty;
        }
    }
    return dirty;
}

}  // namespace

int order_producers(Program &p, const Options &) {
    Defs defs;
    defs.collect(p.body);
    int marked = 0;
    scan_producers(p.body, false, defs, marked);
    return marked;
}

// ---- analyze-issuers -----------------------------------------------------------------------------------

namespace {

struct Lexer {
    std::string s;
    std::size_t at = 0;
    std::string peek() {
        const std::size_t save = at;
        std::string t = next();
        at = save;
        return t;
    }
    std::string next() {
        while (at < s.size() && std::isspace(static_cast<unsigned char>(s[at])))
            ++at;
        if (at >= s.size())
            return "";
        if (std::isalnum(static_cast<unsigned char>(s[at])) || s[at] == '_' || s[at] == '.') {
            std::size_t b = at;
            while (at < s.size() && (std::isalnum(static_cast<unsigned char>(s[at])) || s[at] == '_' || s[at] == '.'))
                ++at;
            return s.substr(b, at - b);
        }
        if (at + 1 < s.size() && (s.substr(at, 2) == ">=" || s.substr(at, 2) == "<=" ||
                                  s.substr(at, 2) == "==" || s.substr(at, 2) == "!=")) {
            at += 2;
            return s.substr(at - 2, 2);
        }
        return std::string(1, s[at++]);
    }
};

// value = scale * pid + uniform, or unknown.
struct Lin {
    bool known = true;
    long long scale = 0;
    bool constant = false;  // uniform part is a literal
    long long literal = 0;
    bool modular = false;
    long long modulus = 0;
};

struct AffineParser {
    Lexer lex;
    const std::map<std::string, std::string> &lets;
    int depth = 0;

    Lin unknown() { Lin l; l.known = false; return l; }

    Lin primary() {
        const std::string t = lex.next();
        if (t == "(") {
            Lin v = sum();
            if (lex.next() != ")")
                return unknown();
            return v;
        }
        if (t.empty())
            return unknown();
        if (is_integer(t)) {
            Lin l;
            l.constant = true;
            l.literal = to_integer(t);
            return l;
        }
        if (t == "pid" || t == "blockIdx.x") {
            Lin l;
            l.scale = 1;
            l.constant = true;
            return l;
        }
        auto it = lets.find(t);
        if (it != lets.end() && depth < 8) {
            AffineParser inner{Lexer{it->second}, lets, depth + 1};
            Lin v = inner.sum();
            return inner.lex.peek().empty() ? v : unknown();
        }
        if (std::isalpha(static_cast<unsigned char>(t[0])) || t[0] == '_') {
            Lin l;  // a kernel argument or constant: uniform across programs
            return l;
        }
        return unknown();
    }

    Lin product() {
        Lin v = primary();
        while (true) {
            const std::string op = lex.peek();
            if (op == "*") {
                lex.next();
                Lin r = primary();
                if (!v.known || !r.known || v.modular || r.modular)
                    return unknown();
                if (v.scale != 0 && r.scale != 0)
                    return unknown();
                if (v.scale != 0) {
                    if (!r.constant)
                        return unknown();  // pid * uniform-but-unknown: may be zero
                    v.scale *= r.literal;
                    v.literal *= r.literal;
                } else if (r.scale != 0) {
                    if (!v.constant)
                        return unknown();
                    r.scale *= v.literal;
                    r.literal *= v.literal;
                    v = r;
                } else {
                    v.constant = v.constant && r.constant;
                    v.literal *= r.literal;
                }
            } else if (op == "%") {
                lex.next();
                Lin r = primary();
                if (!v.known || !r.known || r.scale != 0 || !r.constant || v.modular)
                    return unknown();
                if (v.scale == 1 || v.scale == -1) {
                    v.modular = true;
                    v.modulus = r.literal;
                } else if (v.scale != 0) {
                    return unknown();
                }
            } else if (op == "/" || op == ">=" || op == "<=" || op == "<" || op == ">" ||
                       op == "==" || op == "!=" || op == "?" || op == "&" || op == "|") {
                return unknown();  // not affine in the program id
            } else {
                return v;
            }
        }
    }

    Lin sum() {
        Lin v = product();
        while (true) {
            const std::string op = lex.peek();
            if (op != "+" && op != "-")
                return v;
            lex.next();
            Lin r = product();
            if (!v.known || !r.known)
                return unknown();
            if ((v.modular && r.scale != 0) || (r.modular && v.scale != 0) || (v.modular && r.modular))
                return unknown();
            const long long sign = op == "+" ? 1 : -1;
            v.scale += sign * r.scale;
            v.constant = v.constant && r.constant;
            v.literal += sign * r.literal;
            if (r.modular) {
                v.modular = true;
                v.modulus = r.modulus;
            }
        }
    }
};

}  // namespace

Affine affine_in_pid(const std::string &expr, const std::map<std::string, std::string> &lets) {
    AffineParser parser{Lexer{strip_parens(expr)}, lets};
    Lin v = parser.sum();
    Affine a;
    if (!v.known || !parser.lex.peek().empty())
        return a;
    a.known = true;
    a.scale = v.scale;
    a.modular = v.modular;
    a.modulus = v.modulus;
    return a;
}

int analyze_issuers(Program &p, const Options &o) {
    if (!o.on("analyze-issuers"))
        return 0;
    std::map<std::string, std::string> lets;
    walk(p.body, [&](const Op &op) {
        if (op.kind == "let" && op.operands.size() == 2)
            lets[op.operands[0]] = op.operands[1];
    });
    std::set<std::string> exclusive;
    int changed = 0;
    const std::string grid = p.get("grid");
    walk(p.body, [&](Op &op) {
        if (op.kind != "endpoint" || op.operands.size() != 2)
            return;
        const Affine a = affine_in_pid(op.operands[1], lets);
        if (!a.known || a.scale == 0)
            return;
        if (a.modular) {
            // (pid + c) % N is injective only while the grid is no larger than N.
            if (!is_integer(grid) || to_integer(grid) > a.modulus)
                return;
            op.attrs["exclusiveGridShape"] = std::to_string(a.modulus);
        }
        op.attrs["exclusiveAxis"] = "0";
        exclusive.insert(op.result);
        ++changed;
    });
    if (exclusive.empty())
        return 0;
    Defs defs;
    defs.collect(p.body);
    walk(p.body, [&](Op &op) {
        if (op.kind == "submit") {
            const Op *cmd = defs.find(op.operands[0]);
            if (cmd && exclusive.count(endpoint_of(*cmd)))
                op.attrs["exclusiveIssuer"] = "";
        } else if (op.kind == "drain" && !op.operands.empty() && exclusive.count(op.operands[0])) {
            op.attrs["exclusiveIssuer"] = "";
        }
    });
    return changed;
}

}  // namespace spec
