// Lowerings of Queue IR to CUDA C++ for sm_100a: peer memory (p2p) and the
// host-proxy ring (proxy; also serves the rdma / efa / ionic names here).
//
// p2p follows the reference's lowering decisions
// (compiler/lib/Target/P2P/LowerP2P.cpp:311-346,453-490,550-591,610-647):
//   * a put is a predicated copy, cooperative over the CTA when large enough;
//   * after the copies of a submission comes one CTA barrier - and a system
//     fence ONLY when no strong signal in that submission publishes them;
//   * a strong signal is one release store at system scope, a weak signal a
//     relaxed store; wait_signal is an acquire spin (bounded here);
//   * submit, poll, groups, drain, system_fence, publish_head lower to nothing.
// proxy follows compiler/lib/Target/Proxy/LowerProxy.cpp:74-403: one sequence
// reservation per batch, one 32-byte command per posted op, one release store
// of ready_sequence, polls as bounded acquire loads of completed_sequence.
#include <algorithm>

#include "passes.hpp"

namespace spec {

namespace {

std::string ident(const std::string &value) {
    std::string out = value;
    if (!out.empty() && out[0] == '%')
        out = "v_" + out.substr(1);
    return out;
}

std::string ctype(const std::string &type) {
    if (type == "ptr" || type == "u64")
        return "unsigned long long";
    if (type == "table")
        return "const unsigned long long *";
    if (type == "i32")
        return "int";
    if (type == "i64")
        return "long long";
    if (type == "f32")
        return "float";
    throw Error("unknown argument type '" + type + "'");
}

struct BatchInfo {
    const Op *submit = nullptr;
    bool has_put = false;
    bool has_strong = false;
    std::string first_put, last_put;
};

struct Emitter {
    const Program &program;
    const Options &options;
    std::ostringstream out;
    std::map<std::string, BatchInfo> batch_of;  // token -> its batch
    std::map<std::string, const Op *> defs;
    // facts
    int batches = 0, commands = 0, reservations = 0, ready_stores = 0, completion_waits = 0;
    int barriers = 0, producer_barriers = 0, system_fences = 0, inline_puts = 0, trimmed = 0;
    int deferred_placements = 0;
    int weak = 0, strong = 0, elided = 0, exclusive = 0, cooperative_puts = 0;
    std::vector<std::string> fences, flag_writes, flag_reads;
    int wait_sites = 0;

    Emitter(const Program &p, const Options &o) : program(p), options(o) {
        collect(p.body);
    }

    void collect(const std::vector<Op> &ops) {
        for (const Op &op : ops) {
            if (!op.result.empty())
                defs[op.result] = &op;
            collect(op.body);
        }
        for (const Op &op : ops) {
            if (op.kind != "submit")
                continue;
            BatchInfo info;
            info.submit = &op;
            for (const auto &t : op.operands) {
                const Op *cmd = defs.count(t) ? defs[t] : nullptr;
                if (cmd == nullptr)
                    continue;
                if (cmd->kind == "post_put") {
                    info.has_put = true;
                    if (info.first_put.empty())
                        info.first_put = t;
                    info.last_put = t;
                }
                if (cmd->kind == "post_signal" && cmd->has("strong"))
                    info.has_strong = true;
            }
            for (const auto &t : op.operands)
                batch_of[t] = info;
        }
    }

    void line(int indent, const std::string &text) {
        out << std::string(static_cast<std::size_t>(indent) * 4, ' ') << text << "\n";
    }

    std::string pred_of(const Op &op) const { return op.get("pred", ""); }

    void open_pred(int &indent, const Op &op) {
        if (!pred_of(op).empty()) {
            line(indent, "if (" + pred_of(op) + ") {");
            ++indent;
        }
    }
    void close_pred(int &indent, const Op &op) {
        if (!pred_of(op).empty()) {
            --indent;
            line(indent, "}");
        }
    }

    void prologue(const std::string &backend_note) {
        line(0, "// Emitted by the aboleth_b200 Tier-2 specializer.  Program '" + program.name +
                    "', transport " + options.backend + backend_note + ".");
        line(0, "#include \"aboleth/tier2.cuh\"");
        line(0, "");
        std::string args;
        for (const Arg &arg : program.args)
            args += ctype(arg.type) + " " + arg.name + ", ";
        line(0, "extern \"C\" __global__ void " + program.name + "(" + args +
                    "unsigned long long *ab_status) {");
        line(1, "using namespace aboleth;");
        line(1, "const long long pid = blockIdx.x;");
        line(1, "(void)pid;");
        for (const char *key : {"rank", "world"})
            if (!program.get(key).empty()) {
                std::string upper = key;
                std::transform(upper.begin(), upper.end(), upper.begin(), ::toupper);
                line(1, "constexpr long long " + upper + " = " + program.get(key) + ";");
                line(1, "(void)" + upper + ";");
            }
    }

    void bindings(const Op &op, int indent) {
        if (op.kind == "let") {
            line(indent, "const long long " + op.operands[0] + " = " + op.operands[1] + ";");
        } else if (op.kind == "endpoint") {
            // Load the handle and strip the kind bits (low three).
            line(indent, "const unsigned long long " + ident(op.result) + " = " + op.operands[0] + "[" +
                             op.operands[1] + "] & ~7ull;");
            line(indent, "(void)" + ident(op.result) + ";");
        } else if (op.kind == "local") {
            line(indent, "const unsigned long long " + ident(op.result) + " = (unsigned long long)(" +
                             op.operands[0] + ") + (" + op.get("at", "0") + ");");
            line(indent, "const unsigned " + ident(op.result) + "_key = " + op.get("key", "0") + ";");
            line(indent, "(void)" + ident(op.result) + "_key;");
        } else if (op.kind == "remote") {
            // (address, key) pairs, rank-major.
            line(indent, "const unsigned long long " + ident(op.result) + " = " + op.operands[0] + "[2 * (" +
                             op.operands[1] + ")] + (" + op.get("offset", "0") + ");");
            line(indent, "const unsigned " + ident(op.result) + "_key = (unsigned)" + op.operands[0] +
                             "[2 * (" + op.operands[1] + ") + 1];");
            line(indent, "(void)" + ident(op.result) + "_key;");
        } else if (op.kind == "remote_at") {
            line(indent, "const unsigned long long " + ident(op.result) + " = (unsigned long long)(" +
                             op.operands[0] + ");");
            line(indent, "const unsigned " + ident(op.result) + "_key = " + op.get("key", "0") + ";");
            line(indent, "(void)" + ident(op.result) + "_key;");
        }
    }

    bool frontend(const Op &op, int indent) {
        if (op.kind == "store") {
            const std::string width = op.get("width", "64");
            line(indent, "if (threadIdx.x == 0) t2::store_inline<std::uint" + width +
                             "_t>((unsigned long long)(" + op.operands[0] + ") + " + op.get("offset", "0") +
                             ", (unsigned long long)(" + op.get("value", "0") + "));");
            return true;
        }
        if (op.kind == "tensor_store" || op.kind == "load" || op.kind == "compute") {
            line(indent, "// " + op.kind + (op.operands.empty() ? "" : " " + op.operands[0]));
            return true;
        }
        if (op.kind == "stmt") {
            std::string code;
            for (const auto &tok : op.operands)
                code += (code.empty() ? "" : " ") + tok;
            if (code.size() >= 2 && code.front() == '"' && code.back() == '"')
                code = code.substr(1, code.size() - 2);
            line(indent, code);
            return true;
        }
        if (op.kind == "barrier") {
            line(indent, "__syncthreads();");
            ++barriers;
            fences.push_back("bar.sync");
            return true;
        }
        return false;
    }

    void inline_values(const Op &op, int indent, const std::string &dst) {
        const std::string values = op.get("values");
        std::size_t start = 0;
        int depth = 0;
        long long offset = 0;
        for (std::size_t i = 0; i <= values.size(); ++i) {
            if (i < values.size() && values[i] == '(')
                ++depth;
            if (i < values.size() && values[i] == ')')
                --depth;
            if (i == values.size() || (values[i] == ',' && depth == 0)) {
                const std::string item = values.substr(start, i - start);
                const std::size_t colon = item.rfind(':');
                const long long bits = std::stoll(item.substr(colon + 1));
                const std::string expr = item.substr(0, colon);
                const std::string at = dst + " + " + std::to_string(offset);
                if (bits == 24)
                    line(indent, "t2::store_inline24(" + at + ", (unsigned long long)(" + expr + "));");
                else
                    line(indent, "t2::store_inline<std::uint" + std::to_string(bits) + "_t>(" + at +
                                     ", (unsigned long long)(" + expr + "));");
                offset += bits / 8;
                start = i + 1;
            }
        }
    }

    std::string facts_json(const std::string &completion) const {
        Json j;
        j.begin_object();
        j.key("backend").value(options.backend);
        j.key("batches").value(batches);
        j.key("commands").value(commands);
        j.key("reservations").value(reservations);
        j.key("ready_stores").value(ready_stores);
        j.key("completion_waits").value(completion_waits);
        j.key("completion").value(completion);
        j.key("barriers").value(barriers);
        j.key("producer_barriers").value(producer_barriers);
        j.key("system_fences").value(system_fences);
        j.key("deferred_placements").value(deferred_placements);
        j.key("cooperative_puts").value(cooperative_puts);
        j.key("inline_puts").value(inline_puts);
        j.key("trimmed_puts").value(trimmed);
        j.key("weak_signals").value(weak);
        j.key("strong_signals").value(strong);
        j.key("elided_signals").value(elided);
        j.key("exclusive_issuers").value(exclusive);
        j.key("fences").begin_array();
        for (const auto &f : fences)
            j.value(f);
        j.end_array();
        j.key("flag_writes").begin_array();
        for (const auto &f : flag_writes)
            j.value(f);
        j.end_array();
        j.key("flag_reads").begin_array();
        for (const auto &f : flag_reads)
            j.value(f);
        j.end_array();
        j.end_object();
        return j.str();
    }
};

// ---- p2p -------------------------------------------------------------------------------------

struct P2PEmitter : Emitter {
    using Emitter::Emitter;

    // All commands of a batch are lowered where the batch is submitted, in
    // token order: one producer barrier (if the analysis asked for it), the
    // copies, then one CTA barrier before the first strong signal - or, when
    // nothing in the batch publishes the copies, a barrier and a system fence.
    // Copies of an earlier submission that no barrier has ordered yet (see `placed_later`).
    bool deferred_copies = false;

    // Does a later submission of the same block place this one's copies?  True when only bindings,
    // plain stores and other commands lie between, nothing polls this submission, and the next
    // submission with an effect either releases a strong, unpredicated signal (its CTA barrier and
    // release cover every earlier store of the CTA) or ends in its own barrier and system fence.
    // Nothing promised the copies any earlier: no signal of this submission names them and no
    // completion of it is awaited.  Part of coalesce-submissions (the peer-memory form of it).
    bool placed_later(const std::vector<Op> &ops, std::size_t at) const {
        if (!options.on("coalesce-submissions"))
            return false;
        static const std::set<std::string> plain = {"endpoint", "local", "remote", "remote_at", "let", "load",
                                                    "store", "tensor_store", "compute"};
        for (std::size_t j = at + 1; j < ops.size(); ++j) {
            const Op &next = ops[j];
            if (next.kind == "poll" || next.kind == "wait") {
                if (next.operands[0] == ops[at].result)
                    return false;
                continue;
            }
            if (plain.count(next.kind) || is_posted(next))
                continue;
            if (next.kind != "submit")
                return false;
            bool copies = false, strong = false, conditional = false;
            for (const auto &token : next.operands) {
                const Op &cmd = *defs.at(token);
                copies = copies || cmd.kind == "post_put";
                if (cmd.kind == "post_signal" && cmd.has("strong")) {
                    strong = true;
                    conditional = conditional || cmd.has("pred");
                }
            }
            if (strong)
                return !conditional;
            if (copies && !placed_later(ops, j))
                return true;  // ends in a barrier and a system fence of its own
            // Otherwise that submission defers as well: keep looking for the placing one.
        }
        return false;
    }

    void emit_submit(const Op &submit, int in, bool defer_placement = false) {
        ++batches;
        if (submit.has("exclusiveIssuer"))
            ++exclusive;
        line(in, "// submit " + submit.result + ": " + submit.get("batch") +
                     " command(s); peer memory has no queue, nothing to reserve or ring");
        if (submit.has("producerBarrier")) {
            line(in, "__syncthreads();  // producer barrier: a source was written by other threads");
            ++barriers;
            ++producer_barriers;
            fences.push_back("bar.sync(producer)");
        }
        bool copies_pending = false;  // copies since the last CTA barrier
        for (const auto &token : submit.operands) {
            const Op &op = *defs.at(token);
            int level = in;
            ++commands;
            if (op.kind == "post_put") {
                if (op.get("extent") == "trimmed")
                    ++trimmed;
                const std::string bytes = op.get("bytes");
                // Chunk: the smallest power of two of 8-byte elements covering a constant size.
                unsigned elements = options.coop_elements;
                if (is_integer(bytes)) {
                    unsigned need = 32;
                    while (need < elements && static_cast<long long>(need) * 8 < to_integer(bytes))
                        need *= 2;
                    elements = need;
                }
                if (!options.p2p_scalar && (!is_integer(bytes) || to_integer(bytes) >= options.coop_min))
                    ++cooperative_puts;
                open_pred(level, op);
                line(level, "t2::put_p2p<" + std::to_string(elements) + ">(" + ident(op.operands[1]) + ", " +
                                ident(op.operands[2]) + ", (std::uint32_t)(" + t2(bytes) + "), " +
                                std::to_string(options.coop_min) + "u, " +
                                (options.p2p_scalar ? "true" : "false") + ");");
                close_pred(level, op);
                copies_pending = true;
            } else if (op.kind == "post_inline") {
                ++inline_puts;
                open_pred(level, op);
                line(level, "if (threadIdx.x == 0) {");
                inline_values(op, level + 1, ident(op.operands[1]));
                line(level, "}");
                close_pred(level, op);
            } else if (op.kind == "post_signal") {
                if (op.has("elided"))
                    ++elided;
                const bool is_strong = op.has("strong");
                (is_strong ? strong : weak) += 1;
                if (is_strong && (copies_pending || deferred_copies)) {
                    deferred_copies = false;
                    line(level, "__syncthreads();  // every thread's copy precedes the release; no membar.sys");
                    ++barriers;
                    fences.push_back("bar.sync");
                    copies_pending = false;
                }
                open_pred(level, op);
                if (is_strong) {
                    line(level, "if (threadIdx.x == 0) detail::st_release_sys((std::uint64_t *)" +
                                    ident(op.operands[1]) + ", (std::uint64_t)(" + op.get("epoch") + "));");
                    fences.push_back("st.release.sys");
                    flag_writes.push_back("release.sys:" + op.get("epoch"));
                } else {
                    line(level, "if (threadIdx.x == 0) detail::st_relaxed_sys((std::uint64_t *)" +
                                    ident(op.operands[1]) + ", (std::uint64_t)(" + op.get("epoch") + "));");
                    flag_writes.push_back("relaxed.sys:" + op.get("epoch"));
                }
                close_pred(level, op);
            }
        }
        if (copies_pending && defer_placement) {
            line(in, "// no signal follows here: the next submission's barrier and release / fence place these copies");
            deferred_copies = true;
            ++deferred_placements;
        } else if (copies_pending || deferred_copies) {
            // Nothing in this submission publishes the copies: place them now.
            deferred_copies = false;
            line(in, "__syncthreads();");
            line(in, "if (threadIdx.x == 0) detail::fence_acq_rel_sys();  // no signal follows: membar.sys");
            ++barriers;
            ++system_fences;
            fences.push_back("bar.sync");
            fences.push_back("membar.sys");
        }
    }

    void emit_block(const std::vector<Op> &ops, int indent) {
        for (std::size_t at = 0; at < ops.size(); ++at) {
            const Op &op = ops[at];
            if (op.kind == "for") {
                line(indent, "for (long long " + op.operands[0] + " = " + op.operands[1] + "; " +
                                 op.operands[0] + " < " + op.operands[2] + "; ++" + op.operands[0] + ") {");
                emit_block(op.body, indent + 1);
                line(indent, "}");
                continue;
            }
            if (op.kind == "if") {
                line(indent, "if (" + op.operands[0] + ") {");
                emit_block(op.body, indent + 1);
                line(indent, "}");
                continue;
            }
            bindings(op, indent);
            if (frontend(op, indent))
                continue;
            int in = indent;
            if (is_posted(op)) {
                // The transfer is asynchronous: it is carried out where its batch is submitted.
                line(in, "// " + op.kind + " " + op.result + ": carried out at its submission");
            } else if (op.kind == "submit") {
                emit_submit(op, in, placed_later(ops, at));
            } else if (op.kind == "poll" || op.kind == "wait") {
                line(in, "// completion of " + op.operands[0] + ": program order (vacuous on peer memory)");
            } else if (op.kind == "wait_signal") {
                line(in, "t2::wait_signal_cta((unsigned long long)(" + op.operands[0] + "), (std::uint64_t)(" +
                             op.operands[1] + "), ab_status, " + std::to_string(0x5000 + wait_sites++) + ");");
                flag_reads.push_back("acquire.sys>=" + op.operands[1]);
                fences.push_back("ld.acquire.sys");
            } else if (op.kind == "begin_group" || op.kind == "wait_group" || op.kind == "drain" ||
                       op.kind == "system_fence" || op.kind == "publish_head") {
                line(in, "// " + op.kind + ": nothing on peer memory");
            } else if (op.kind == "put" || op.kind == "put_inline" || op.kind == "signal" ||
                       op.kind == "planned_wait") {
                throw Error("line " + std::to_string(op.line) + ": '" + op.kind +
                            "' survived to the lowering; run form-batches first");
            }
        }
    }

    static std::string t2(const std::string &bytes) {
        if (bytes.rfind("ab_valid_bytes", 0) == 0 || bytes.rfind("ab_checked_bytes", 0) == 0)
            return "t2::" + bytes;
        return bytes;
    }
};

// ---- proxy ring --------------------------------------------------------------------------------

struct ProxyEmitter : Emitter {
    using Emitter::Emitter;

    std::string endpoint_of_batch(const Op &submit) const {
        auto it = defs.find(submit.operands[0]);
        return it == defs.end() ? "" : ident(it->second->operands[0]);
    }

    void emit_block(const std::vector<Op> &ops, int indent) {
        for (const Op &op : ops) {
            if (op.kind == "for") {
                line(indent, "for (long long " + op.operands[0] + " = " + op.operands[1] + "; " +
                                 op.operands[0] + " < " + op.operands[2] + "; ++" + op.operands[0] + ") {");
                emit_block(op.body, indent + 1);
                line(indent, "}");
                continue;
            }
            if (op.kind == "if") {
                line(indent, "if (" + op.operands[0] + ") {");
                emit_block(op.body, indent + 1);
                line(indent, "}");
                continue;
            }
            bindings(op, indent);
            if (frontend(op, indent))
                continue;
            if (is_posted(op)) {
                line(indent, "// " + op.kind + " " + op.result + ": written into its batch at the submission");
                continue;
            }
            if (op.kind == "submit") {
                ++batches;
                ++reservations;
                ++ready_stores;
                if (op.has("exclusiveIssuer"))
                    ++exclusive;
                if (op.has("producerBarrier")) {
                    line(indent, "__syncthreads();  // producer barrier");
                    ++barriers;
                    ++producer_barriers;
                    fences.push_back("bar.sync(producer)");
                }
                const std::string seq = "seq_" + ident(op.result);
                line(indent, "std::uint64_t " + seq + " = 0;");
                line(indent, "if (threadIdx.x == 0) {");
                line(indent + 1, "// one reservation, " + op.get("batch") + " command(s), one release store of ready_sequence");
                line(indent + 1, "abi::ProxyCommand cmds[" + op.get("batch") + "];");
                int n = 0;
                for (const auto &t : op.operands) {
                    const Op &cmd = *defs.at(t);
                    ++commands;
                    const std::string slot = "cmds[" + std::to_string(n++) + "]";
                    const std::string pred = cmd.get("pred");
                    std::string body;
                    if (cmd.kind == "post_put") {
                        if (cmd.get("extent") == "trimmed")
                            ++trimmed;
                        std::string bytes = cmd.get("bytes");
                        if (bytes.rfind("ab_", 0) == 0)
                            bytes = "t2::" + bytes;
                        body = "{" + ident(cmd.operands[2]) + ", " + ident(cmd.operands[1]) + ", (std::uint32_t)(" +
                               bytes + "), " + ident(cmd.operands[2]) + "_key, " + ident(cmd.operands[1]) +
                               "_key, abi::kProxyCommandWrite}";
                    } else if (cmd.kind == "post_inline") {
                        ++inline_puts;
                        const std::string values = cmd.get("values");
                        const std::size_t colon = values.rfind(':');
                        if (values.find(',') != std::string::npos || values.substr(colon + 1) != "64")
                            throw Error("line " + std::to_string(cmd.line) +
                                        ": the ring carries one 64-bit inline value per command");
                        body = "{(unsigned long long)(" + values.substr(0, colon) + "), " + ident(cmd.operands[1]) +
                               ", 8, 0, " + ident(cmd.operands[1]) + "_key, abi::kProxyCommandWeakSignal}";
                    } else if (cmd.kind == "post_signal") {
                        const bool is_strong = cmd.has("strong");
                        (is_strong ? strong : weak) += 1;
                        if (cmd.has("elided"))
                            ++elided;
                        body = "{(unsigned long long)(" + cmd.get("epoch") + "), " + ident(cmd.operands[1]) +
                               ", 8, 0, " + ident(cmd.operands[1]) + "_key, " +
                               (is_strong ? "abi::kProxyCommandStrongSignal" : "abi::kProxyCommandWeakSignal") + "}";
                        flag_writes.push_back(std::string(is_strong ? "strong:" : "weak:") + cmd.get("epoch"));
                    } else {
                        body = "{0, 0, 0, 0, 0, abi::kProxyCommandNop}";
                    }
                    if (pred.empty())
                        line(indent + 1, slot + " = abi::ProxyCommand" + body + ";");
                    else  // a predicated-off command still occupies its slot, as an ordered NOP
                        line(indent + 1, slot + " = (" + pred + ") ? abi::ProxyCommand" + body +
                                             " : abi::ProxyCommand{0, 0, 0, 0, 0, abi::kProxyCommandNop};");
                }
                line(indent + 1, "t2::record(ab_status, proxy::submit(" + endpoint_of_batch(op) + ", cmds, " +
                                     op.get("batch") + ", &" + seq + "), " + std::to_string(0x6000 + batches) + ");");
                line(indent, "}");
                fences.push_back("st.release.sys(ready_sequence)");
                continue;
            }
            if (op.kind == "poll") {
                ++completion_waits;
                const std::string seq = "seq_" + ident(op.operands[0]);
                const std::string pred = op.get("pred");
                line(indent, "if (threadIdx.x == 0" + (pred.empty() || pred == "1" ? std::string() : " && (" + pred + ")") +
                                 ") t2::record(ab_status, proxy::poll(" + endpoint_for(op.operands[0]) + ", " + seq +
                                 "), " + std::to_string(0x6100 + completion_waits) + ");");
                fences.push_back("ld.acquire.sys(completed_sequence)");
                continue;
            }
            if (op.kind == "wait_signal") {
                line(indent, "t2::wait_signal_cta((unsigned long long)(" + op.operands[0] + "), (std::uint64_t)(" +
                                 op.operands[1] + "), ab_status, " + std::to_string(0x5000 + wait_sites++) + ");");
                flag_reads.push_back("acquire.sys>=" + op.operands[1]);
                continue;
            }
            if (op.kind == "drain" || op.kind == "wait_group") {
                ++completion_waits;
                const std::string ep = op.kind == "drain" ? ident(op.operands[0]) : group_endpoint(op.operands[0]);
                line(indent, "if (threadIdx.x == 0) t2::record(ab_status, proxy::drain(" + ep + "), " +
                                 std::to_string(0x6200 + completion_waits) + ");");
                continue;
            }
            if (op.kind == "begin_group" || op.kind == "system_fence" || op.kind == "publish_head") {
                line(indent, "// " + op.kind + ": the ring orders and publishes by itself");
                continue;
            }
            if (op.kind == "put" || op.kind == "put_inline" || op.kind == "signal" || op.kind == "planned_wait" ||
                op.kind == "wait")
                throw Error("line " + std::to_string(op.line) + ": '" + op.kind +
                            "' survived to the lowering; run form-batches first");
        }
    }

    std::string endpoint_for(const std::string &submit_name) const {
        auto it = defs.find(submit_name);
        return it == defs.end() ? "0" : endpoint_of_batch(*it->second);
    }
    std::string group_endpoint(const std::string &group) const {
        auto it = defs.find(group);
        return it == defs.end() || it->second->operands.empty() ? "0" : ident(it->second->operands[0]);
    }
};

}  // namespace

Lowered lower_p2p(const Program &p, const Options &o) {
    P2PEmitter e(p, o);
    e.prologue("");
    e.emit_block(p.body, 1);
    e.line(0, "}");
    return {e.out.str(), e.facts_json("vacuous")};
}

Lowered lower_proxy(const Program &p, const Options &o) {
    ProxyEmitter e(p, o);
    e.prologue(o.backend == "proxy" ? "" : " (served by the host-proxy ring)");
    e.emit_block(p.body, 1);
    e.line(0, "}");
    return {e.out.str(), e.facts_json(e.completion_waits ? "poll" : "none")};
}

}  // namespace spec
