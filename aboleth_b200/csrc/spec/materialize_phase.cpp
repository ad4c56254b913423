// materialize-transport-phase: splice externally planned fragments into a program.
//
// What the reference's pass does (compiler/lib/Transforms/MaterializeTransportPhase.cpp:
// 28-69 index fragments and their phases' plans, 71-100 pointer placeholders and argument
// types, 143-172 clone the body, 174-217 driver) restated for the text IR:
//
//   program kernel backend=rdma ...          program moe.plan kind=transport_program
//   arg slots ptr                             phase dispatch program_id=3 interval=4 capacities=64,32
//   ...                                       fragment send program_id=3 params=ep:i64,dst:i64,n:i64 {
//   invoke_phase 3 %e slots (count*16)          %r = remote_at dst
//                                               ...
//                                             }
//
// Every `invoke_phase <id> <args...>` is replaced by a copy of the body of the fragment
// with that program id: parameters are replaced by the arguments, values defined in the
// body get a suffix unique to the invocation, and every planned_wait without a reuse
// distance receives the resolved completion interval (the smallest over the phases bound
// to the id) and the smallest peer queue capacity of those phases.  An i64 parameter may
// stand for a pointer when the fragment only binds it (endpoint / local / remote /
// remote_at), and for an endpoint value when it only appears in `endpoint` bindings - that
// binding is then dropped and its result becomes the argument itself.  Everything else is
// an argument type error.  An invocation that survives is an error.
#include <algorithm>
#include <cctype>
#include <climits>

#include "passes.hpp"

namespace spec {

namespace {

struct Param {
    std::string name, type;
};

struct Fragment {
    const Op *op = nullptr;
    std::vector<Param> params;
    bool has_plan = false;
    long long interval = LLONG_MAX, capacity = LLONG_MAX;
};

[[noreturn]] void fail_at(const Op &op, const std::string &message) {
    throw Error("line " + std::to_string(op.line) + ": " + op.kind + ": " + message);
}

bool word_char(char c) { return std::isalnum(static_cast<unsigned char>(c)) || c == '_' || c == '.' || c == '%'; }

// Replace whole-word occurrences of the keys of `map` in `text`.
std::string substitute(const std::string &text, const std::map<std::string, std::string> &map) {
    std::string out;
    std::size_t i = 0;
    while (i < text.size()) {
        if (!word_char(text[i])) {
            out += text[i++];
            continue;
        }
        std::size_t j = i;
        while (j < text.size() && word_char(text[j]))
            ++j;
        const std::string word = text.substr(i, j - i);
        auto it = map.find(word);
        out += it == map.end() ? word : it->second;
        i = j;
    }
    return out;
}

bool mentions(const std::string &text, const std::string &name) {
    std::size_t i = 0;
    while (i < text.size()) {
        if (!word_char(text[i])) {
            ++i;
            continue;
        }
        std::size_t j = i;
        while (j < text.size() && word_char(text[j]))
            ++j;
        if (text.compare(i, j - i, name) == 0)
            return true;
        i = j;
    }
    return false;
}

bool op_mentions(const Op &op, const std::string &name) {
    for (const auto &operand : op.operands)
        if (mentions(operand, name))
            return true;
    for (const auto &[key, value] : op.attrs)
        if (mentions(value, name))
            return true;
    return false;
}

std::vector<Param> parse_params(const Op &fragment) {
    std::vector<Param> params;
    std::stringstream in(fragment.get("params"));
    std::string item;
    while (std::getline(in, item, ',')) {
        const std::size_t colon = item.find(':');
        if (colon == std::string::npos || colon == 0 || colon + 1 == item.size())
            fail_at(fragment, "params are <name>:<type>,...; got '" + item + "'");
        params.push_back({item.substr(0, colon), item.substr(colon + 1)});
    }
    return params;
}

long long min_of_list(const Op &op, const std::string &list) {
    long long least = LLONG_MAX;
    std::stringstream in(list);
    std::string item;
    while (std::getline(in, item, ',')) {
        if (!is_integer(item))
            fail_at(op, "capacities must be integers");
        least = std::min(least, to_integer(item));
    }
    return least;
}

std::map<long long, Fragment> index_fragments(const Program &plan) {
    std::map<long long, long long> intervals, capacities;
    for (const Op &op : plan.body) {
        if (op.kind != "phase" || !op.has("program_id"))
            continue;
        if (!is_integer(op.get("program_id")))
            fail_at(op, "program_id must be an integer");
        if (!is_integer(op.get("interval", "x")) || to_integer(op.get("interval")) < 1)
            fail_at(op, "a bound fragment requires a resolved completion interval (interval=<k>, k >= 1)");
        const long long id = to_integer(op.get("program_id"));
        const long long interval = to_integer(op.get("interval"));
        intervals[id] = intervals.count(id) ? std::min(intervals[id], interval) : interval;
        const long long capacity = min_of_list(op, op.get("capacities"));
        capacities[id] = capacities.count(id) ? std::min(capacities[id], capacity) : capacity;
    }
    std::map<long long, Fragment> fragments;
    for (const Op &op : plan.body) {
        if (op.kind != "fragment")
            continue;
        if (!is_integer(op.get("program_id", "x")))
            fail_at(op, "needs program_id=<integer>");
        const long long id = to_integer(op.get("program_id"));
        if (fragments.count(id))
            fail_at(op, "duplicate programId " + std::to_string(id) + " in external transport program");
        Fragment f;
        f.op = &op;
        f.params = parse_params(op);
        if (intervals.count(id)) {
            f.has_plan = true;
            f.interval = intervals[id];
            f.capacity = capacities[id];
        }
        fragments[id] = f;
    }
    return fragments;
}

bool is_binding(const Op &op) {
    return op.kind == "endpoint" || op.kind == "local" || op.kind == "remote" || op.kind == "remote_at";
}

// Type of an argument as the invoking program sees it.
std::string argument_type(const std::string &arg, const Program &program,
                          const std::map<std::string, std::string> &defs) {
    if (!arg.empty() && arg[0] == '%') {
        auto it = defs.find(arg);
        if (it != defs.end() && it->second == "endpoint")
            return "endpoint";
        return "token";
    }
    for (const Arg &a : program.args)
        if (a.name == arg)
            return a.type == "u64" || a.type == "i32" || a.type == "u32" ? "i64" : a.type;
    return "i64";  // constants and expressions
}

void rename_and_substitute(std::vector<Op> &ops, const std::map<std::string, std::string> &map) {
    for (Op &op : ops) {
        if (!op.result.empty())
            op.result = substitute(op.result, map);
        for (auto &operand : op.operands)
            operand = substitute(operand, map);
        for (auto &[key, value] : op.attrs)
            value = substitute(value, map);
        rename_and_substitute(op.body, map);
    }
}

std::vector<Op> expand(const Op &invoke, const Fragment &fragment, const Program &program,
                       const std::map<std::string, std::string> &defs, int serial) {
    const std::size_t given = invoke.operands.size() - 1;
    if (given != fragment.params.size())
        fail_at(invoke, "argument count does not match fragment '" +
                            (fragment.op->operands.empty() ? std::string("?") : fragment.op->operands[0]) + "'");
    std::map<std::string, std::string> map;
    std::vector<std::string> dropped_bindings;
    for (std::size_t i = 0; i < given; ++i) {
        const Param &param = fragment.params[i];
        const std::string &arg = invoke.operands[i + 1];
        const std::string type = argument_type(arg, program, defs);
        bool ok = type == param.type;
        if (!ok && param.type == "i64" && (type == "ptr" || type == "table" || type == "endpoint")) {
            // A placeholder: legal when the fragment only binds it.
            ok = true;
            walk(fragment.op->body, [&](const Op &op) {
                if (!op_mentions(op, param.name))
                    return;
                if (type == "endpoint" ? op.kind != "endpoint" : !is_binding(op))
                    ok = false;
            });
        }
        if (!ok)
            fail_at(invoke, "argument #" + std::to_string(i) + " has type " + type + ", but fragment '" +
                                (fragment.op->operands.empty() ? std::string("?") : fragment.op->operands[0]) +
                                "' expects " + param.type);
        // An expression stays one operand of whatever it is substituted into.
        const bool atom = is_integer(arg) || std::all_of(arg.begin(), arg.end(), word_char) ||
                          (arg.size() >= 2 && arg.front() == '(' && strip_parens(arg) != arg);
        map[param.name] = atom ? arg : "(" + arg + ")";
        if (type == "endpoint")
            dropped_bindings.push_back(param.name);
    }
    // Values defined in the body get a suffix of their own per invocation.
    // So do the names a fragment introduces itself (loop variables, lets): an argument
    // expression that mentions the kernel's own `i` must not be captured by a fragment's `i`.
    walk(fragment.op->body, [&](const Op &op) {
        if (!op.result.empty())
            map[op.result] = op.result + ".p" + std::to_string(serial);
        if ((op.kind == "for" || op.kind == "let") && !op.operands.empty()) {
            const std::string &name = op.operands[0];
            for (const Param &param : fragment.params)
                if (param.name == name)
                    fail_at(op, "'" + name + "' is a parameter of the fragment and cannot be redefined in it");
            map[name] = name + "_p" + std::to_string(serial);
        }
    });
    std::vector<Op> body;
    for (const Op &op : fragment.op->body) {
        bool dropped = false;
        if (op.kind == "endpoint")
            for (const auto &name : dropped_bindings)
                if (op_mentions(op, name)) {
                    map[op.result] = map[name];  // the binding's result is the endpoint itself
                    dropped = true;
                }
        if (!dropped)
            body.push_back(op);
    }
    rename_and_substitute(body, map);
    walk(body, [&](Op &op) {
        op.line = invoke.line;
        if (op.kind == "planned_wait" && !op.has("reuse") && fragment.has_plan) {
            op.attrs["interval"] = std::to_string(fragment.interval);
            if (fragment.capacity != LLONG_MAX)
                op.attrs["queue_capacity"] = std::to_string(fragment.capacity);
        }
    });
    return body;
}

int materialize_block(std::vector<Op> &ops, const std::map<long long, Fragment> &fragments,
                      const Program &program, std::map<std::string, std::string> defs, int &serial) {
    // `defs` maps every value visible so far (enclosing blocks, then this block in order)
    // to the kind of operation that defines it.
    int count = 0;
    std::vector<Op> out;
    for (Op &op : ops) {
        if (op.kind == "invoke_phase") {
            if (op.operands.empty() || !is_integer(op.operands[0]))
                fail_at(op, "programId must be an integer constant");
            auto found = fragments.find(to_integer(op.operands[0]));
            if (found == fragments.end())
                fail_at(op, "references missing transport fragment " + op.operands[0]);
            for (Op &spliced : expand(op, found->second, program, defs, serial++)) {
                if (!spliced.result.empty())
                    defs[spliced.result] = spliced.kind;
                out.push_back(std::move(spliced));
            }
            ++count;
            continue;
        }
        if (!op.result.empty())
            defs[op.result] = op.kind;
        if (!op.body.empty())
            count += materialize_block(op.body, fragments, program, defs, serial);
        out.push_back(std::move(op));
    }
    ops = std::move(out);
    return count;
}

}  // namespace

int materialize_transport_phase(Program &program, const Program &plan) {
    const std::map<long long, Fragment> fragments = index_fragments(plan);
    int serial = 0;
    std::map<std::string, std::string> defs;
    const int count = materialize_block(program.body, fragments, program, defs, serial);
    walk(program.body, [](const Op &op) {
        if (op.kind == "invoke_phase")
            fail_at(op, "survived transport phase materialization");
    });
    return count;
}

}  // namespace spec
