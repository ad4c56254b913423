// Parser, printer and verifier of the communication IR (see ir.hpp).
//
// The verifier enforces the structural rules the reference states for its
// dialect (compiler/lib/IR/Dialect.cpp:26-38,104-139,206-520): inline payload
// widths and size, `after` tokens on the same endpoint and defined earlier,
// wait_group after its begin_group in the same block, and - once Queue IR
// exists - the shape of a submission (segments of chained puts each optionally
// closed by a signal, one endpoint, batch size equal to the token count, a
// trailing post_nop only in last position).
#include "ir.hpp"

#include <algorithm>
#include <cctype>
#include <set>
#include <sstream>

namespace spec {

namespace {

// Split a line into tokens at whitespace outside parentheses / quotes.
std::vector<std::string> tokenize(const std::string &line) {
    std::vector<std::string> out;
    std::string cur;
    int depth = 0;
    bool quoted = false;
    for (char c : line) {
        if (quoted) {
            cur += c;
            if (c == '"')
                quoted = false;
            continue;
        }
        if (c == '"') {
            quoted = true;
            cur += c;
        } else if (c == '(' || c == '[') {
            ++depth;
            cur += c;
        } else if (c == ')' || c == ']') {
            --depth;
            cur += c;
        } else if (std::isspace(static_cast<unsigned char>(c)) && depth == 0) {
            if (!cur.empty()) {
                out.push_back(cur);
                cur.clear();
            }
        } else {
            cur += c;
        }
    }
    if (!cur.empty())
        out.push_back(cur);
    return out;
}

bool is_attr_token(const std::string &tok, std::string &key, std::string &value) {
    // key=value where key is an identifier and '=' is not part of "==".
    std::size_t i = 0;
    while (i < tok.size() && (std::isalnum(static_cast<unsigned char>(tok[i])) || tok[i] == '_'))
        ++i;
    if (i == 0 || i >= tok.size() || tok[i] != '=' || (i + 1 < tok.size() && tok[i + 1] == '='))
        return false;
    key = tok.substr(0, i);
    value = tok.substr(i + 1);
    return true;
}

const std::set<std::string> kFlagAttrs = {"weak",  "strong", "producerBarrier", "exclusiveIssuer",
                                         "deferCompletion", "deferredAnnouncement", "selfReclaim",
                                         "externalPublication", "elided", "cooperative", "final",
                                         "unknown_write", "ordering_point"};

struct Lines {
    std::vector<std::pair<int, std::string>> items;
    std::size_t at = 0;
};

Op parse_op(Lines &lines);

std::vector<Op> parse_block(Lines &lines, bool nested) {
    std::vector<Op> ops;
    while (lines.at < lines.items.size()) {
        const std::string &text = lines.items[lines.at].second;
        if (text == "}") {
            if (!nested)
                throw Error("line " + std::to_string(lines.items[lines.at].first) + ": unmatched }");
            ++lines.at;
            return ops;
        }
        ops.push_back(parse_op(lines));
    }
    if (nested)
        throw Error("unterminated block: missing }");
    return ops;
}

Op parse_op(Lines &lines) {
    const int line_no = lines.items[lines.at].first;
    std::vector<std::string> toks = tokenize(lines.items[lines.at].second);
    ++lines.at;
    Op op;
    op.line = line_no;
    std::size_t i = 0;
    if (toks.size() >= 3 && toks[0][0] == '%' && toks[1] == "=") {
        op.result = toks[0];
        i = 2;
    }
    if (i >= toks.size())
        throw Error("line " + std::to_string(line_no) + ": missing operation name");
    op.kind = toks[i++];
    bool opens = false;
    for (; i < toks.size(); ++i) {
        if (toks[i] == "{") {
            opens = true;
            continue;
        }
        std::string key, value;
        if (op.kind != "stmt" && is_attr_token(toks[i], key, value))
            op.attrs[key] = value;
        else if (op.kind != "stmt" && kFlagAttrs.count(toks[i]))
            op.attrs[toks[i]] = "";
        else
            op.operands.push_back(toks[i]);
    }
    if (opens)
        op.body = parse_block(lines, true);
    else if (op.kind == "for" || op.kind == "if")
        throw Error("line " + std::to_string(line_no) + ": " + op.kind + " needs a { block }");
    return op;
}

std::string join_op(const Op &op) {
    std::ostringstream out;
    if (!op.result.empty())
        out << op.result << " = ";
    out << op.kind;
    for (const auto &o : op.operands)
        out << ' ' << o;
    for (const auto &kv : op.attrs) {
        out << ' ' << kv.first;
        if (!kv.second.empty() || !kFlagAttrs.count(kv.first))
            out << '=' << kv.second;
    }
    return out.str();
}

}  // namespace

bool is_integer(const std::string &raw) {
    const std::string text = strip_parens(raw);
    if (text.empty())
        return false;
    std::size_t i = (text[0] == '-' || text[0] == '+') ? 1 : 0;
    if (i >= text.size())
        return false;
    if (text.size() > i + 2 && text[i] == '0' && (text[i + 1] == 'x' || text[i + 1] == 'X')) {
        for (std::size_t k = i + 2; k < text.size(); ++k)
            if (!std::isxdigit(static_cast<unsigned char>(text[k])))
                return false;
        return true;
    }
    for (; i < text.size(); ++i)
        if (!std::isdigit(static_cast<unsigned char>(text[i])))
            return false;
    return true;
}

long long to_integer(const std::string &text) {
    if (!is_integer(text))
        throw Error("'" + text + "' is not an integer constant");
    return std::stoll(strip_parens(text), nullptr, 0);
}

std::string strip_parens(const std::string &text) {
    std::string t = text;
    while (t.size() >= 2 && t.front() == '(' && t.back() == ')') {
        int depth = 0;
        bool wraps = true;
        for (std::size_t i = 0; i + 1 < t.size(); ++i) {
            if (t[i] == '(')
                ++depth;
            else if (t[i] == ')')
                --depth;
            if (depth == 0) {
                wraps = false;
                break;
            }
        }
        if (!wraps)
            break;
        t = t.substr(1, t.size() - 2);
    }
    return t;
}

Program parse(const std::string &text) {
    Lines lines;
    std::istringstream in(text);
    std::string raw;
    int n = 0;
    while (std::getline(in, raw)) {
        ++n;
        const std::size_t hash = raw.find('#');
        if (hash != std::string::npos && raw.find("stmt") == std::string::npos)
            raw = raw.substr(0, hash);
        std::size_t b = raw.find_first_not_of(" \t\r");
        if (b == std::string::npos)
            continue;
        std::size_t e = raw.find_last_not_of(" \t\r");
        lines.items.emplace_back(n, raw.substr(b, e - b + 1));
    }
    if (lines.items.empty())
        throw Error("empty program");
    Program program;
    {
        std::vector<std::string> toks = tokenize(lines.items[0].second);
        if (toks.size() < 2 || toks[0] != "program")
            throw Error("line " + std::to_string(lines.items[0].first) +
                        ": a program starts with 'program <name> key=value...'");
        program.name = toks[1];
        for (std::size_t i = 2; i < toks.size(); ++i) {
            std::string key, value;
            if (!is_attr_token(toks[i], key, value))
                throw Error("line 1: expected key=value, got '" + toks[i] + "'");
            program.attrs[key] = value;
        }
        lines.at = 1;
    }
    while (lines.at < lines.items.size()) {
        std::vector<std::string> toks = tokenize(lines.items[lines.at].second);
        if (toks.empty() || toks[0] != "arg")
            break;
        if (toks.size() != 3)
            throw Error("line " + std::to_string(lines.items[lines.at].first) +
                        ": 'arg <name> <type>'");
        program.args.push_back({toks[1], toks[2]});
        ++lines.at;
    }
    program.body = parse_block(lines, false);
    return program;
}

std::string print(const Op &op, int indent) {
    std::ostringstream out;
    const std::string pad(indent * 2, ' ');
    out << pad << join_op(op);
    if (op.kind == "for" || op.kind == "if") {
        out << " {\n";
        for (const auto &child : op.body)
            out << print(child, indent + 1);
        out << pad << "}";
    }
    out << "\n";
    return out.str();
}

std::string print(const Program &program) {
    std::ostringstream out;
    out << "program " << program.name;
    for (const auto &kv : program.attrs)
        out << ' ' << kv.first << '=' << kv.second;
    out << "\n";
    for (const auto &arg : program.args)
        out << "arg " << arg.name << ' ' << arg.type << "\n";
    for (const auto &op : program.body)
        out << print(op, 0);
    return out.str();
}

std::string Json::quote(const std::string &s) {
    std::string out = "\"";
    for (char c : s) {
        switch (c) {
        case '"': out += "\\\""; break;
        case '\\': out += "\\\\"; break;
        case '\n': out += "\\n"; break;
        case '\t': out += "\\t"; break;
        case '\r': out += "\\r"; break;
        default:
            if (static_cast<unsigned char>(c) < 0x20) {
                char buf[8];
                std::snprintf(buf, sizeof(buf), "\\u%04x", c);
                out += buf;
            } else {
                out += c;
            }
        }
    }
    return out + "\"";
}

// ---- verifier ---------------------------------------------------------------------------

namespace {

struct Scope {
    std::map<std::string, const Op *> defs;  // visible values
    const Scope *parent = nullptr;
    const Op *find(const std::string &name) const {
        for (const Scope *s = this; s; s = s->parent) {
            auto it = s->defs.find(name);
            if (it != s->defs.end())
                return it->second;
        }
        return nullptr;
    }
};

[[noreturn]] void fail(const Op &op, const std::string &message) {
    throw Error("line " + std::to_string(op.line) + ": " + op.kind + ": " + message);
}

std::string endpoint_of(const Op &op) {
    if (op.operands.empty())
        return "";
    return op.operands[0];
}

void verify_inline(const Op &op) {
    const std::string values = op.get("values");
    if (values.empty())
        fail(op, "needs values=<expr:bits>,...");
    long long bits_total = 0;
    std::size_t start = 0;
    int depth = 0;
    for (std::size_t i = 0; i <= values.size(); ++i) {
        if (i < values.size() && values[i] == '(')
            ++depth;
        if (i < values.size() && values[i] == ')')
            --depth;
        if (i == values.size() || (values[i] == ',' && depth == 0)) {
            const std::string item = values.substr(start, i - start);
            const std::size_t colon = item.rfind(':');
            if (colon == std::string::npos)
                fail(op, "inline value '" + item + "' needs a :bits suffix");
            const long long bits = std::stoll(item.substr(colon + 1));
            if (bits != 8 && bits != 16 && bits != 24 && bits != 32 && bits != 64)
                fail(op, "inline payload width " + std::to_string(bits) +
                             " is not one of 8, 16, 24, 32, 64 bits");
            bits_total += bits;
            start = i + 1;
        }
    }
    if (bits_total / 8 > 972)
        fail(op, "inline payload of " + std::to_string(bits_total / 8) +
                     " bytes exceeds the 972-byte limit");
}

void verify_submit(const Op &op, const Scope &scope) {
    if (op.operands.empty())
        fail(op, "a submission needs at least one token");
    const long long batch = to_integer(op.get("batch", "0"));
    if (batch != static_cast<long long>(op.operands.size()))
        fail(op, "batch=" + std::to_string(batch) + " but " + std::to_string(op.operands.size()) +
                     " tokens are listed");
    std::string endpoint;
    std::set<std::string> in_batch;
    std::string previous;
    bool segment_open = false;  // inside a put chain not yet closed by a signal
    // A coalesced submission lists the sizes of the submissions it was merged from
    // ("segments=3+1+2"): a chain may also end at such a boundary without a signal.
    std::set<std::size_t> boundaries;
    if (op.has("segments")) {
        std::size_t start = 0;
        std::stringstream sizes(op.get("segments"));
        std::string size;
        while (std::getline(sizes, size, '+')) {
            boundaries.insert(start);
            start += static_cast<std::size_t>(std::stoul(size));
        }
        if (start != op.operands.size())
            fail(op, "segments=" + op.get("segments") + " does not add up to the batch size");
    }
    for (std::size_t i = 0; i < op.operands.size(); ++i) {
        if (boundaries.count(i))
            segment_open = false;
        const Op *cmd = scope.find(op.operands[i]);
        if (cmd == nullptr || !is_posted(*cmd))
            fail(op, "token " + op.operands[i] + " is not a posted command in scope");
        if (endpoint.empty())
            endpoint = endpoint_of(*cmd);
        else if (endpoint_of(*cmd) != endpoint)
            fail(op, "commands of one submission must share an endpoint");
        if (cmd->kind == "post_nop" && i + 1 != op.operands.size())
            fail(op, "post_nop may only be the last command of a submission");
        const std::string after = cmd->get("after");
        if (op.has("publicationsOrdered")) {
            // order-publications moved payload ahead of the (chained) signals; the
            // per-segment chain rule was checked before that rewrite.
        } else if (!segment_open) {
            if (!after.empty() && in_batch.count(after))
                fail(op, "the first command of a segment depends on a command in the batch");
        } else if (after != previous) {
            fail(op, "command " + op.operands[i] + " does not depend on its predecessor");
        }
        segment_open = cmd->kind == "post_put" || cmd->kind == "post_inline";
        in_batch.insert(op.operands[i]);
        previous = op.operands[i];
    }
    if (op.has("deferredAnnouncement") && !op.has("poll_predicate"))
        fail(op, "deferredAnnouncement needs a predicated poll");
    if (op.has("externalPublication") && !op.has("deferCompletion"))
        fail(op, "externalPublication implies deferCompletion");
}

void verify_block(const std::vector<Op> &ops, const Scope *parent) {
    Scope scope;
    scope.parent = parent;
    std::set<std::string> open_groups;
    for (const Op &op : ops) {
        for (const char *key : {"after", "group"}) {
            if (!op.has(key))
                continue;
            const Op *def = scope.find(op.get(key));
            if (def == nullptr)
                fail(op, std::string(key) + "=" + op.get(key) + " is not defined before this op");
            if (std::string(key) == "after") {
                const bool token = is_command(*def) || is_posted(*def);
                if (!token)
                    fail(op, "after=" + op.get(key) + " is not a transfer token");
                if (endpoint_of(*def) != endpoint_of(op))
                    fail(op, "after=" + op.get(key) + " belongs to another endpoint");
            }
        }
        // Operand counts of the binding and control operations: the passes and the
        // lowerings index operands by position, so a short operation is refused here.
        static const std::map<std::string, std::pair<std::size_t, const char *>> arity = {
            {"let", {2, "<name> <expr>"}},
            {"endpoint", {2, "<table> <index>"}},
            {"local", {1, "<address> [key=] [at=] [valid=]"}},
            {"remote", {2, "<table> <peer> [offset=]"}},
            {"remote_at", {1, "<address> [key=]"}},
            {"store", {1, "<address> value=<v> [offset=] [width=]"}},
            {"for", {3, "<var> <begin> <end> { ... }"}},
            {"if", {1, "<condition> { ... }"}},
            {"drain", {1, "<endpoint>"}},
            {"publish_head", {1, "<endpoint>"}},
            {"post_nop", {1, "<endpoint>"}},
        };
        if (auto it = arity.find(op.kind); it != arity.end()) {
            const bool exact = op.kind != "let" && op.kind != "if";  // expressions may tokenise further
            if (op.operands.size() < it->second.first || (exact && op.operands.size() != it->second.first))
                fail(op, std::string("expects ") + it->second.second);
        }
        if ((op.kind == "endpoint" || op.kind == "local" || op.kind == "remote" || op.kind == "remote_at" ||
             op.kind == "begin_group") && op.result.empty())
            fail(op, "defines a value and needs a %name = in front");
        if (op.kind == "put" || op.kind == "post_put") {
            if (op.operands.size() != 3 || !op.has("bytes"))
                fail(op, "expects <endpoint> <remote> <local> bytes=<n>");
        } else if (op.kind == "put_inline" || op.kind == "post_inline") {
            if (op.operands.size() != 2)
                fail(op, "expects <endpoint> <remote> values=...");
            verify_inline(op);
        } else if (op.kind == "signal" || op.kind == "post_signal") {
            if (op.operands.size() != 2 || !op.has("epoch"))
                fail(op, "expects <endpoint> <remote flag> epoch=<e>");
        } else if (op.kind == "wait" || op.kind == "planned_wait" || op.kind == "poll") {
            if (op.operands.size() != 1 || scope.find(op.operands[0]) == nullptr)
                fail(op, "expects one token defined earlier");
            // The bound is a reuse distance, or an interval a transport plan resolved already.
            if (op.kind == "planned_wait" && (!op.has("iteration") || !(op.has("reuse") || op.has("interval"))))
                fail(op, "needs iteration= and reuse= (or a planned interval=)");
        } else if (op.kind == "begin_group") {
            open_groups.insert(op.result);
        } else if (op.kind == "wait_group") {
            if (op.operands.size() != 1 || !open_groups.count(op.operands[0]))
                fail(op, "must follow its begin_group in the same block (post-dominate it)");
            open_groups.erase(op.operands[0]);
        } else if (op.kind == "wait_signal") {
            if (op.operands.size() != 2)
                fail(op, "expects <flag address> <epoch>");
        } else if (op.kind == "submit") {
            verify_submit(op, scope);
        } else if (op.kind == "local") {
            if (op.has("valid")) {
                const std::string v = op.get("valid");
                if (std::count(v.begin(), v.end(), ',') < 2)
                    fail(op, "valid=<count>,<capacity>,<item_bytes>");
            }
        }
        if (!op.result.empty()) {
            if (scope.defs.count(op.result))
                fail(op, "value " + op.result + " is defined twice in one block");
            scope.defs[op.result] = &op;
        }
        if (!op.body.empty())
            verify_block(op.body, &scope);
    }
    if (!open_groups.empty())
        throw Error("begin_group " + *open_groups.begin() + " has no wait_group in its block");
}

}  // namespace

void verify(const Program &program) {
    static const std::set<std::string> backends = {"p2p", "proxy", "rdma", "efa", "ionic"};
    if (!backends.count(program.get("backend", "p2p")))
        throw Error("unknown transport '" + program.get("backend") +
                    "': a transport the capability registry does not know is rejected");
    verify_block(program.body, nullptr);
}

}  // namespace spec
