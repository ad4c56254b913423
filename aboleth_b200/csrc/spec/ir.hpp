// Communication IR of the Tier-2 specializer.
//
// A program is a tree of operations written as text, one per line:
//
//   program alltoall backend=p2p world=2 rank=0 threads=32
//   arg send ptr
//   %e = endpoint endpoints peer
//   %src = local (send+peer*4096) key=0
//   %dst = remote recv_table peer offset=(RANK*4096)
//   %t = put %e %dst %src bytes=4096
//   %s = signal %e %flag epoch=1 after=%t
//   wait_signal (my_flags+peer) 1
//   wait %s
//
// Three strata, as in the reference dialect
// (compiler/include/aboleth/IR/AbolethOps.td:14-1019): binding ops (endpoint,
// local, remote), semantic ops (put, put_inline, signal, wait, planned_wait,
// begin_group, wait_group, wait_signal, drain, system_fence, publish_head) and
// Queue IR (post_put, post_inline, post_signal, post_nop, submit, poll).
// Frontend code that matters to the analyses is kept as `store` (a scalar
// store at a constant offset), `tensor_store` (a CTA-wide write of local
// memory), `load`, `stmt` (opaque) and the structured `for` / `if`.
//
// Operands and attribute values are C expressions kept as text; the passes
// inspect them only where an analysis needs to (constants, the program-id
// patterns of the issuer analysis).
#pragma once

#include <map>
#include <memory>
#include <set>
#include <sstream>
#include <stdexcept>
#include <string>
#include <vector>

namespace spec {

struct Error : std::runtime_error {
    using std::runtime_error::runtime_error;
};

struct Op {
    std::string kind;
    std::string result;                       // "%name" or empty
    std::vector<std::string> operands;        // positional
    std::map<std::string, std::string> attrs; // key=value (flag attrs have empty value)
    std::vector<Op> body;                     // for / if
    int line = 0;

    bool has(const std::string &key) const { return attrs.count(key) != 0; }
    std::string get(const std::string &key, const std::string &fallback = "") const {
        auto it = attrs.find(key);
        return it == attrs.end() ? fallback : it->second;
    }
};

struct Arg {
    std::string name, type;
};

struct Program {
    std::string name;
    std::map<std::string, std::string> attrs;  // backend, world, rank, threads, ...
    std::vector<Arg> args;
    std::vector<Op> body;

    std::string get(const std::string &key, const std::string &fallback = "") const {
        auto it = attrs.find(key);
        return it == attrs.end() ? fallback : it->second;
    }
};

Program parse(const std::string &text);
std::string print(const Program &program);
std::string print(const Op &op, int indent = 0);

// Structural rules of the dialect; throws Error with the offending line.
void verify(const Program &program);

// ---- helpers shared by the passes ----------------------------------------------------

bool is_integer(const std::string &text);
long long to_integer(const std::string &text);  // throws if not a constant
std::string strip_parens(const std::string &text);

inline bool is_command(const Op &op) {
    return op.kind == "put" || op.kind == "put_inline" || op.kind == "signal";
}
inline bool is_posted(const Op &op) {
    return op.kind == "post_put" || op.kind == "post_inline" || op.kind == "post_signal" ||
           op.kind == "post_nop";
}

// Visit every op (pre-order), including nested bodies.
template <typename Fn>
void walk(std::vector<Op> &ops, Fn &&fn) {
    for (auto &op : ops) {
        fn(op);
        walk(op.body, fn);
    }
}
template <typename Fn>
void walk(const std::vector<Op> &ops, Fn &&fn) {
    for (const auto &op : ops) {
        fn(op);
        walk(op.body, fn);
    }
}

// Apply `fn` to every block (vector of ops) of the program, innermost last.
template <typename Fn>
void for_each_block(std::vector<Op> &ops, Fn &&fn) {
    fn(ops);
    for (auto &op : ops)
        if (!op.body.empty())
            for_each_block(op.body, fn);
}

// Minimal JSON writer (objects, arrays, strings, numbers, bools).
class Json {
  public:
    static std::string quote(const std::string &s);
    Json &begin_object() { return open('{'); }
    Json &end_object() { return close('}'); }
    Json &begin_array() { return open('['); }
    Json &end_array() { return close(']'); }
    Json &key(const std::string &k) {
        comma();
        out_ << quote(k) << ": ";
        fresh_ = true;
        return *this;
    }
    Json &value(const std::string &s) { comma(); out_ << quote(s); return *this; }
    Json &value(const char *s) { return value(std::string(s)); }
    Json &value(long long v) { comma(); out_ << v; return *this; }
    Json &value(int v) { return value(static_cast<long long>(v)); }
    Json &value(unsigned v) { return value(static_cast<long long>(v)); }
    Json &value(std::size_t v) { return value(static_cast<long long>(v)); }
    Json &value(bool v) { comma(); out_ << (v ? "true" : "false"); return *this; }
    Json &raw(const std::string &json) { comma(); out_ << json; return *this; }
    std::string str() const { return out_.str(); }

  private:
    Json &open(char c) { comma(); out_ << c; fresh_ = true; return *this; }
    Json &close(char c) { out_ << c; fresh_ = false; return *this; }
    void comma() {
        if (!fresh_)
            out_ << ", ";
        fresh_ = false;
    }
    std::ostringstream out_;
    bool fresh_ = true;
};

}  // namespace spec
