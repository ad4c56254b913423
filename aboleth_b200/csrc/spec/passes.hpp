// Pass pipeline of the Tier-2 specializer.
//
// Order and switches follow the reference driver (python/aboleth/compiler.py:79-134,
// 333-428; docs/COMPILER_SEMANTICS.md:39-75):
//
//   materialize-valid-extents -> materialize-completion -> forward-inline-payloads
//   -> plan-publication -> form-batches (always) -> coalesce-submissions
//   -> order-publications -> elide-epochs -> [defer-announcement]
//   -> order-producers (always) -> analyze-issuers -> lower-<backend>
//
// Passes ask the capability registry what the transport can do, never which
// transport it is.
#pragma once

#include <set>
#include <string>

#include "aboleth/abi/transport_plan.h"
#include "ir.hpp"

namespace spec {

struct Options {
    std::string backend = "p2p";
    const aboleth::abi::TransportCaps *caps = nullptr;
    std::set<std::string> enabled;       // switch names that are on
    unsigned inline_bytes = 28;          // largest payload forwarded into a command
    unsigned queue_capacity = 0;         // 0: transport default / unbounded
    unsigned completion_interval = 0;    // 0: transport preference
    bool strict_registrations = false;
    unsigned coop_min = 256;             // p2p: smallest put copied by the whole CTA
    unsigned coop_elements = 2048;       // p2p: 8-byte elements per cooperative step
    bool p2p_scalar = false;             // p2p: force the single-thread copy
    std::string stop_after;              // run the pipeline up to and including this pass

    bool on(const std::string &name) const { return enabled.count(name) != 0; }
};

Options parse_options(const std::string &text);

// Each pass returns how many rewrites it made (0 = no-op), for the ablation facts.
int materialize_valid_extents(Program &p, const Options &o);
int materialize_completion(Program &p, const Options &o);
int forward_inline_payloads(Program &p, const Options &o);
int plan_publication(Program &p, const Options &o);
int form_batches(Program &p, const Options &o);
int coalesce_submissions(Program &p, const Options &o);
int order_publications(Program &p, const Options &o);
int elide_epochs(Program &p, const Options &o);
int defer_announcement(Program &p, const Options &o);
int mark_self_reclaim(Program &p, const Options &o);
int order_producers(Program &p, const Options &o);
int analyze_issuers(Program &p, const Options &o);

// Splice the fragments of an external transport program (`plan`) into `p` at every
// invoke_phase; returns the number of invocations replaced (materialize_phase.cpp).
int materialize_transport_phase(Program &p, const Program &plan);

struct Lowered {
    std::string cuda;   // CUDA C++ translation unit
    std::string facts;  // JSON object
};
Lowered lower_p2p(const Program &p, const Options &o);
Lowered lower_proxy(const Program &p, const Options &o);

// Affine-in-program-id analysis used by analyze_issuers (exposed for tests).
struct Affine {
    bool known = false;
    long long scale = 0;   // coefficient of the program id
    bool modular = false;  // wrapped by "% modulus"
    long long modulus = 0;
};
Affine affine_in_pid(const std::string &expr, const std::map<std::string, std::string> &lets);

}  // namespace spec
