// C entry points of the specializer library (libab200_spec.so).
//
//   char *ab200_spec_compile(const char *program, const char *options)
//       parse -> verify -> pass pipeline -> verify -> lower; returns a JSON object
//       {"ok", "error", "ir", "cuda", "facts", "passes"} that the caller frees with
//       ab200_spec_free().
//   char *ab200_spec_materialize(const char *program, const char *plan)
//       materialize-transport-phase: every invoke_phase of `program` replaced by the
//       fragment of the external transport program `plan`; {"ok", "error", "ir", "invocations"}.
//   char *ab200_spec_plan(const char *kind, const char *request)
//       the planning passes (plan-shapes, plan-endpoints, plan-storage,
//       plan-transport, simplify-dataflow); JSON in the same envelope.
#include <cstring>

#include "passes.hpp"
#include "planning.hpp"

namespace {

char *dup(const std::string &s) {
    char *out = static_cast<char *>(std::malloc(s.size() + 1));
    std::memcpy(out, s.c_str(), s.size() + 1);
    return out;
}

std::string envelope_error(const std::string &message) {
    spec::Json j;
    j.begin_object();
    j.key("ok").value(false);
    j.key("error").value(message);
    j.end_object();
    return j.str();
}

}  // namespace

extern "C" {

char *ab200_spec_compile(const char *program_text, const char *options_text) {
    using namespace spec;
    try {
        Options options = parse_options(options_text ? options_text : "");
        Program program = parse(program_text ? program_text : "");
        if (program.get("backend").empty())
            program.attrs["backend"] = options.backend;
        else if (program.get("backend") != options.backend)
            throw Error("program was written for transport '" + program.get("backend") +
                        "' but is being compiled for '" + options.backend + "'");
        walk(program.body, [](const Op &op) {
            if (op.kind == "invoke_phase")
                throw Error("line " + std::to_string(op.line) +
                            ": invoke_phase needs its external transport program: materialise the phases first");
        });
        verify(program);
        struct Step {
            const char *name;
            int (*run)(Program &, const Options &);
        };
        const Step steps[] = {
            {"materialize-valid-extents", materialize_valid_extents},
            {"materialize-completion", materialize_completion},
            {"forward-inline-payloads", forward_inline_payloads},
            {"plan-publication", plan_publication},
            {"form-batches", form_batches},
            {"coalesce-submissions", coalesce_submissions},
            {"order-publications", order_publications},
            {"elide-epochs", elide_epochs},
            {"defer-announcement", defer_announcement},
            {"self-reclaim", mark_self_reclaim},
            {"order-producers", order_producers},
            {"analyze-issuers", analyze_issuers},
        };
        Json passes;
        passes.begin_object();
        bool stopped = false;
        for (const Step &step : steps) {
            passes.key(step.name).value(step.run(program, options));
            verify(program);
            if (options.stop_after == step.name) {
                stopped = true;
                break;
            }
        }
        passes.end_object();
        Json j;
        j.begin_object();
        j.key("ok").value(true);
        j.key("ir").value(print(program));
        j.key("passes").raw(passes.str());
        if (!stopped) {
            const Lowered lowered = options.caps->load_store_addressable ? lower_p2p(program, options)
                                                                        : lower_proxy(program, options);
            j.key("cuda").value(lowered.cuda);
            j.key("facts").raw(lowered.facts);
        }
        j.end_object();
        return dup(j.str());
    } catch (const std::exception &error) {
        return dup(envelope_error(error.what()));
    }
}

char *ab200_spec_materialize(const char *program_text, const char *plan_text) {
    using namespace spec;
    try {
        Program program = parse(program_text ? program_text : "");
        const Program plan = parse(plan_text ? plan_text : "");
        const int count = materialize_transport_phase(program, plan);
        verify(program);
        Json j;
        j.begin_object();
        j.key("ok").value(true);
        j.key("ir").value(print(program));
        j.key("invocations").value(count);
        j.end_object();
        return dup(j.str());
    } catch (const std::exception &error) {
        return dup(envelope_error(error.what()));
    }
}

char *ab200_spec_plan(const char *kind, const char *request) {
    try {
        return dup(spec::run_planner(kind ? kind : "", request ? request : ""));
    } catch (const std::exception &error) {
        return dup(envelope_error(error.what()));
    }
}

char *ab200_spec_affine(const char *expr) {
    spec::Affine a;
    try {
        a = spec::affine_in_pid(expr ? expr : "", {});
    } catch (const std::exception &) {
        a = spec::Affine{};  // an expression that cannot be read is simply not proven
        a.known = false;
    }
    spec::Json j;
    j.begin_object();
    j.key("known").value(a.known);
    j.key("scale").value(a.scale);
    j.key("modular").value(a.modular);
    j.key("modulus").value(a.modulus);
    j.end_object();
    return dup(j.str());
}

void ab200_spec_free(char *text) { std::free(text); }

}  // extern "C"
