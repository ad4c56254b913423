// Planning passes: shape families, endpoint lanes, storage, transport phases and
// dataflow simplification.  Each takes a request written in the IR's line
// syntax and answers with a JSON document.
#pragma once

#include <string>

namespace spec {

// kind: "plan-shapes" | "plan-endpoints" | "plan-storage" | "plan-transport" |
//       "simplify-dataflow".  Returns {"ok": true, ...}.
std::string run_planner(const std::string &kind, const std::string &request);

}  // namespace spec
