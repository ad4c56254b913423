// Runs the specializer's C entry points over a corpus of programs and over
// deterministic corruptions of them.  Built with -fsanitize=address,undefined by
// tests/test_sanitizers.py: the run passes when every intact program compiles and
// no corrupted one makes the library crash, read out of bounds or overflow (a
// diagnostic in the JSON envelope is the expected answer to a corrupted program).
//
//   spec_sanitize <corpus-dir> <cases>      cases are <dir>/<i>.prog + <dir>/<i>.opts
#include <cctype>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <sstream>
#include <string>
#include <utility>
#include <vector>

extern "C" {
char *ab200_spec_compile(const char *program, const char *options);
char *ab200_spec_plan(const char *kind, const char *request);
char *ab200_spec_materialize(const char *program, const char *plan);
char *ab200_spec_affine(const char *expr);
void ab200_spec_free(char *text);
}

namespace {

std::string slurp(const std::string &path) {
    std::ifstream in(path);
    std::stringstream ss;
    ss << in.rdbuf();
    return ss.str();
}

bool compiles(const std::string &program, const std::string &options) {
    char *out = ab200_spec_compile(program.c_str(), options.c_str());
    const bool ok = out != nullptr && std::strncmp(out, "{\"ok\": true", 11) == 0;
    ab200_spec_free(out);
    return ok;
}

std::vector<std::string> lines_of(const std::string &text) {
    std::vector<std::string> lines;
    std::istringstream in(text);
    for (std::string line; std::getline(in, line);)
        lines.push_back(line);
    return lines;
}

std::string join(const std::vector<std::string> &lines, std::size_t skip, std::size_t limit) {
    std::string out;
    for (std::size_t i = 0; i < lines.size() && i < limit; ++i)
        if (i != skip)
            out += lines[i] + "\n";
    return out;
}

struct Lcg {
    std::uint64_t state;
    std::uint32_t next() {
        state = state * 6364136223846793005ull + 1442695040888963407ull;
        return static_cast<std::uint32_t>(state >> 33);
    }
};

}  // namespace

int main(int argc, char **argv) {
    if (argc != 3) {
        std::fprintf(stderr, "usage: spec_sanitize <corpus-dir> <cases>\n");
        return 2;
    }
    const std::string dir = argv[1];
    const int cases = std::atoi(argv[2]);
    long accepted = 0, refused = 0;
    for (int c = 0; c < cases; ++c) {
        const std::string program = slurp(dir + "/" + std::to_string(c) + ".prog");
        const std::string options = slurp(dir + "/" + std::to_string(c) + ".opts");
        if (!compiles(program, options)) {
            std::fprintf(stderr, "case %d: the intact program does not compile\n", c);
            return 1;
        }
        const std::vector<std::string> lines = lines_of(program);
        // Every prefix, and the program with each single line removed.
        for (std::size_t i = 0; i <= lines.size(); ++i) {
            (compiles(join(lines, lines.size(), i), options) ? accepted : refused)++;
            if (i < lines.size())
                (compiles(join(lines, i, lines.size()), options) ? accepted : refused)++;
        }
        // Byte-level damage: digits blown up, separators swapped, bytes dropped.
        Lcg rng{0x9e3779b97f4a7c15ull + static_cast<std::uint64_t>(c)};
        for (int round = 0; round < 300; ++round) {
            std::string damaged = program;
            const int edits = 1 + static_cast<int>(rng.next() % 4);
            for (int e = 0; e < edits && !damaged.empty(); ++e) {
                const std::size_t at = rng.next() % damaged.size();
                switch (rng.next() % 5) {
                case 0: damaged.erase(at, 1 + rng.next() % 8); break;
                case 1: damaged.insert(at, "99999999999999999999"); break;
                case 2: damaged[at] = "=,%[](){}-\" \n"[rng.next() % 13]; break;
                case 3: damaged.insert(at, damaged.substr(at, rng.next() % 40)); break;
                default: damaged[at] = static_cast<char>(rng.next() & 0x7f); break;
                }
            }
            (compiles(damaged, options) ? accepted : refused)++;
        }
        // The options string is parsed by the library too.
        for (const char *bad : {"backend=", "backend=nosuch", "inline_bytes=x", "queue_capacity=-1",
                                "enable=,,,", "stop_after=form-batches", "completion_interval=0"})
            (compiles(program, bad) ? accepted : refused)++;
    }
    for (const char *expr : {"pid", "(pid + 3) % 8", "lane*4+peer", "pid*", "((((", "", "pid % 0",
                             "99999999999999999999*pid", "pid + pid + pid", "-pid"}) {
        char *out = ab200_spec_affine(expr);
        ab200_spec_free(out);
    }
    for (const char *kind : {"plan-shapes", "plan-endpoints", "plan-storage", "plan-transport",
                             "simplify-dataflow", "nosuch", ""})
        for (const char *request : {"", "{", "{}", "[]", "{\"a\":", "{\"min\":1,\"max\":0}", "null"}) {
            char *out = ab200_spec_plan(kind, request);
            ab200_spec_free(out);
        }
    // materialize-transport-phase over a damaged kernel and a damaged external program.
    {
        const std::string kernel = slurp(dir + "/phase.kernel"), plan = slurp(dir + "/phase.plan");
        if (!kernel.empty()) {
            char *intact = ab200_spec_materialize(kernel.c_str(), plan.c_str());
            const bool ok = std::strncmp(intact, "{\"ok\": true", 11) == 0;
            ab200_spec_free(intact);
            if (!ok) {
                std::fprintf(stderr, "the intact phase program does not materialise\n");
                return 1;
            }
            Lcg rng{12345};
            for (int round = 0; round < 2000; ++round) {
                std::string k = kernel, p = plan;
                std::string &victim = (round & 1) ? k : p;
                const std::size_t at = rng.next() % victim.size();
                switch (rng.next() % 4) {
                case 0: victim.erase(at, 1 + rng.next() % 12); break;
                case 1: victim.insert(at, "99999999999999999999"); break;
                case 2: victim[at] = "=,%:(){} \n"[rng.next() % 11]; break;
                default: victim.insert(at, victim.substr(at, rng.next() % 30)); break;
                }
                char *out = ab200_spec_materialize(k.c_str(), p.c_str());
                (std::strncmp(out, "{\"ok\": true", 11) == 0 ? accepted : refused)++;
                ab200_spec_free(out);
            }
        }
    }
    // The planners over their own requests with the numbers pushed to the edges (0, -1, 1, huge)
    // and with byte damage: a planner answers with a plan or a diagnostic, never a crash.
    for (int c = 0;; ++c) {
        const std::string kind = slurp(dir + "/planner." + std::to_string(c) + ".kind");
        const std::string request = slurp(dir + "/planner." + std::to_string(c) + ".req");
        if (kind.empty())
            break;
        char *intact = ab200_spec_plan(kind.c_str(), request.c_str());
        const bool ok = std::strncmp(intact, "{\"ok\": true", 11) == 0;
        ab200_spec_free(intact);
        if (!ok) {
            std::fprintf(stderr, "planner case %d (%s): the intact request is refused\n", c, kind.c_str());
            return 1;
        }
        // Every integer literal, one at a time, replaced by each edge value.
        std::vector<std::pair<std::size_t, std::size_t>> numbers;
        for (std::size_t i = 0; i < request.size();) {
            const bool starts = std::isdigit(static_cast<unsigned char>(request[i])) &&
                                (i == 0 || request[i - 1] == '=' || request[i - 1] == ',' || request[i - 1] == ' ' ||
                                 request[i - 1] == ':');
            if (!starts) {
                ++i;
                continue;
            }
            std::size_t j = i;
            while (j < request.size() && std::isdigit(static_cast<unsigned char>(request[j])))
                ++j;
            numbers.emplace_back(i, j - i);
            i = j;
        }
        for (const auto &[at, length] : numbers)
            for (const char *edge : {"0", "-1", "1", "3", "4294967296", "9223372036854775807", "99999999999999999999"}) {
                std::string damaged = request;
                damaged.replace(at, length, edge);
                char *out = ab200_spec_plan(kind.c_str(), damaged.c_str());
                (std::strncmp(out, "{\"ok\": true", 11) == 0 ? accepted : refused)++;
                ab200_spec_free(out);
            }
        Lcg rng{777u + static_cast<std::uint64_t>(c)};
        for (int round = 0; round < 300; ++round) {
            std::string damaged = request;
            const std::size_t at = rng.next() % damaged.size();
            switch (rng.next() % 4) {
            case 0: damaged.erase(at, 1 + rng.next() % 10); break;
            case 1: damaged[at] = "=,:() \n-"[rng.next() % 8]; break;
            case 2: damaged.insert(at, damaged.substr(at, rng.next() % 40)); break;
            default: damaged.resize(at); break;
            }
            char *out = ab200_spec_plan(kind.c_str(), damaged.c_str());
            (std::strncmp(out, "{\"ok\": true", 11) == 0 ? accepted : refused)++;
            ab200_spec_free(out);
        }
    }
    std::printf("corrupted programs: %ld accepted, %ld refused\n", accepted, refused);
    return 0;
}
