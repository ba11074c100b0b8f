// topology_linter <config>
//
// Prints the decomposition report and the library's pre-compile checks (cai::lint_config: memory budget,
// tensor-parallel placement, rank <-> location round trips, pipeline bubble). Exit code 0 when nothing
// failed, 1 on a failed check or an unreadable config, 2 on a usage error, like the reference tool
// (tools/topology_linter.c).
#include <cstdio>

#include "plan.h"

using namespace cai;

int main(int argc, char** argv) {
    if (argc != 2) { std::fprintf(stderr, "usage: %s <config>\n", argv[0]); return 2; }
    Config cfg;
    std::string err;
    Decomp d;
    if (config_load(argv[1], &cfg, &err) != OK) { std::fprintf(stderr, "config error: %s\n", err.c_str()); return 1; }
    if (topology_finalize(&cfg.topo, &err) != OK) { std::fprintf(stderr, "[FAIL] topology: %s\n", err.c_str()); return 1; }
    if (decompose(cfg, &d, &err) != OK) { std::fprintf(stderr, "[FAIL] decompose: %s\n", err.c_str()); return 1; }
    std::printf("=== decomposition ===\n");
    const bool fits = report_decomp(stdout, cfg, d);
    std::printf("=====================\nchecks:\n");
    VerifyReport rep;
    lint_config(cfg, d, fits, &rep);
    for (const std::string& l : rep.lines) std::fprintf(l.find("[ok]") != std::string::npos ? stdout : stderr, "%s\n", l.c_str());
    if (rep.problems) std::printf("\nRESULT: %d problem(s)\n", rep.problems);
    else std::printf("\nRESULT: all checks passed\n");
    return rep.problems ? 1 : 0;
}
