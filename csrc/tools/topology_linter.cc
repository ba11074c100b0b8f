// topology_linter <config>
//
// Pre-compile sanity checks: memory fits the budget, tensor-parallel groups stay inside one
// NVLink domain, rank <-> physical location round-trips, pipeline bubble is not excessive.
// Output format follows the reference tool (tools/topology_linter.c).
#include <cstdarg>
#include <cstdio>

#include "plan.h"

using namespace cai;

static int g_problems = 0;
static void problem(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    std::fprintf(stderr, "  [FAIL] ");
    std::vfprintf(stderr, fmt, ap);
    std::fputc('\n', stderr);
    va_end(ap);
    ++g_problems;
}
static void warn(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    std::fprintf(stderr, "  [warn] ");
    std::vfprintf(stderr, fmt, ap);
    std::fputc('\n', stderr);
    va_end(ap);
}

int main(int argc, char** argv) {
    if (argc != 2) { std::fprintf(stderr, "usage: %s <config>\n", argv[0]); return 2; }
    Config cfg;
    std::string err;
    if (config_load(argv[1], &cfg, &err) != OK) { std::fprintf(stderr, "config error: %s\n", err.c_str()); return 1; }
    if (topology_finalize(&cfg.topo, &err) != OK) { std::fprintf(stderr, "[FAIL] topology: %s\n", err.c_str()); return 1; }
    Decomp d;
    if (decompose(cfg, &d, &err) != OK) { std::fprintf(stderr, "[FAIL] decompose: %s\n", err.c_str()); return 1; }
    std::printf("=== decomposition ===\n");
    const bool fits = report_decomp(stdout, cfg, d);
    std::printf("=====================\n");
    const Topology& t = cfg.topo;
    std::printf("checks:\n");
    if (!fits) problem("per-GPU memory over budget");
    if (d.tp > t.gpus_per_rack) problem("TP=%u exceeds gpus_per_rack=%u (spans NVLink domains)", d.tp, t.gpus_per_rack);
    else if (t.gpus_per_rack % d.tp) warn("TP=%u does not divide gpus_per_rack=%u; some TP groups cross racks", d.tp, t.gpus_per_rack);
    else std::printf("  [ok]   TP=%u fits intra-rack (%u groups/rack)\n", d.tp, t.gpus_per_rack / d.tp);
    const uint32_t probes[] = {0, t.gpus_per_rack - 1, t.gpus_per_rack, t.world_size - 1};
    for (uint32_t r : probes) {
        if (r >= t.world_size) continue;
        const PhysId p = phys_of_rank(t, r);
        const uint32_t back = rank_of(t, p.rack_id, p.tray_id, p.gpu_in_tray);
        if (back != r) problem("rank %u maps to (rack %u,tray %u,gpu %u) but back to %u", r, p.rack_id, p.tray_id, p.gpu_in_tray, back);
        else std::printf("  [ok]   rank %u -> rack %u tray %u gpu %u (nic %u rail %u)\n", r, p.rack_id, p.tray_id, p.gpu_in_tray, p.nic_id, p.rail_id);
    }
    if (d.bubble_ratio > 0.25) warn("pipeline bubble %.1f%% is high; raise grad_accum or lower PP", d.bubble_ratio * 100.0);
    if (g_problems) std::printf("\nRESULT: %d problem(s)\n", g_problems);
    else std::printf("\nRESULT: all checks passed\n");
    return g_problems ? 1 : 0;
}
