// plan_recover <config> <failed_rank> <outdir> [--exec]
//
// Spare-rank substitution: a plan depends only on the logical coordinate of a rank, so recovery
// picks a spare physical GPU (preferring another rack), regenerates the failed rank's identical
// plan and tells the operator where to resume it (reference: tools/plan_recover.c).
#include <cstdio>
#include <cstdlib>
#include <cstring>

#include "plan.h"

using namespace cai;

int main(int argc, char** argv) {
    if (argc < 4) { std::fprintf(stderr, "usage: %s <config> <failed_rank> <outdir> [--exec]\n", argv[0]); return 2; }
    const uint32_t failed = std::strtoul(argv[2], nullptr, 10);
    const std::string outdir = argv[3];
    const bool exec = argc > 4 && !std::strcmp(argv[4], "--exec");
    Config cfg;
    std::string err;
    if (config_load(argv[1], &cfg, &err) != OK) { std::fprintf(stderr, "config error: %s\n", err.c_str()); return 1; }
    if (topology_finalize(&cfg.topo, &err) != OK) { std::fprintf(stderr, "topology: %s\n", err.c_str()); return 1; }
    Decomp d;
    if (decompose(cfg, &d, &err) != OK) { std::fprintf(stderr, "decompose: %s\n", err.c_str()); return 1; }
    if (failed >= cfg.topo.world_size) { std::fprintf(stderr, "failed_rank %u >= world_size %u\n", failed, cfg.topo.world_size); return 1; }
    uint32_t spare = 0;
    if (spare_rank(cfg.topo, failed, &spare) != OK) {
        std::fprintf(stderr, "no spare GPUs available (set spare_gpus > 0 in the config so failures can be absorbed)\n");
        return 1;
    }
    const PhysId fp = phys_of_rank(cfg.topo, failed), sp = phys_of_rank(cfg.topo, spare);
    const uint64_t ph = plan_hash(cfg, d), th = topology_hash(cfg.topo);
    Plan plan;
    const int rc = exec ? build_plan_v2(cfg, d, failed, ph, th, &plan, &err) : build_plan_v1(cfg, d, failed, ph, th, &plan, &err);
    if (rc != OK) { std::fprintf(stderr, "build: %s\n", err.c_str()); return 1; }
    mkdir_p(outdir);
    char name[80];
    std::snprintf(name, sizeof name, "/plan.recover.rank%06u.bin", failed);
    const std::string path = outdir + name;
    if (plan_write(path, plan) != OK) { std::fprintf(stderr, "write %s failed\n", path.c_str()); return 1; }
    std::printf("recovery plan for rank %u:\n", failed);
    std::printf("  failed rank %u  was on rack %u tray %u gpu %u (stage %u)\n", failed, fp.rack_id, fp.tray_id, fp.gpu_in_tray, rank_stage(d, failed));
    std::printf("  spare phys  %u  -> rack %u tray %u gpu %u  [%s rack]\n", spare, sp.rack_id, sp.tray_id, sp.gpu_in_tray, sp.rack_id == fp.rack_id ? "SAME" : "different");
    std::printf("  wrote %s\n", path.c_str());
    std::printf("  resume: load this plan + topology.bin on the spare and restore the latest checkpoint for rank %u\n", failed);
    return 0;
}
