// plan_compiler <config> <outdir> [--rank R | --ranks N | --all | --sample] [--force] [--quiet]
//               [--exec | --v1]
//
// Offline compiler: reads a key = value config, prints the decomposition report, writes
// topology.bin and one plan.rankNNNNNN.bin per requested rank. Command line, file names and
// report text follow the reference tool (tools/plan_compiler.c); `--exec` writes version-2
// (executable) plans instead of cost-only version-1 plans.
#include <cstdio>
#include <fstream>
#include <cstdlib>
#include <cstring>
#include <set>
#include <string>

#include "plan.h"

using namespace cai;

static void usage(const char* p) {
    std::fprintf(stderr,
                 "usage: %s <config> <outdir> [options]\n"
                 "  --rank R     compile only global rank R\n"
                 "  --ranks N    compile ranks [0, N)\n"
                 "  --all        compile every rank (needs --force above 4096)\n"
                 "  --sample     compile a representative handful (default)\n"
                 "  --force      allow large --all\n"
                 "  --quiet      suppress the decomposition report\n"
                 "  --exec       write executable (version 2) plans\n"
                 "  --v1         write cost-only (version 1) plans (default)\n",
                 p);
}

int main(int argc, char** argv) {
    if (argc < 3) { usage(argv[0]); return 2; }
    const std::string cfgpath = argv[1], outdir = argv[2];
    enum { SAMPLE, ONE, RANGE, ALL } mode = SAMPLE;
    bool force = false, quiet = false, exec = false;
    uint32_t arg_rank = 0, arg_n = 0;
    for (int i = 3; i < argc; ++i) {
        const std::string a = argv[i];
        if (a == "--rank" && i + 1 < argc) { mode = ONE; arg_rank = std::strtoul(argv[++i], nullptr, 10); }
        else if (a == "--ranks" && i + 1 < argc) { mode = RANGE; arg_n = std::strtoul(argv[++i], nullptr, 10); }
        else if (a == "--all") mode = ALL;
        else if (a == "--sample") mode = SAMPLE;
        else if (a == "--force") force = true;
        else if (a == "--quiet") quiet = true;
        else if (a == "--exec") exec = true;
        else if (a == "--v1") exec = false;
        else { usage(argv[0]); return 2; }
    }
    Config cfg;
    std::string err;
    if (config_load(cfgpath, &cfg, &err) != OK) { std::fprintf(stderr, "config error: %s\n", err.c_str()); return 1; }
    if (topology_finalize(&cfg.topo, &err) != OK) { std::fprintf(stderr, "topology error: %s\n", err.c_str()); return 1; }
    Decomp d;
    if (decompose(cfg, &d, &err) != OK) { std::fprintf(stderr, "decompose error: %s\n", err.c_str()); return 1; }
    if (!quiet) {
        std::printf("=== decomposition ===\n");
        const bool fits = report_decomp(stdout, cfg, d);
        std::printf("=====================\n");
        if (!fits)
            std::fprintf(stderr, "WARNING: per-GPU memory exceeds budget; adjust tp/pp/dp, recompute, or precision.\n");
    }
    const uint64_t th = topology_hash(cfg.topo), ph = plan_hash(cfg, d);
    if (!mkdir_p(outdir)) { std::fprintf(stderr, "cannot create %s\n", outdir.c_str()); return 1; }
    const std::string tpath = outdir + "/topology.bin";
    if (topology_write(tpath, cfg.topo) != OK) { std::fprintf(stderr, "cannot write %s\n", tpath.c_str()); return 1; }
    std::printf("wrote %s (topology_hash=%016llx, plan_hash=%016llx)\n", tpath.c_str(), (unsigned long long)th,
                (unsigned long long)ph);
    {
        // keep the config next to the plans: the device trainer derives communicator membership from it
        std::ifstream in(cfgpath, std::ios::binary);
        std::ofstream out(outdir + "/config.cfg", std::ios::binary);
        out << in.rdbuf();
    }

    const uint32_t ws = cfg.topo.world_size;
    std::vector<uint32_t> ranks;
    if (mode == ONE) {
        if (arg_rank >= ws) { std::fprintf(stderr, "rank %u out of range (world=%u)\n", arg_rank, ws); return 1; }
        ranks.push_back(arg_rank);
    } else if (mode == RANGE) {
        for (uint32_t r = 0; r < std::min(arg_n, ws); ++r) ranks.push_back(r);
    } else if (mode == ALL) {
        if (ws > 4096 && !force) { std::fprintf(stderr, "refusing to write %u plans without --force\n", ws); return 1; }
        for (uint32_t r = 0; r < ws; ++r) ranks.push_back(r);
    } else {
        std::vector<uint32_t> s{0};
        if (d.pp > 1) s.push_back((d.pp - 1) * d.tp * d.cp);  // last stage
        if (d.dp > 1) s.push_back(d.model_replica_gpus);       // second data-parallel replica
        s.push_back(ws - 1);
        std::printf("compiling %zu sample ranks:\n", s.size());
        std::set<uint32_t> seen;
        for (uint32_t r : s)
            if (seen.insert(r).second) ranks.push_back(r);
    }
    bool failed = false;
    for (uint32_t r : ranks) {
        Plan p;
        const int rc = exec ? build_plan_v2(cfg, d, r, ph, th, &p, &err) : build_plan_v1(cfg, d, r, ph, th, &p, &err);
        if (rc != OK) {
            std::fprintf(stderr, "rank %u: build failed: %s\n", r, err.c_str());
            failed = true;
            continue;
        }
        char name[64];
        std::snprintf(name, sizeof name, "/plan.rank%06u.bin", r);
        const std::string path = outdir + name;
        if (plan_write(path, p) != OK) {
            std::fprintf(stderr, "rank %u: write failed\n", r);
            failed = true;
            continue;
        }
        std::printf("  wrote %s  (stage %u, ops=%u, arena=%.2f GiB)\n", path.c_str(), p.hdr.pipeline_stage, p.hdr.num_ops,
                    p.hdr.arena_bytes / (1024.0 * 1024.0 * 1024.0));
        if (exec) {
            // what this rank's device allocates, class by class (the report above is the reference's memory model)
            uint64_t cb[TC_COUNT];
            plan_class_bytes(p, cb);
            std::printf("    arena by class:");
            for (int c = 0; c < TC_COUNT; ++c) std::printf(" %s=%.2f GiB", tclass_name(static_cast<uint16_t>(c)), cb[c] / (1024.0 * 1024.0 * 1024.0));
            std::printf("\n");
        }
    }
    return failed ? 1 : 0;
}
