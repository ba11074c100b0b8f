// plan_verify <config> [--exec] [--dir PLANDIR]
//
// Whole-cluster proof before launch, no GPU needed: communicators tile the world, all stages
// agree on the hashes, pipeline sends and receives are conserved, ranks of one stage emit
// identical op streams (checks 1-4 of the reference's tools/plan_verify.c). With --exec it
// also builds the executable plans and proves event order, absence of cross-stream data hazards on
// the arena and pairwise send/receive order. With --dir it additionally checks that the plan
// files on disk carry the hashes this config produces.
#include <dirent.h>

#include <cstdio>
#include <cstring>
#include <string>
#include <vector>

#include "cai.h"
#include "plan.h"

int main(int argc, char** argv) {
    if (argc < 2) { std::fprintf(stderr, "usage: %s <config> [--exec] [--dir PLANDIR]\n", argv[0]); return 2; }
    int exec = 0;
    const char* dir = nullptr;
    for (int i = 2; i < argc; ++i) {
        if (!std::strcmp(argv[i], "--exec")) exec = 1;
        else if (!std::strcmp(argv[i], "--dir") && i + 1 < argc) dir = argv[++i];
        else { std::fprintf(stderr, "usage: %s <config> [--exec] [--dir PLANDIR]\n", argv[0]); return 2; }
    }
    std::vector<char> report(1 << 20);
    int rc = cai_verify(argv[1], exec, report.data(), report.size());
    std::fputs(report.data(), stdout);
    if (rc < 0) return 1;
    if (dir) {
        uint64_t ph = 0, th = 0;
        char err[256];
        if (cai_compile(argv[1], nullptr, 0, 0, 1, &ph, &th, err, sizeof err) != 0) { std::fprintf(stderr, "%s\n", err); return 1; }
        int bad = 0, seen = 0;
        if (DIR* d = opendir(dir)) {
            while (dirent* e = readdir(d)) {
                if (std::strncmp(e->d_name, "plan.rank", 9) != 0) continue;
                cai::Plan p;
                const std::string path = std::string(dir) + "/" + e->d_name;
                if (cai::plan_read(path, &p) != cai::OK) { std::printf("  [FAIL] %s: unreadable\n", path.c_str()); ++bad; continue; }
                ++seen;
                if (p.hdr.plan_hash != ph || p.hdr.topology_hash != th) { std::printf("  [FAIL] %s: hash mismatch\n", path.c_str()); ++bad; }
            }
            closedir(d);
        } else { std::printf("  [FAIL] cannot open %s\n", dir); ++bad; }
        if (!bad) std::printf("  [ok]   %d plan files in %s carry the expected hashes\n", seen, dir);
        rc += bad;
    }
    return rc ? 1 : 0;
}
