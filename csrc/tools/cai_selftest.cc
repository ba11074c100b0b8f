// cai_selftest - unit tests of the GPU-free library, one binary, exit code = number of failures.
//
// Covers what the reference's tests/cai_test.c covers (topology math, arena packing, 1F1B schedule,
// decomposition, plan round trip, cost model, expert-parallel memory, group tiling, spare ranks)
// plus the executable-plan checks that are new here (event order, hazard analysis, pipeline
// pairing, checkpoint files, golden hashes of the bundled configs).
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <set>

#include "cai.h"
#include "backend.h"
#include "plan.h"

using namespace cai;

static int g_fail = 0, g_checks = 0;
#define CHECK(cond, ...)                                   \
    do {                                                   \
        ++g_checks;                                        \
        if (!(cond)) {                                     \
            ++g_fail;                                      \
            std::printf("FAIL %s:%d: ", __FILE__, __LINE__); \
            std::printf(__VA_ARGS__);                      \
            std::printf("\n");                             \
        }                                                  \
    } while (0)

static Config small_cfg() {
    Config c;
    config_defaults(&c);
    ModelSpec& m = c.model;
    m.hidden_size = 4096; m.ffn_hidden = 14336; m.num_layers = 24; m.num_heads = 32; m.num_kv_heads = 8;
    m.head_dim = 128; m.vocab_size = 128000; m.seq_len = 4096;
    m.tp = 4; m.pp = 3; m.grad_accum = 12; m.microbatch = 1; m.recompute = 1;
    c.topo.gpus_per_rack = 72; c.topo.num_racks = 1;
    return c;
}

static void test_topology() {
    Topology t;
    topology_default(&t);
    t.num_racks = 3056;
    std::string err;
    CHECK(topology_finalize(&t, &err) == OK, "finalize: %s", err.c_str());
    CHECK(t.world_size == 220032, "world %u", t.world_size);
    for (uint32_t r : {0u, 1u, 71u, 72u, 73u, 100000u, 220031u}) {
        const PhysId p = phys_of_rank(t, r);
        CHECK(rank_of(t, p.rack_id, p.tray_id, p.gpu_in_tray) == r, "round trip of rank %u", r);
        CHECK(p.gpu_in_rack == r % 72 && p.rack_id == r / 72, "coords of rank %u", r);
    }
    CHECK(same_rack(t, 0, 71) && !same_rack(t, 71, 72), "same_rack");
    Topology bad = t;
    bad.trays_per_rack = 5;
    CHECK(topology_finalize(&bad, &err) == ERR_TOPOLOGY, "inconsistent trays accepted");
    CHECK(topology_hash(t) != topology_hash(bad), "hash ignores fields");
}

static void test_arena() {
    const uint64_t want[TC_COUNT] = {1000, 513, 0, 7, 4096, 1};
    Arena a;
    arena_layout(&a, want);
    uint64_t prev_end = 0;
    for (int c = 0; c < TC_COUNT; ++c) {
        CHECK(a.seg_off[c] % 512 == 0, "segment %d not aligned", c);
        CHECK(a.seg_off[c] >= prev_end, "segment %d overlaps", c);
        CHECK(a.seg_len[c] == want[c], "segment %d length", c);
        prev_end = a.seg_off[c] + a.seg_len[c];
    }
    CHECK(a.total % 512 == 0 && a.total >= prev_end, "total");
    TensorDesc t{};
    t.tclass = TC_COMM;
    t.offset = 16;
    arena_relocate(a, &t, 1);
    CHECK(t.offset == a.seg_off[TC_COMM] + 16, "relocate");
}

static void test_pipeline() {
    CHECK(std::fabs(pipeline_bubble(16, 128) - 15.0 / 143.0) < 1e-12, "bubble 16/128");
    CHECK(pipeline_bubble(1, 8) == 0.0 && pipeline_bubble(4, 0) == 0.0, "degenerate bubble");
    CHECK(pipeline_bubble_interleaved(3, 12, 2) < pipeline_bubble_interleaved(3, 12, 1), "vpp lowers bubble");
    CHECK(std::fabs(pipeline_bubble_interleaved(3, 12, 2) - 2.0 / 26.0) < 1e-12, "vpp=2 value");
    const uint32_t pp = 4, m = 8;
    for (uint32_t s = 0; s < pp; ++s) {
        const std::vector<Tick> t = schedule_1f1b(s, pp, m);
        CHECK(t.size() == 2 * m, "stage %u has %zu ticks", s, t.size());
        std::vector<int> f(m, -1), b(m, -1);
        for (size_t i = 0; i < t.size(); ++i) (t[i].kind == 0 ? f : b)[t[i].microbatch] = static_cast<int>(i);
        int in_flight = 0, max_in_flight = 0;
        for (const Tick& k : t) {
            in_flight += k.kind == 0 ? 1 : -1;
            max_in_flight = std::max(max_in_flight, in_flight);
        }
        CHECK(max_in_flight == static_cast<int>(pp - s), "stage %u keeps %d microbatches in flight", s, max_in_flight);
        for (uint32_t k = 0; k < m; ++k) CHECK(f[k] >= 0 && b[k] > f[k], "stage %u mb %u order", s, k);
    }
}

static void test_decompose() {
    Config c = small_cfg();
    Decomp d;
    std::string err;
    CHECK(decompose(c, &d, &err) == OK, "%s", err.c_str());
    CHECK(d.model_replica_gpus == 12 && d.dp == 6 && d.global_batch == 72, "replica %u dp %u gb %llu",
          d.model_replica_gpus, d.dp, (unsigned long long)d.global_batch);
    CHECK(d.total_params > 5700000000ull && d.total_params < 5800000000ull, "params %llu", (unsigned long long)d.total_params);
    Config bad = c;
    bad.model.tp = 5;
    CHECK(decompose(bad, &d, &err) == ERR_INVALID, "tp=5 accepted");
    bad = c;
    bad.model.vpp = 5;
    CHECK(decompose(bad, &d, &err) == ERR_INVALID, "vpp=5 accepted");
    bad = c;
    bad.model.vpp = 2;
    Decomp d2;
    CHECK(decompose(bad, &d2, &err) == OK && d2.bubble_ratio < pipeline_bubble(3, 12), "vpp=2");
    bad = c;
    bad.model.pp = 100;
    CHECK(decompose(bad, &d, &err) == ERR_INVALID, "pp > layers accepted");
}

static void test_plan_roundtrip() {
    Config c = small_cfg();
    std::string err;
    topology_finalize(&c.topo, &err);
    Decomp d;
    decompose(c, &d, &err);
    const uint64_t ph = plan_hash(c, d), th = topology_hash(c.topo);
    CHECK(ph == 0x61eec02c9563ad48ull, "small.cfg plan_hash %016llx", (unsigned long long)ph);
    CHECK(th == 0xa6628b5f000e9efaull, "small.cfg topology_hash %016llx", (unsigned long long)th);
    Plan p, q;
    CHECK(build_plan_v1(c, d, 4, ph, th, &p, &err) == OK, "%s", err.c_str());
    CHECK(p.hdr.pipeline_stage == 1 && p.ops.size() == 3327 && p.hdr.num_events == 721, "stage %u ops %zu events %u",
          p.hdr.pipeline_stage, p.ops.size(), p.hdr.num_events);
    CHECK(p.hdr.arena_bytes == 1959259136ull, "arena %llu", (unsigned long long)p.hdr.arena_bytes);
    const std::string path = "/tmp/cai_selftest_plan.bin";
    CHECK(plan_write(path, p) == OK, "write");
    CHECK(plan_read(path, &q) == OK, "read");
    CHECK(std::memcmp(&p.hdr, &q.hdr, sizeof p.hdr) == 0, "header differs");
    CHECK(p.ops.size() == q.ops.size() && std::memcmp(p.ops.data(), q.ops.data(), p.ops.size() * sizeof(Op)) == 0, "ops differ");
    CHECK(std::memcmp(p.groups.data(), q.groups.data(), p.groups.size() * sizeof(CommGroup)) == 0, "groups differ");
    uint64_t by_class[TC_COUNT];
    plan_arena_breakdown(q, by_class);
    uint64_t sum = 0;
    for (uint64_t b : by_class) sum += b;
    CHECK(sum <= q.hdr.arena_bytes, "breakdown exceeds arena");
    Config c2 = c;
    c2.topo.num_racks = 2;
    topology_finalize(&c2.topo, &err);
    CHECK(topology_hash(c2.topo) != th, "topology hash insensitive");
    std::remove(path.c_str());
}

static void test_costmodel() {
    // replay single-op plans through the public runtime API
    Config c = small_cfg();
    std::string err;
    c.topo.num_racks = 20;
    c.model.tp = 8; c.model.pp = 1;
    topology_finalize(&c.topo, &err);
    Decomp d;
    CHECK(decompose(c, &d, &err) == OK, "%s", err.c_str());
    const uint64_t ph = plan_hash(c, d), th = topology_hash(c.topo);
    topology_write("/tmp/cai_selftest_topo.bin", c.topo);
    auto time_of = [&](Op op, CommGroup g) {
        Plan p;
        build_plan_v1(c, d, 0, ph, th, &p, &err);
        p.ops.assign(1, op);
        p.groups.assign(1, g);
        p.hdr.num_ops = 1; p.hdr.num_groups = 1; p.hdr.num_events = 0;
        p.hdr.num_stages = 1;
        plan_write("/tmp/cai_selftest_one.bin", p);
        cai_init_desc_t desc{};
        desc.plan_path = "/tmp/cai_selftest_one.bin";
        desc.topology_path = "/tmp/cai_selftest_topo.bin";
        cai_context_t* ctx = nullptr;
        log_set_level(LOG_ERROR);
        if (cai_init(&ctx, &desc) != 0) return -1.0;
        cai_batch_t b;
        cai_next_batch(ctx, &b);
        cai_train_step(ctx, &b);
        cai_step_stats_t st;
        cai_last_step_stats(ctx, &st);
        cai_finalize(ctx);
        return st.step_time_s;
    };
    Op ar{};
    ar.kind = OP_ALL_REDUCE; ar.stream_id = ST_COMM_TP; ar.bytes = 1 << 26;
    CommGroup g{0, GROUP_TP, 1, 8, 0};
    const double intra = time_of(ar, g);
    g.intra_rack = 0;
    const double inter = time_of(ar, g);
    g.size = 1024;
    const double big = time_of(ar, g);
    CHECK(intra > 0 && intra < inter, "intra %g inter %g", intra, inter);
    CHECK(big > inter, "1024-rank all-reduce not slower");
    Op gm{};
    gm.kind = OP_GEMM; gm.stream_id = ST_COMPUTE_HI; gm.flops = static_cast<uint64_t>(c.topo.gpu_flops_bf16);
    CHECK(std::fabs(time_of(gm, g) - 1.0) < 1e-6, "peak-flops GEMM should take 1 s");
}

static void test_ep_memory() {
    Config c;
    config_load("configs/full220k_moe.cfg", &c, nullptr);
    std::string err;
    Decomp a, b;
    c.model.ep = 191;
    const int ra = decompose(c, &a, &err);
    c.model.ep = 9;
    const int rb = decompose(c, &b, &err);
    CHECK(ra == OK && rb == OK, "moe decompose: %s", err.c_str());
    if (ra == OK && rb == OK) CHECK(a.mem_param < b.mem_param, "larger ep should shrink param memory");
}

static void test_grouptiling_and_spare() {
    Config c = small_cfg();
    std::string err;
    topology_finalize(&c.topo, &err);
    Decomp d;
    decompose(c, &d, &err);
    VerifyReport rep;
    verify_tiling(d, c.topo, false, GROUP_TP, "TP", &rep);
    verify_tiling(d, c.topo, false, GROUP_DP, "DP", &rep);
    verify_tiling(d, c.topo, false, GROUP_PP, "PP", &rep);
    CHECK(rep.problems == 0, "tiling problems: %d", rep.problems);
    // members lists are consistent with the coordinates
    const std::vector<uint32_t> tpm = group_members(d, false, GROUP_TP, 5), ppm = group_members(d, false, GROUP_PP, 5),
                                dpm = group_members(d, false, GROUP_DP, 5);
    CHECK(tpm == (std::vector<uint32_t>{4, 5, 6, 7}), "tp members");
    CHECK(ppm == (std::vector<uint32_t>{1, 5, 9}), "pp members");
    CHECK(dpm.size() == 6 && dpm[0] == 5 && dpm[1] == 17, "dp members");

    Topology t = c.topo;
    t.num_racks = 2;
    t.spare_gpus = 4;
    topology_finalize(&t, &err);
    uint32_t spare = 0;
    CHECK(spare_rank(t, 100, &spare) == OK && spare >= t.world_size, "spare pick");
    CHECK(spare_rank(t, 3, &spare) == OK && spare / 72 != 0, "spare %u should sit in another rack", spare);
    t.spare_gpus = 0;
    topology_finalize(&t, &err);
    CHECK(spare_rank(t, 3, &spare) != OK, "no spares but got one");
}

static void test_config_parser() {
    Config c;
    std::string err;
    CHECK(config_parse("hidden_size = 1024 # comment\n\n gpu_mem_bytes=288e9\nparam_dtype = fp8e4m3\n", &c, &err) == OK, "%s", err.c_str());
    CHECK(c.model.hidden_size == 1024 && c.topo.gpu_mem_bytes == 288000000000ull && c.model.param_dtype == DT_FP8_E4M3, "values");
    CHECK(config_parse("bogus_key = 3\n", &c, &err) == ERR_INVALID && err.find("line 1") != std::string::npos, "unknown key: %s", err.c_str());
    CHECK(config_parse("tp = 2\nthis line has no equals\n", &c, &err) == ERR_INVALID && err.find("line 2") != std::string::npos, "%s", err.c_str());
    CHECK(config_parse("lr = 3e-4\ncomm = baseline\nseed = 7\n", &c, &err) == OK && c.train.comm_mode == 0 && c.train.seed == 7, "train keys");
    CHECK(sizeof(ModelSpec) == 96, "ModelSpec size");
}

static void test_exec_plans() {
    for (const char* path : {"configs/tiny.cfg", "configs/b200_tp8.cfg", "configs/b200_pp2tp4.cfg", "configs/tiny_moe.cfg",
                             "configs/b200_moe_ep8.cfg"}) {
        for (const char* mode : {"fused", "baseline"}) {
            Config c;
            std::string err;
            if (config_load(path, &c, &err) != OK) { CHECK(false, "%s: %s", path, err.c_str()); continue; }
            c.train.comm_mode = std::strcmp(mode, "fused") == 0;
            if (c.model.is_moe && !c.train.comm_mode) {
                // expert exchange exists only as in-kernel dispatch / combine: a baseline plan must be refused
                topology_finalize(&c.topo, &err);
                Decomp dm;
                Plan pm;
                CHECK(decompose(c, &dm, &err) == OK && build_plan_v2(c, dm, 0, 0, 0, &pm, &err) == ERR_INVALID, "%s: baseline MoE", path);
                continue;
            }
            topology_finalize(&c.topo, &err);
            Decomp d;
            CHECK(decompose(c, &d, &err) == OK, "%s", err.c_str());
            const uint64_t ph = plan_hash(c, d), th = topology_hash(c.topo);
            std::vector<Plan> stages;
            for (uint32_t s = 0; s < d.pp; ++s) {
                Plan p;
                CHECK(build_plan_v2(c, d, s * d.tp * d.cp, ph, th, &p, &err) == OK, "%s: %s", path, err.c_str());
                VerifyReport rep;
                verify_event_order(p, &rep);
                verify_hazards(p, &rep);
                CHECK(rep.problems == 0, "%s (%s) stage %u: %d problems: %s", path, mode, s, rep.problems,
                      rep.lines.empty() ? "" : rep.lines.back().c_str());
                for (const TensorDesc& t : p.tensors) CHECK(t.offset + t.nbytes <= p.hdr.arena_bytes, "tensor outside arena");
                // file round trip keeps the execution section
                CHECK(plan_write("/tmp/cai_selftest_x.bin", p) == OK, "write v2");
                Plan q;
                CHECK(plan_read("/tmp/cai_selftest_x.bin", &q) == OK && q.exec.size() == p.exec.size() &&
                          q.named.size() == p.named.size() && q.shapes == p.shapes,
                      "v2 round trip");
                stages.push_back(std::move(p));
            }
            VerifyReport rep;
            verify_pipeline_pairing(stages, &rep);
            CHECK(rep.problems == 0, "%s: pipeline pairing", path);
        }
    }
    // a deliberately broken schedule must be caught: drop every wait of the tp8 baseline plan
    Config c;
    std::string err;
    config_load("configs/b200_tp8.cfg", &c, &err);
    c.train.comm_mode = 0;
    topology_finalize(&c.topo, &err);
    Decomp d;
    decompose(c, &d, &err);
    Plan p;
    build_plan_v2(c, d, 0, plan_hash(c, d), topology_hash(c.topo), &p, &err);
    std::vector<Op> kept;
    for (const Op& o : p.ops)
        if (o.kind != OP_EVENT_WAIT) kept.push_back(o);
    p.ops = kept;
    VerifyReport rep;
    verify_hazards(p, &rep);
    CHECK(rep.problems > 0, "hazard checker missed a schedule without waits");

    // Cross-rank reuse: the fused tp = 8 plan passes; turn every all-gather -> GEMM into a plain GEMM (so that two
    // reduce-scatters follow each other with nothing that orders the group in between) and the proof must fail.
    {
        Config cf;
        config_load("configs/b200_tp8.cfg", &cf, &err);
        cf.train.comm_mode = 1;
        topology_finalize(&cf.topo, &err);
        Decomp df;
        decompose(cf, &df, &err);
        Plan pf;
        CHECK(build_plan_v2(cf, df, 0, plan_hash(cf, df), topology_hash(cf.topo), &pf, &err) == OK, "fused tp8 plan: %s", err.c_str());
        VerifyReport good;
        verify_peer_reuse(pf, &good);
        CHECK(good.problems == 0 && !good.lines.empty(), "peer reuse of the fused tp8 plan: %d problems", good.problems);
        for (ExecOp& x : pf.exec)
            if (x.kernel == K_AG_GEMM) x.kernel = K_GEMM;
        VerifyReport bad;
        verify_peer_reuse(pf, &bad);
        CHECK(bad.problems > 0, "peer-reuse proof missed reduce-scatters that share a staging buffer without a group-ordering op");
    }

    // Expert exchange: the ep = 8 plan passes; without the combine's entry hand-shake (announce flag cleared) a member
    // would load expert outputs its peers may not have written yet, and the proof must say so.
    {
        Config cf;
        config_load("configs/b200_moe_ep8.cfg", &cf, &err);
        cf.train.comm_mode = 1;
        topology_finalize(&cf.topo, &err);
        Decomp df;
        decompose(cf, &df, &err);
        Plan pf;
        CHECK(build_plan_v2(cf, df, 0, plan_hash(cf, df), topology_hash(cf.topo), &pf, &err) == OK, "moe ep8 plan: %s", err.c_str());
        VerifyReport good;
        verify_peer_reuse(pf, &good);
        bool said = false;
        for (const std::string& l : good.lines) said = said || l.find("slabs of the expert exchange") != std::string::npos;
        CHECK(good.problems == 0 && said, "expert-exchange reuse of the ep8 plan: %d problems", good.problems);
        for (ExecOp& x : pf.exec)
            if (x.kernel == K_MOE_GEMM_COMBINE) x.flags &= static_cast<uint16_t>(~1u);
        VerifyReport bad;
        verify_peer_reuse(pf, &bad);
        CHECK(bad.problems > 0, "expert-exchange proof missed combines that load from peers without a hand-shake");
    }

    // Column views: two unordered writers on different streams are fine when they cover disjoint columns of
    // the same rows (dQ beside dK/dV), and a hazard as soon as the column intervals touch.
    for (int overlap = 0; overlap < 2; ++overlap) {
        Plan q;
        q.hdr.version = 2;
        auto tensor = [&](uint64_t off, uint32_t rows, uint32_t cols, uint32_t ld) {
            TensorDesc t{};
            t.offset = off; t.dtype = DT_BF16; t.tclass = TC_WORKSPACE;
            t.nbytes = (static_cast<uint64_t>(rows - 1) * ld + cols) * 2;
            q.tensors.push_back(t);
            q.shapes.insert(q.shapes.end(), {rows, cols, ld, 1u});
            return static_cast<int>(q.tensors.size()) - 1;
        };
        const int left = tensor(1024, 64, 256, 768);                                // columns [0, 256) of a [64, 768] buffer
        const int right = tensor(1024 + (overlap ? 255 : 256) * 2, 64, 512, 768);   // columns [256, 768) or one column early
        for (int k = 0; k < 2; ++k) {
            ExecOp x{};
            for (int& t : x.t) t = -1;
            x.kernel = K_ZERO;
            x.t[0] = k ? right : left;
            q.exec.push_back(x);
            Op o{};
            o.kind = OP_ELEMENTWISE;
            o.stream_id = k ? ST_COMM_DP : ST_COMPUTE_HI;
            o.exec = static_cast<uint32_t>(q.exec.size());
            q.ops.push_back(o);
        }
        VerifyReport r2;
        verify_hazards(q, &r2);
        CHECK((r2.problems > 0) == (overlap == 1), "column views, overlap=%d: %d problems", overlap, r2.problems);
    }
}

static void test_checkpoint_files() {
    const char* base = "/tmp/cai_selftest_ckpt";
    const float w[4] = {1, 2, 3, 4};
    const double v[2] = {5, 6};
    const char* names[2] = {"weights", "moments"};
    const void* data[2] = {w, v};
    const uint64_t nbytes[2] = {sizeof w, sizeof v};
    CHECK(cai_ckpt_write(base, "periodic", 3, 17, 0xabcdefull, 2, names, data, nbytes) == 0, "write");
    uint32_t step = 0, nsec = 0;
    uint64_t ph = 0;
    char file[512];
    CHECK(cai_ckpt_probe(base, 3, &step, &ph, &nsec, file, sizeof file) == 0 && step == 17 && ph == 0xabcdefull && nsec == 2, "probe");
    CHECK(std::strstr(file, ".latest.rank000003") != nullptr, "latest pointer: %s", file);
    char name[16];
    uint64_t n = 0;
    double back[2] = {0, 0};
    CHECK(cai_ckpt_section(file, 1, name, &n, back, sizeof back) == 0 && n == sizeof v && back[1] == 6 && !std::strcmp(name, "moments"), "section");
    CHECK(cai_ckpt_probe("/tmp/cai_selftest_nothing_here", 0, &step, &ph, &nsec, file, sizeof file) == 1, "missing checkpoint");
    // the first 12 bytes keep the reference's layout: u32 step, u64 plan_hash
    FILE* f = std::fopen(file, "rb");
    uint32_t s2 = 0;
    uint64_t h2 = 0;
    CHECK(f && std::fread(&s2, 4, 1, f) == 1 && std::fread(&h2, 8, 1, f) == 1 && s2 == 17 && h2 == 0xabcdefull, "prefix");
    if (f) std::fclose(f);
}

// The calibrated pricing backend through the public C API: a version-2 plan replayed with measured kernel costs takes
// longer than with the datasheet model, streams overlap only as far as the SMs allow, and a calibration file with an
// unknown key is refused at cai_init.
static void test_calibrated_backend() {
    Config c;
    std::string err;
    if (config_load("configs/b200_tp8.cfg", &c, &err) != OK) { CHECK(false, "%s", err.c_str()); return; }
    topology_finalize(&c.topo, &err);
    Decomp d;
    CHECK(decompose(c, &d, &err) == OK, "%s", err.c_str());
    Plan p;
    CHECK(build_plan_v2(c, d, 0, plan_hash(c, d), topology_hash(c.topo), &p, &err) == OK, "%s", err.c_str());
    CHECK(plan_write("/tmp/cai_selftest_cal.bin", p) == OK && topology_write("/tmp/cai_selftest_cal_topo.bin", c.topo) == OK, "write");
    double t[2] = {0, 0};
    for (int k = 0; k < 2; ++k) {
        cai_init_desc_t desc{};
        desc.plan_path = "/tmp/cai_selftest_cal.bin";
        desc.topology_path = "/tmp/cai_selftest_cal_topo.bin";
        desc.backend = k ? CAI_BACKEND_CALIBRATED : CAI_BACKEND_ANALYTIC;
        unsetenv("CAI_CALIBRATION");
        cai_context_t* ctx = nullptr;
        CHECK(cai_init(&ctx, &desc) == 0, "cai_init backend %d", k);
        if (!ctx) return;
        CHECK(!std::strcmp(cai_backend_name(ctx), k ? "calibrated" : "analytic"), "backend name");
        CHECK(cai_train_step(ctx, nullptr) == 0, "step");
        cai_step_stats_t st;
        cai_last_step_stats(ctx, &st);
        t[k] = st.step_time_s;
        if (k) CHECK(st.step_time_s >= st.stream_busy[ST_COMPUTE_HI] * 0.9999 &&
                     st.step_time_s <= (st.stream_busy[ST_COMPUTE_HI] + st.stream_busy[ST_COMPUTE_LO]) * 1.0001, "SM-work bound");
        cai_finalize(ctx);
    }
    CHECK(t[1] > 2.0 * t[0] && t[1] > 0.08 && t[1] < 0.13, "calibrated %.4f s against analytic %.4f s (measured: 0.108 s)", t[1], t[0]);
    FILE* f = std::fopen("/tmp/cai_selftest_cal_bad.cfg", "w");
    if (f) {
        std::fputs("no_such_constant = 1\n", f);
        std::fclose(f);
    }
    setenv("CAI_CALIBRATION", "/tmp/cai_selftest_cal_bad.cfg", 1);
    cai_init_desc_t desc{};
    desc.plan_path = "/tmp/cai_selftest_cal.bin";
    desc.topology_path = "/tmp/cai_selftest_cal_topo.bin";
    desc.backend = CAI_BACKEND_CALIBRATED;
    cai_context_t* ctx = nullptr;
    CHECK(cai_init(&ctx, &desc) != 0, "unknown calibration key accepted");
    unsetenv("CAI_CALIBRATION");
}

// Joint replay of the stages of a pipeline: a healthy schedule replays, a missing receive is counted, and a schedule in
// which two stages wait for each other (a gradient receive moved in front of the first activation send on the same
// in-order stream) is reported as a deadlock instead of producing a time.
static void test_pipeline_replay() {
    Config c;
    std::string err;
    if (config_load("configs/b200_pp2tp4.cfg", &c, &err) != OK) { CHECK(false, "%s", err.c_str()); return; }
    topology_finalize(&c.topo, &err);
    Decomp d;
    CHECK(decompose(c, &d, &err) == OK, "%s", err.c_str());
    const uint64_t ph = plan_hash(c, d), th = topology_hash(c.topo);
    Plan st0, st1;
    CHECK(build_plan_v2(c, d, 0, ph, th, &st0, &err) == OK, "%s", err.c_str());
    CHECK(build_plan_v2(c, d, d.tp * d.cp, ph, th, &st1, &err) == OK, "%s", err.c_str());
    Backend* be = backend_analytic_create();
    PipelineResult r;
    CHECK(replay_pipeline({&st0, &st1}, c.topo, be, &r, &err) == OK, "healthy pipeline: %s", err.c_str());
    CHECK(r.stages.size() == 2 && r.step_time_s > 0 && r.step_time_s >= r.stages[0].stream_busy[ST_COMPUTE_HI], "step %.4f", r.step_time_s);
    CHECK(replay_pipeline({&st1, &st0}, c.topo, be, &r, &err) == ERR_PLAN, "stages in the wrong order accepted");
    {   // one receive fewer on the upper stage
        Plan broken = st1;
        for (size_t i = 0; i < broken.ops.size(); ++i)
            if (broken.ops[i].kind == OP_PIPE_RECV) { broken.ops.erase(broken.ops.begin() + static_cast<long>(i)); break; }
        CHECK(replay_pipeline({&st0, &broken}, c.topo, be, &r, &err) == ERR_DEPENDENCY && err.find("receives") != std::string::npos,
              "missing receive: %s", err.c_str());
    }
    {   // stage 0 posts its first gradient receive in front of its first activation send, on the same stream
        Plan broken = st0;
        size_t first_send = broken.ops.size(), first_recv = broken.ops.size();
        for (size_t i = 0; i < broken.ops.size(); ++i) {
            if (broken.ops[i].kind == OP_PIPE_SEND && first_send == broken.ops.size()) first_send = i;
            if (broken.ops[i].kind == OP_PIPE_RECV && first_recv == broken.ops.size()) first_recv = i;
        }
        CHECK(first_send < first_recv && first_recv < broken.ops.size(), "stage 0 sends before it receives");
        if (first_send < first_recv && first_recv < broken.ops.size()) {
            Op moved = broken.ops[first_recv];
            moved.stream_id = broken.ops[first_send].stream_id;
            broken.ops.erase(broken.ops.begin() + static_cast<long>(first_recv));
            broken.ops.insert(broken.ops.begin() + static_cast<long>(first_send), moved);
            CHECK(replay_pipeline({&broken, &st1}, c.topo, be, &r, &err) == ERR_DEPENDENCY && err.find("deadlock") != std::string::npos,
                  "deadlock not reported: %s", err.c_str());
        }
    }
    be->destroy(be);
}

int main() {
    log_set_level(LOG_ERROR);
    test_topology();
    test_arena();
    test_pipeline();
    test_decompose();
    test_plan_roundtrip();
    test_costmodel();
    test_ep_memory();
    test_grouptiling_and_spare();
    test_config_parser();
    test_exec_plans();
    test_checkpoint_files();
    test_calibrated_backend();
    test_pipeline_replay();
    std::printf("%d checks, %d failures\n", g_checks, g_fail);
    return g_fail ? 1 : 0;
}
