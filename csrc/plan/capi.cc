// capi.cc - C entry points of the compiler half of libcai_host.so (see cai.h).
#include <cstring>
#include <sstream>

#include "cai.h"
#include "backend.h"
#include "plan.h"

using namespace cai;

namespace {

void put_err(char* err, size_t n, const std::string& s) {
    if (err && n) std::snprintf(err, n, "%s", s.c_str());
}

int compile_cfg(Config& cfg, const char* outdir, uint32_t lo, uint32_t hi, uint32_t version, uint64_t* ph_out,
                uint64_t* th_out, char* err, size_t errlen) {
    std::string e;
    if (int rc = topology_finalize(&cfg.topo, &e); rc != OK) { put_err(err, errlen, e); return rc; }
    Decomp d;
    if (int rc = decompose(cfg, &d, &e); rc != OK) { put_err(err, errlen, e); return rc; }
    const uint64_t th = topology_hash(cfg.topo), ph = plan_hash(cfg, d);
    if (ph_out) *ph_out = ph;
    if (th_out) *th_out = th;
    if (!outdir) return OK;
    if (!mkdir_p(outdir)) { put_err(err, errlen, std::string("cannot create ") + outdir); return ERR_IO; }
    if (topology_write(std::string(outdir) + "/topology.bin", cfg.topo) != OK) {
        put_err(err, errlen, "cannot write topology.bin");
        return ERR_IO;
    }
    if (hi > cfg.topo.world_size) hi = cfg.topo.world_size;
    for (uint32_t r = lo; r < hi; ++r) {
        Plan p;
        int rc = version >= 2 ? build_plan_v2(cfg, d, r, ph, th, &p, &e) : build_plan_v1(cfg, d, r, ph, th, &p, &e);
        if (rc != OK) { put_err(err, errlen, e); return rc; }
        char name[64];
        std::snprintf(name, sizeof name, "/plan.rank%06u.bin", r);
        if ((rc = plan_write(std::string(outdir) + name, p)) != OK) { put_err(err, errlen, "cannot write plan"); return rc; }
    }
    return OK;
}

}  // namespace

extern "C" {

int cai_compile(const char* config_path, const char* outdir, uint32_t lo, uint32_t hi, uint32_t version,
                uint64_t* ph, uint64_t* th, char* err, size_t errlen) {
    Config cfg;
    std::string e;
    if (int rc = config_load(config_path, &cfg, &e); rc != OK) { put_err(err, errlen, e); return rc; }
    return compile_cfg(cfg, outdir, lo, hi, version, ph, th, err, errlen);
}

int cai_compile_text(const char* text, const char* outdir, uint32_t lo, uint32_t hi, uint32_t version, uint64_t* ph,
                     uint64_t* th, char* err, size_t errlen) {
    Config cfg;
    std::string e;
    if (int rc = config_parse(text, &cfg, &e); rc != OK) { put_err(err, errlen, e); return rc; }
    return compile_cfg(cfg, outdir, lo, hi, version, ph, th, err, errlen);
}

int cai_describe(const char* text, char* out, size_t out_len, char* err, size_t errlen) {
    Config cfg;
    std::string e;
    if (int rc = config_parse(text, &cfg, &e); rc != OK) { put_err(err, errlen, e); return rc; }
    if (int rc = topology_finalize(&cfg.topo, &e); rc != OK) { put_err(err, errlen, e); return rc; }
    Decomp d;
    if (int rc = decompose(cfg, &d, &e); rc != OK) { put_err(err, errlen, e); return rc; }
    std::ostringstream o;
    const ModelSpec& m = cfg.model;
    o << "world_size=" << cfg.topo.world_size << "\nspare_gpus=" << cfg.topo.spare_gpus << "\ntp=" << d.tp << "\npp=" << d.pp << "\ndp=" << d.dp << "\nep=" << d.ep
      << "\ncp=" << d.cp << "\nvpp=" << d.vpp << "\nreplica=" << d.model_replica_gpus << "\nglobal_batch=" << d.global_batch
      << "\nglobal_tokens=" << d.global_tokens << "\nnum_microbatches=" << d.num_microbatches
      << "\nlayers_per_stage=" << d.layers_per_stage << "\nbubble_ratio=" << d.bubble_ratio
      << "\ntotal_params=" << d.total_params << "\nactive_params=" << d.active_params
      << "\nflops_per_token_useful=" << static_cast<uint64_t>(d.flops_per_token_useful)
      << "\nflops_per_token_train=" << static_cast<uint64_t>(d.flops_per_token_train) << "\nmem_param=" << d.mem_param
      << "\nmem_grad=" << d.mem_grad << "\nmem_opt=" << d.mem_opt << "\nmem_act=" << d.mem_act << "\nmem_comm=" << d.mem_comm
      << "\nmem_ws=" << d.mem_ws << "\nmem_total=" << d.mem_total << "\nmem_budget=" << mem_budget(cfg)
      << "\nplan_hash=" << plan_hash(cfg, d) << "\ntopology_hash=" << topology_hash(cfg.topo)
      << "\nhidden_size=" << m.hidden_size << "\nffn_hidden=" << m.ffn_hidden << "\nnum_layers=" << m.num_layers
      << "\nnum_heads=" << m.num_heads << "\nnum_kv_heads=" << m.num_kv_heads << "\nhead_dim=" << m.head_dim
      << "\nvocab_size=" << m.vocab_size << "\nseq_len=" << m.seq_len << "\nmicrobatch=" << m.microbatch
      << "\ngrad_accum=" << m.grad_accum << "\nis_moe=" << m.is_moe << "\nnum_experts=" << m.num_experts
      << "\nmoe_top_k=" << m.moe_top_k << "\nparam_dtype=" << dtype_name(m.param_dtype) << "\nrecompute=" << m.recompute
      << "\ngpu_flops_bf16=" << cfg.topo.gpu_flops_bf16 << "\nlr=" << cfg.train.lr << "\nseed=" << cfg.train.seed
      << "\ncomm_mode=" << cfg.train.comm_mode << "\ninit_std=" << cfg.train.init_std << "\nrope_theta=" << cfg.train.rope_theta
      << "\n";
    const std::string s = o.str();
    if (s.size() + 1 > out_len) { put_err(err, errlen, "output buffer too small"); return ERR_INVALID; }
    std::memcpy(out, s.c_str(), s.size() + 1);
    return OK;
}

int cai_group_members(const char* text, uint16_t kind, uint32_t rank, uint32_t* out, uint32_t cap) {
    Config cfg;
    std::string e;
    if (config_parse(text, &cfg, &e) != OK || topology_finalize(&cfg.topo, &e) != OK) return ERR_INVALID;
    Decomp d;
    if (decompose(cfg, &d, &e) != OK) return ERR_INVALID;
    const std::vector<uint32_t> m = group_members(d, cfg.model.is_moe != 0, kind, rank);
    if (m.size() > cap) return ERR_INVALID;
    for (size_t i = 0; i < m.size(); ++i) out[i] = m[i];
    return static_cast<int>(m.size());
}

int cai_lint(const char* config_path, char* report, size_t report_len) {
    Config cfg;
    std::string e;
    Decomp d;
    std::ostringstream o;
    int rc = 0;
    if (config_load(config_path, &cfg, &e) != OK) { o << "config error: " << e << "\n"; rc = ERR_INVALID; }
    else if (topology_finalize(&cfg.topo, &e) != OK) { o << "topology: " << e << "\n"; rc = ERR_TOPOLOGY; }
    else if (decompose(cfg, &d, &e) != OK) { o << "decompose: " << e << "\n"; rc = ERR_INVALID; }
    else {
        VerifyReport rep;
        lint_config(cfg, d, d.mem_total <= mem_budget(cfg), &rep);
        for (const std::string& l : rep.lines) o << l << "\n";
        rc = rep.problems;
    }
    if (report && report_len) std::snprintf(report, report_len, "%s", o.str().c_str());
    return rc;
}

int cai_verify(const char* config_path, int check_exec, char* report, size_t report_len) {
    Config cfg;
    std::string e;
    std::ostringstream o;
    auto flush = [&](int rc) {
        const std::string s = o.str();
        if (report && report_len) std::snprintf(report, report_len, "%s", s.c_str());
        return rc;
    };
    if (config_load(config_path, &cfg, &e) != OK) { o << "config error: " << e << "\n"; return flush(ERR_INVALID); }
    if (topology_finalize(&cfg.topo, &e) != OK) { o << "topology: " << e << "\n"; return flush(ERR_TOPOLOGY); }
    Decomp d;
    if (decompose(cfg, &d, &e) != OK) { o << "decompose: " << e << "\n"; return flush(ERR_INVALID); }
    const uint64_t ph = plan_hash(cfg, d), th = topology_hash(cfg.topo);
    const bool moe = cfg.model.is_moe != 0;
    VerifyReport rep;
    char line[256];
    std::snprintf(line, sizeof line, "verifying %u ranks (TP=%u PP=%u DP=%u EP=%u)\n", cfg.topo.world_size, d.tp, d.pp,
                  d.dp, d.ep);
    o << line << "[1] communicator tiling (all ranks)\n";
    size_t shown = 0;
    auto dump = [&] {
        for (; shown < rep.lines.size(); ++shown) o << rep.lines[shown] << "\n";
    };
    verify_tiling(d, cfg.topo, moe, GROUP_TP, "TP", &rep);
    verify_tiling(d, cfg.topo, moe, GROUP_DP, "DP", &rep);
    verify_tiling(d, cfg.topo, moe, GROUP_PP, "PP", &rep);
    if (moe && d.ep > 1) verify_tiling(d, cfg.topo, moe, GROUP_EP, "EP", &rep);
    dump();

    o << "[2] hash agreement + [4] pipeline p2p conservation\n";
    uint64_t sends = 0, recvs = 0;
    bool hash_ok = true;
    std::vector<Plan> stage_plans;
    for (uint32_t s = 0; s < d.pp; ++s) {
        const uint32_t r = s * d.tp * d.cp;
        Plan p;
        if (build_plan_v1(cfg, d, r, ph, th, &p, &e) != OK) {
            rep.lines.push_back("  [FAIL] stage " + std::to_string(s) + ": build: " + e);
            rep.problems++;
            continue;
        }
        if (p.hdr.plan_hash != ph || p.hdr.topology_hash != th || p.hdr.pipeline_stage != s) hash_ok = false;
        for (const Op& op : p.ops) {
            if (op.kind == OP_PIPE_SEND) ++sends;
            else if (op.kind == OP_PIPE_RECV) ++recvs;
        }
    }
    if (hash_ok) {
        std::snprintf(line, sizeof line, "  [ok]   all %u stages share plan_hash=%016llx topology_hash=%016llx", d.pp,
                      (unsigned long long)ph, (unsigned long long)th);
        rep.lines.push_back(line);
    } else {
        rep.lines.push_back("  [FAIL] hash / stage mismatch across stages");
        rep.problems++;
    }
    const uint64_t expect = 2ull * (d.pp - 1) * d.num_microbatches;
    if (sends == recvs && sends == expect) {
        std::snprintf(line, sizeof line, "  [ok]   pipeline p2p conserved: %llu sends == %llu recvs == 2*(PP-1)*m",
                      (unsigned long long)sends, (unsigned long long)recvs);
        rep.lines.push_back(line);
    } else {
        std::snprintf(line, sizeof line, "  [FAIL] pipeline p2p: sends=%llu recvs=%llu expected=%llu",
                      (unsigned long long)sends, (unsigned long long)recvs, (unsigned long long)expect);
        rep.lines.push_back(line);
        rep.problems++;
    }
    dump();

    o << "[3] intra-stage op-stream identity\n";
    if (d.dp > 1) {
        Plan a, b;
        const uint32_t ra = 0, rb = d.model_replica_gpus;
        if (build_plan_v1(cfg, d, ra, ph, th, &a, &e) == OK && build_plan_v1(cfg, d, rb, ph, th, &b, &e) == OK) {
            const bool same = a.ops.size() == b.ops.size() &&
                              std::memcmp(a.ops.data(), b.ops.data(), a.ops.size() * sizeof(Op)) == 0;
            std::snprintf(line, sizeof line,
                          same ? "  [ok]   stage-0 ranks %u and %u emit identical %zu-op streams"
                               : "  [FAIL] stage-0 ranks %u and %u differ in op stream (%zu ops)",
                          ra, rb, a.ops.size());
            rep.lines.push_back(line);
            if (!same) rep.problems++;
        } else {
            rep.lines.push_back("  [FAIL] build for identity check failed");
            rep.problems++;
        }
    } else {
        rep.lines.push_back("  [ok]   DP=1: nothing to cross-check");
    }
    dump();

    if (check_exec) {
        o << "[5] executable plan: event order, arena hazards, pipeline pairing\n";
        std::vector<Plan> plans;
        bool built = true;
        for (uint32_t s = 0; s < d.pp && built; ++s) {
            Plan p;
            if (build_plan_v2(cfg, d, s * d.tp * d.cp, ph, th, &p, &e) != OK) {
                rep.lines.push_back("  [warn] no executable plan for this config: " + e);
                built = false;
                break;
            }
            plans.push_back(std::move(p));
        }
        if (built) {
            for (const Plan& p : plans) {
                verify_event_order(p, &rep);
                verify_hazards(p, &rep);
                verify_peer_reuse(p, &rep);
            }
            verify_pipeline_pairing(plans, &rep);
            if (plans.size() > 1) {
                // every send must be able to meet its receive once streams, events and the rendezvous of NCCL
                // point-to-point calls are taken together: replay all stages as one graph and look for a cycle
                std::vector<const Plan*> ptrs;
                for (const Plan& p : plans) ptrs.push_back(&p);
                Backend* be = backend_analytic_create();
                PipelineResult pr;
                std::string why;
                const int rc = replay_pipeline(ptrs, cfg.topo, be, &pr, &why);
                be->destroy(be);
                if (rc == OK) {
                    std::snprintf(line, sizeof line, "  [ok]   the %zu stages replay together without a deadlock", plans.size());
                    rep.lines.push_back(line);
                } else {
                    rep.lines.push_back("  [FAIL] joint replay of the stages: " + why);
                    rep.problems++;
                }
            }
        }
        dump();
    }
    if (rep.problems) o << "\nRESULT: " << rep.problems << " problem(s)\n";
    else o << "\nRESULT: all checks passed\n";
    return flush(rep.problems);
}

}  // extern "C"
