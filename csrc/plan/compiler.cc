// compiler.cc - config parsing, sizing / decomposition, the decomposition report, hash guards,
// the 1F1B tick generator and arena packing.
//
// Numbers, report text and hashes agree with the reference (src/model.c:13-359, src/pipeline.c,
// src/arena.c) so that the same config gives the same plan_hash / topology_hash; the code is
// organised around a key table and small pure functions instead.
#include <cmath>
#include <cstdarg>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <sstream>

#include "plan.h"

namespace cai {

// ------------------------------------------------------------------ config
void config_defaults(Config* cfg) {
    std::memset(&cfg->model, 0, sizeof cfg->model);
    ModelSpec& m = cfg->model;
    m.hidden_size = 8192; m.ffn_hidden = 28672; m.num_layers = 80;
    m.num_heads = 64; m.num_kv_heads = 8; m.head_dim = 128;
    m.vocab_size = 128000; m.seq_len = 8192;
    m.param_dtype = DT_BF16; m.optim_dtype = DT_FP32; m.optim_states = 2;
    m.master_weights = 1; m.recompute = 1;
    m.tp = 8; m.pp = 8; m.ep = 1; m.cp = 1; m.vpp = 1; m.microbatch = 1; m.grad_accum = 32;
    topology_default(&cfg->topo);
    cfg->train = TrainSpec{};
}

namespace {

enum FieldType { F_U32, F_I32, F_U64, F_F64, F_F32, F_DTYPE, F_COMM };
struct Key { const char* name; FieldType type; size_t off; int where; };  // where: 0 model, 1 topo, 2 train
#define MKEY(n, t) {#n, t, offsetof(ModelSpec, n), 0}
#define TKEY(n, t) {#n, t, offsetof(Topology, n), 1}
#define XKEY(name, field, t) {name, t, offsetof(TrainSpec, field), 2}
const Key kKeys[] = {
    MKEY(hidden_size, F_U32), MKEY(ffn_hidden, F_U32), MKEY(num_layers, F_U32), MKEY(num_heads, F_U32),
    MKEY(num_kv_heads, F_U32), MKEY(head_dim, F_U32), MKEY(vocab_size, F_U32), MKEY(seq_len, F_U32),
    MKEY(is_moe, F_I32), MKEY(num_experts, F_U32), MKEY(moe_top_k, F_U32), MKEY(optim_states, F_U32),
    MKEY(master_weights, F_I32), MKEY(recompute, F_I32), MKEY(tp, F_U32), MKEY(pp, F_U32), MKEY(ep, F_U32),
    MKEY(cp, F_U32), MKEY(vpp, F_U32), MKEY(microbatch, F_U32), MKEY(grad_accum, F_U32), MKEY(mem_budget, F_U64),
    MKEY(param_dtype, F_DTYPE), MKEY(optim_dtype, F_DTYPE),
    TKEY(gpus_per_rack, F_U32), TKEY(trays_per_rack, F_U32), TKEY(gpus_per_tray, F_U32), TKEY(num_racks, F_U32),
    TKEY(spare_gpus, F_U32), TKEY(intra_rack_bw, F_U64), TKEY(inter_rack_bw, F_U64), TKEY(hbm_bw, F_U64),
    TKEY(gpu_flops_bf16, F_F64), TKEY(gpu_mem_bytes, F_U64),
    // keys the reference does not have; all optional
    XKEY("lr", lr, F_F32), XKEY("adam_beta1", beta1, F_F32), XKEY("adam_beta2", beta2, F_F32),
    XKEY("adam_eps", adam_eps, F_F32), XKEY("weight_decay", weight_decay, F_F32),
    XKEY("rope_theta", rope_theta, F_F32), XKEY("norm_eps", norm_eps, F_F32), XKEY("init_std", init_std, F_F32),
    XKEY("seed", seed, F_U32), XKEY("tie_embeddings", tie_embeddings, F_U32), XKEY("zero_stage", zero_stage, F_U32), XKEY("wgrad_overlap", wgrad_overlap, F_U32),
    XKEY("fp8_block", fp8_block, F_U32), XKEY("comm", comm_mode, F_COMM), XKEY("ce_chunk", ce_chunk, F_U32),
    XKEY("moe_capacity_factor", moe_capacity_factor_x100, F_F32),
    XKEY("mb_group", mb_group, F_U32), XKEY("fuse_swiglu", fuse_swiglu, F_U32), XKEY("dp_buckets", dp_buckets, F_U32),
    XKEY("wait_limit_ms", wait_limit_ms, F_U32),
};

std::string trimmed(const std::string& s) {
    size_t b = s.find_first_not_of(" \t\r\n");
    if (b == std::string::npos) return "";
    size_t e = s.find_last_not_of(" \t\r\n");
    return s.substr(b, e - b + 1);
}

bool assign(Config* cfg, const std::string& k, const std::string& v) {
    for (const Key& key : kKeys) {
        if (k != key.name) continue;
        char* base = key.where == 0 ? reinterpret_cast<char*>(&cfg->model)
                   : key.where == 1 ? reinterpret_cast<char*>(&cfg->topo)
                                    : reinterpret_cast<char*>(&cfg->train);
        void* dst = base + key.off;
        // every number goes through strtod so "288e9" works, as in the reference
        const double d = std::strtod(v.c_str(), nullptr);
        const uint64_t u = static_cast<uint64_t>(d);
        switch (key.type) {
            case F_U32: *static_cast<uint32_t*>(dst) = static_cast<uint32_t>(u); return true;
            case F_I32: *static_cast<int32_t*>(dst) = static_cast<int32_t>(u); return true;
            case F_U64: *static_cast<uint64_t*>(dst) = u; return true;
            case F_F64: *static_cast<double*>(dst) = d; return true;
            case F_F32:
                if (k == "moe_capacity_factor") *static_cast<uint32_t*>(dst) = static_cast<uint32_t>(d * 100.0 + 0.5);
                else *static_cast<float*>(dst) = static_cast<float>(d);
                return true;
            case F_DTYPE:
                for (uint16_t t = 0; t < DT_COUNT; ++t)
                    if (v == dtype_name(t)) {
                        *static_cast<uint16_t*>(dst) = t;
                        return true;
                    }
                return false;
            case F_COMM:
                if (v == "baseline" || v == "nccl" || v == "0") *static_cast<uint32_t*>(dst) = 0;
                else if (v == "fused" || v == "1") *static_cast<uint32_t*>(dst) = 1;
                else return false;
                return true;
        }
    }
    return false;
}

int failf(std::string* err, int code, const char* fmt, ...) {
    if (err) {
        char buf[256];
        va_list ap;
        va_start(ap, fmt);
        std::vsnprintf(buf, sizeof buf, fmt, ap);
        va_end(ap);
        *err = buf;
    }
    return code;
}

}  // namespace

int config_parse(const std::string& text, Config* cfg, std::string* err) {
    config_defaults(cfg);
    std::istringstream in(text);
    std::string line;
    int lineno = 0;
    while (std::getline(in, line)) {
        ++lineno;
        const size_t hash = line.find('#');
        if (hash != std::string::npos) line.resize(hash);
        const size_t eq = line.find('=');
        if (eq == std::string::npos) {
            if (!trimmed(line).empty()) return failf(err, ERR_INVALID, "line %d: expected key = value", lineno);
            continue;
        }
        const std::string k = trimmed(line.substr(0, eq)), v = trimmed(line.substr(eq + 1));
        if (k.empty()) continue;
        if (!assign(cfg, k, v))
            return failf(err, ERR_INVALID, "line %d: unknown or invalid key '%s'", lineno, k.c_str());
    }
    return OK;
}

int config_load(const std::string& path, Config* cfg, std::string* err) {
    std::ifstream f(path);
    if (!f) {
        config_defaults(cfg);
        return failf(err, ERR_IO, "cannot open config '%s'", path.c_str());
    }
    std::stringstream ss;
    ss << f.rdbuf();
    return config_parse(ss.str(), cfg, err);
}

// ------------------------------------------------------------------ sizing
static uint64_t attn_params(const ModelSpec& m) {
    const uint64_t qd = static_cast<uint64_t>(m.num_heads) * m.head_dim;
    const uint64_t kvd = static_cast<uint64_t>(m.num_kv_heads) * m.head_dim;
    return m.hidden_size * qd + 2ull * m.hidden_size * kvd + qd * m.hidden_size;
}
static uint64_t mlp_params(const ModelSpec& m) { return 3ull * m.hidden_size * m.ffn_hidden; }

uint64_t layer_params_total(const ModelSpec& m) {
    const uint64_t mlp = m.is_moe ? m.num_experts * mlp_params(m) + static_cast<uint64_t>(m.hidden_size) * m.num_experts
                                  : mlp_params(m);
    return attn_params(m) + mlp + 2ull * m.hidden_size;
}
uint64_t layer_params_active(const ModelSpec& m) {
    return attn_params(m) + (m.is_moe ? m.moe_top_k * mlp_params(m) : mlp_params(m));
}

static double forward_flops_per_token(const ModelSpec& m) {
    const double embed = static_cast<double>(m.vocab_size) * m.hidden_size;
    const double matmul = static_cast<double>(m.num_layers) * layer_params_active(m) + embed;
    const double attn = 2.0 * (static_cast<double>(m.num_heads) * m.head_dim) * m.seq_len;
    return 2.0 * matmul + m.num_layers * attn;
}

int decompose(const Config& cfg, Decomp* out, std::string* err) {
    const ModelSpec& m = cfg.model;
    Topology topo = cfg.topo;
    if (int rc = topology_finalize(&topo, err); rc != OK) return rc;

    const uint32_t ep = m.is_moe ? (m.ep ? m.ep : 1) : 1;
    if (!m.tp || !m.pp || !m.cp) return failf(err, ERR_INVALID, "tp, pp, cp must be >= 1");
    const uint64_t replica = static_cast<uint64_t>(m.tp) * m.pp * m.cp;
    if (replica > topo.world_size)
        return failf(err, ERR_INVALID, "tp*pp*cp=%llu exceeds world_size=%u", (unsigned long long)replica,
                     topo.world_size);
    if (topo.world_size % replica)
        return failf(err, ERR_INVALID, "world_size=%u not divisible by tp*pp*cp=%llu (set spare_gpus)",
                     topo.world_size, (unsigned long long)replica);
    const uint32_t dp = static_cast<uint32_t>(topo.world_size / replica);
    if (m.is_moe && dp % ep) return failf(err, ERR_INVALID, "ep=%u must divide dp=%u", ep, dp);
    if (m.pp > m.num_layers) return failf(err, ERR_INVALID, "pp=%u exceeds num_layers=%u", m.pp, m.num_layers);
    const uint32_t vpp = m.vpp ? m.vpp : 1;
    if (vpp > 1 && m.num_layers % (m.pp * vpp))
        return failf(err, ERR_INVALID, "interleave vpp=%u requires num_layers(%u) divisible by pp*vpp=%u", vpp,
                     m.num_layers, m.pp * vpp);

    Decomp d{};
    d.tp = m.tp; d.pp = m.pp; d.cp = m.cp; d.ep = ep; d.dp = dp; d.vpp = vpp;
    d.model_replica_gpus = static_cast<uint32_t>(replica);
    d.num_microbatches = m.grad_accum;
    d.layers_per_stage = (m.num_layers + m.pp - 1) / m.pp;
    d.global_batch = static_cast<uint64_t>(m.microbatch) * m.grad_accum * dp;
    d.global_tokens = d.global_batch * m.seq_len;
    d.bubble_ratio = pipeline_bubble_interleaved(m.pp, m.grad_accum, vpp);

    const uint64_t lt = layer_params_total(m), la = layer_params_active(m);
    const uint64_t embed = static_cast<uint64_t>(m.vocab_size) * m.hidden_size;  // tied
    d.total_params = m.num_layers * lt + embed + m.hidden_size;
    d.active_params = m.num_layers * la + embed;

    const double fwd = forward_flops_per_token(m);
    d.flops_per_token_useful = 3.0 * fwd;
    d.flops_per_token_train = (m.recompute ? 4.0 : 3.0) * fwd;
    d.step_flops = d.flops_per_token_train * static_cast<double>(d.global_tokens);

    // Per-GPU memory under FSDP/ZeRO-3: non-expert parameters are sharded over tp*dp, expert
    // parameters over tp*ep (replicated over dp/ep).
    const double pb = static_cast<double>(dtype_size(m.param_dtype));
    const double ob = static_cast<double>(dtype_size(m.optim_dtype));
    const uint64_t expert_per = m.is_moe ? m.num_experts * mlp_params(m) : mlp_params(m);
    const uint64_t nonexpert_per =
        attn_params(m) + 2ull * m.hidden_size + (m.is_moe ? static_cast<uint64_t>(m.hidden_size) * m.num_experts : 0);
    const double total_expert = static_cast<double>(m.num_layers) * expert_per;
    const double total_nonexpert = static_cast<double>(m.num_layers) * nonexpert_per + static_cast<double>(embed) + m.hidden_size;
    const double ne_shard = static_cast<double>(m.tp) * dp;
    const double ex_shard = m.is_moe ? static_cast<double>(m.tp) * ep : static_cast<double>(m.tp) * dp;
    const double pcount = (total_nonexpert / m.pp) / ne_shard + (total_expert / m.pp) / ex_shard;
    d.mem_param = static_cast<uint64_t>(pcount * pb);
    d.mem_grad = static_cast<uint64_t>(pcount * pb);
    d.mem_opt = static_cast<uint64_t>(pcount * (m.optim_states * ob + (m.master_weights ? 4.0 : 0.0)));

    const double tokens_eff = static_cast<double>(m.microbatch) * m.seq_len / (static_cast<double>(m.tp) * m.cp);
    const double a_per = (m.recompute ? 2.0 : 16.0) * m.hidden_size * pb;
    const double in_flight = m.pp < m.grad_accum ? m.pp : m.grad_accum;
    d.mem_act = static_cast<uint64_t>(a_per * tokens_eff * (static_cast<double>(m.num_layers) / m.pp) * in_flight);
    const double pipe_buf = 2.0 * m.hidden_size * tokens_eff * pb;
    const double tp_scratch = static_cast<double>(m.hidden_size) * tokens_eff * pb;
    const double dp_w = 2.0 * (static_cast<double>(lt) / m.tp / (m.is_moe ? ep : 1)) * pb;
    d.mem_comm = static_cast<uint64_t>(pipe_buf + tp_scratch + dp_w);
    d.mem_ws = static_cast<uint64_t>(4.0 * m.hidden_size * tokens_eff * pb);
    d.mem_total = d.mem_param + d.mem_grad + d.mem_opt + d.mem_act + d.mem_comm + d.mem_ws;
    *out = d;
    return OK;
}

uint64_t mem_budget(const Config& cfg) { return cfg.model.mem_budget ? cfg.model.mem_budget : cfg.topo.gpu_mem_bytes; }

bool report_decomp(FILE* f, const Config& cfg, const Decomp& d) {
    const ModelSpec& m = cfg.model;
    const uint64_t budget = mem_budget(cfg);
    const bool fits = d.mem_total <= budget;
    std::fprintf(f, "model      : hidden=%u ffn=%u layers=%u heads=%u(kv=%u) head_dim=%u\n", m.hidden_size,
                 m.ffn_hidden, m.num_layers, m.num_heads, m.num_kv_heads, m.head_dim);
    std::fprintf(f, "             vocab=%u seq=%u %s\n", m.vocab_size, m.seq_len, m.is_moe ? "MoE" : "dense");
    if (m.is_moe) std::fprintf(f, "             experts=%u top_k=%u\n", m.num_experts, m.moe_top_k);
    std::fprintf(f, "precision  : param=%s optim=%s states=%u master=%d recompute=%d\n", dtype_name(m.param_dtype),
                 dtype_name(m.optim_dtype), m.optim_states, m.master_weights, m.recompute);
    std::fprintf(f, "cluster    : racks=%u gpus/rack=%u world=%u spare=%u\n", cfg.topo.num_racks,
                 cfg.topo.gpus_per_rack, cfg.topo.world_size, cfg.topo.spare_gpus);
    std::fprintf(f, "per-gpu hw : %s FLOP/s bf16, mem %s\n", fmt_count(cfg.topo.gpu_flops_bf16).c_str(),
                 fmt_bytes(cfg.topo.gpu_mem_bytes).c_str());
    std::fprintf(f, "parallelism: TP=%u PP=%u DP=%u EP=%u CP=%u (replica=%u gpus)\n", d.tp, d.pp, d.dp, d.ep, d.cp,
                 d.model_replica_gpus);
    std::fprintf(f, "batch      : microbatch=%u grad_accum=%u -> global_batch=%llu\n", m.microbatch, m.grad_accum,
                 (unsigned long long)d.global_batch);
    std::fprintf(f, "tokens/step: %s  (%llu)\n", fmt_count((double)d.global_tokens).c_str(),
                 (unsigned long long)d.global_tokens);
    std::fprintf(f, "params     : total=%s  active/token=%s\n", fmt_count((double)d.total_params).c_str(),
                 fmt_count((double)d.active_params).c_str());
    std::fprintf(f, "pipeline   : stages=%u vpp=%u microbatches=%u bubble=%.1f%% layers/stage~%u\n", d.pp, d.vpp,
                 d.num_microbatches, d.bubble_ratio * 100.0, d.layers_per_stage);
    std::fprintf(f, "compute    : useful=%s FLOP/token  step=%s FLOP (cluster)\n",
                 fmt_count(d.flops_per_token_train / (m.recompute ? 4.0 : 3.0) * 3.0).c_str(),
                 fmt_count(d.step_flops).c_str());
    std::fprintf(f, "mem/gpu    : param=%s grad=%s opt=%s\n", fmt_bytes(d.mem_param).c_str(),
                 fmt_bytes(d.mem_grad).c_str(), fmt_bytes(d.mem_opt).c_str());
    std::fprintf(f, "             act=%s comm=%s ws=%s\n", fmt_bytes(d.mem_act).c_str(), fmt_bytes(d.mem_comm).c_str(),
                 fmt_bytes(d.mem_ws).c_str());
    std::fprintf(f, "             total=%s / budget=%s  [%s]\n", fmt_bytes(d.mem_total).c_str(),
                 fmt_bytes(budget).c_str(), fits ? "OK" : "OVER BUDGET");
    if (!fits) std::fprintf(f, "             ^ over by %s\n", fmt_bytes(d.mem_total - budget).c_str());
    return fits;
}

uint64_t plan_hash(const Config& cfg, const Decomp& d) {
    uint64_t h = fnv1a(&cfg.model, sizeof cfg.model);
    h = fnv1a(&d.dp, sizeof d.dp, h);
    return fnv1a(&d.global_batch, sizeof d.global_batch, h);
}

// ------------------------------------------------------------------ pipeline
double pipeline_bubble(uint32_t pp, uint32_t m) { return pipeline_bubble_interleaved(pp, m, 1); }
double pipeline_bubble_interleaved(uint32_t pp, uint32_t m, uint32_t vpp) {
    if (pp <= 1 || m == 0) return 0.0;
    if (vpp < 1) vpp = 1;
    return static_cast<double>(pp - 1) / static_cast<double>(static_cast<uint64_t>(vpp) * m + pp - 1);
}

// Non-interleaved 1F1B for one stage: (pp-1-stage) warm-up forwards, then forward/backward pairs
// until the forwards run out, then the remaining backwards. Always 2*m ticks.
std::vector<Tick> schedule_1f1b(uint32_t stage, uint32_t pp, uint32_t m) {
    std::vector<Tick> t;
    if (!m) return t;
    t.reserve(2 * m);
    uint32_t warm = (pp > 0 && stage < pp) ? pp - 1 - stage : 0;
    if (warm > m) warm = m;
    uint32_t f = 0, b = 0;
    while (f < warm) t.push_back({0, static_cast<uint16_t>(f++)});
    while (f < m) {
        t.push_back({0, static_cast<uint16_t>(f++)});
        t.push_back({1, static_cast<uint16_t>(b++)});
    }
    while (b < m) t.push_back({1, static_cast<uint16_t>(b++)});
    return t;
}

// ------------------------------------------------------------------ arena
void arena_layout(Arena* a, const uint64_t want[TC_COUNT]) {
    uint64_t cur = 0;
    for (int c = 0; c < TC_COUNT; ++c) {
        cur = align_up(cur, kArenaAlign);
        a->seg_off[c] = cur;
        a->seg_len[c] = want[c];
        cur += want[c];
    }
    a->total = align_up(cur, kArenaAlign);
}
void arena_relocate(const Arena& a, TensorDesc* tensors, uint32_t n) {
    for (uint32_t i = 0; i < n; ++i)
        if (tensors[i].tclass < TC_COUNT) tensors[i].offset += a.seg_off[tensors[i].tclass];
}

}  // namespace cai
