// runtime_sim.cc - the op-table replayer with the analytic cost backend, per-step statistics,
// tracing and checkpoint files. No GPU needed.
//
// Semantics follow the reference runtime (src/runtime.c:129-213) and its analytic backend
// (src/backend_cpu.c:51-68): six stream clocks advance in program order, EVENT_RECORD copies a
// stream clock into an event, EVENT_WAIT takes the max, every other op adds its modelled
// duration. Differences on purpose: the plan hash IS checked when a checkpoint is loaded, and
// checkpoint files are written to a temporary name and renamed.
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <memory>

#include "backend.h"
#include "cai.h"
#include "plan.h"

namespace cai {

constexpr double kHopLatency = 1.5e-6;

// Modelled seconds an op occupies its stream.
double analytic_op_seconds(const Topology& topo, const Op& op, const CommGroup* g) {
    double t = 0.0;
    const bool comm = op_is_comm(op.kind);
    if (op_is_compute(op.kind)) t += static_cast<double>(op.flops) / topo.gpu_flops_bf16;
    if (comm || (op.kind >= OP_COUNT_V1 && op.bytes)) {
        const double bw = static_cast<double>((g && g->intra_rack) ? topo.intra_rack_bw : topo.inter_rack_bw);
        const double n = g ? static_cast<double>(g->size) : 1.0;
        if (op.kind == OP_PIPE_SEND || op.kind == OP_PIPE_RECV) return kHopLatency + static_cast<double>(op.bytes) / bw;
        double hops = 0.0;
        for (double k = n; k > 1.0; k *= 0.5) hops += 1.0;  // ceil(log2 n)
        double factor = 1.0, steps = 1.0;
        if (n <= 1.0) {
            factor = 0.0;
            steps = 0.0;
        } else if (op.kind == OP_ALL_REDUCE) {
            factor = 2.0 * (n - 1.0) / n;
            steps = 2.0 * hops;
        } else if (op.kind == OP_REDUCE_SCATTER || op.kind == OP_ALL_GATHER) {
            factor = (n - 1.0) / n;
            steps = hops;
        } else if (op.kind == OP_ALL_TO_ALL) {
            factor = (n - 1.0) / n;
            steps = 1.0;
        } else {
            // fused kernels: the transfer overlaps the math tile by tile, so the op costs the
            // slower of the two (roofline), not their sum
            const double wire = (n - 1.0) / n * static_cast<double>(op.bytes) / bw + kHopLatency;
            return t > wire ? t : wire;
        }
        return kHopLatency * steps + factor * static_cast<double>(op.bytes) / bw;
    }
    return t;
}

namespace {
double analytic_vt(Backend*, const Topology& topo, const Op& op, const CommGroup* g) { return analytic_op_seconds(topo, op, g); }
void analytic_destroy(Backend* be) { delete be; }
}  // namespace

Backend* backend_analytic_create() {
    auto be = new Backend();
    be->name = "analytic";
    be->impl = nullptr;
    be->op_seconds = analytic_vt;
    be->load_plan = nullptr;
    be->run_step = nullptr;
    be->snapshot = nullptr;
    be->restore = nullptr;
    be->sync = nullptr;
    be->destroy = analytic_destroy;
    return be;
}

}  // namespace cai

using namespace cai;

struct cai_context {
    Backend* be = nullptr;
    ~cai_context() { if (be) be->destroy(be); }
    cai_init_desc_t desc{};
    std::string plan_path, topo_path, ckpt_path;
    Topology topo{};
    Plan plan;
    bool plan_loaded = false;
    uint32_t step = 0;
    cai_step_stats_t last{};
    std::vector<double> event_time;
    // The op table with every price looked up. A pricing backend is a function of the op, its communicator and the
    // topology alone, so the table is priced when the first step of a plan runs; every later step only advances the
    // six stream clocks over these entries (one per op, same order).
    struct ReplayEntry {
        double dur;       // modelled seconds (work entries)
        double sm;        // dur x share of the SMs the op keeps busy (0 when the backend does not say)
        uint32_t event;   // record / wait entries
        uint8_t what;     // 0 work, 1 record, 2 wait
        uint8_t stream;
    };
    std::vector<ReplayEntry> replay;
    int replay_status = OK;
    bool trace_on = false;
    std::vector<cai_trace_rec_t> trace;
};

// Prices the loaded plan's op table once. Returns the status the first malformed op would give a step.
static int price_table(cai_context* ctx) {
    const Plan& p = ctx->plan;
    ctx->replay.clear();
    ctx->replay.reserve(p.ops.size());
    const CommGroup* by_id[16] = {};
    for (const CommGroup& c : p.groups)
        if (c.group_id < 16) by_id[c.group_id] = &c;      // later entries win, as a linear search for the last match does
    for (const Op& op : p.ops) {
        cai_context::ReplayEntry r{};
        if (op.stream_id >= ST_COUNT) return ERR_PLAN;
        r.stream = static_cast<uint8_t>(op.stream_id);
        if (op.kind == OP_EVENT_RECORD || op.kind == OP_EVENT_WAIT) {
            if (op.aux0 >= p.hdr.num_events) return op.kind == OP_EVENT_RECORD ? ERR_PLAN : ERR_DEPENDENCY;
            r.what = op.kind == OP_EVENT_RECORD ? 1 : 2;
            r.event = op.aux0;
        } else {
            const CommGroup* g = nullptr;
            if (op_is_comm(op.kind) || op.kind >= OP_COUNT_V1) {
                if (op.aux0 < 16) g = by_id[op.aux0];
                else
                    for (const CommGroup& c : p.groups)
                        if (c.group_id == op.aux0) g = &c;
                if (!g && op_is_comm(op.kind)) return ERR_PLAN;
            }
            r.dur = ctx->be->op_seconds(ctx->be, ctx->topo, op, g);
            if (ctx->be->op_sm_share) r.sm = r.dur * ctx->be->op_sm_share(ctx->be, ctx->topo, op, g);
        }
        ctx->replay.push_back(r);
    }
    return OK;
}

extern "C" {

const char* cai_status_str(int status) { return status_str(status); }
void cai_log_set_level(int level) { log_set_level(static_cast<LogLevel>(level < 0 ? 0 : level > 3 ? 3 : level)); }

int cai_init(cai_context_t** out, const cai_init_desc_t* desc) {
    auto ctx = std::make_unique<cai_context>();
    ctx->desc = *desc;
    std::string err;
    if (desc->topology_path) {
        ctx->topo_path = desc->topology_path;
        if (int rc = topology_read(ctx->topo_path, &ctx->topo); rc != OK) {
            logf(LOG_ERROR, "cannot read topology '%s'", desc->topology_path);
            return rc;
        }
        if (topology_finalize(&ctx->topo, &err) != OK) {
            logf(LOG_ERROR, "bad topology: %s", err.c_str());
            return ERR_TOPOLOGY;
        }
    } else {
        topology_default(&ctx->topo);
        topology_finalize(&ctx->topo, &err);
    }
    if (desc->checkpoint_path) ctx->ckpt_path = desc->checkpoint_path;
    // backend selection: the descriptor, unless it leaves the choice open and the environment makes one
    uint32_t want = desc->backend;
    if (want == CAI_BACKEND_DEFAULT) {
        const char* env = std::getenv("CAI_BACKEND");
        want = !env ? CAI_BACKEND_ANALYTIC : !std::strcmp(env, "device") ? CAI_BACKEND_DEVICE
             : !std::strcmp(env, "auto") ? CAI_BACKEND_AUTO : !std::strcmp(env, "calibrated") ? CAI_BACKEND_CALIBRATED
             : CAI_BACKEND_ANALYTIC;
    }
    if (want == CAI_BACKEND_CALIBRATED) {
        std::string why;
        ctx->be = backend_calibrated_create(std::getenv("CAI_CALIBRATION"), &why);
        if (!ctx->be) {
            logf(LOG_ERROR, "calibrated backend: %s", why.c_str());
            return ERR_BACKEND;
        }
    }
    if (want == CAI_BACKEND_DEVICE || want == CAI_BACKEND_AUTO) {
        std::string why;
        ctx->be = backend_device_create(desc->local_rank, &why);
        if (!ctx->be && want == CAI_BACKEND_DEVICE) {
            logf(LOG_ERROR, "device backend unavailable: %s", why.c_str());
            return ERR_BACKEND;
        }
        if (!ctx->be) logf(LOG_INFO, "device backend unavailable (%s): falling back to the analytic backend", why.c_str());
    }
    if (!ctx->be) ctx->be = backend_analytic_create();
    logf(LOG_INFO, "rank %u/%u backend=%s", desc->global_rank, ctx->topo.world_size, ctx->be->name);
    if (desc->plan_path) {
        if (int rc = cai_load_plan(ctx.get(), desc->plan_path); rc != OK) return rc;
    }
    *out = ctx.release();
    return OK;
}

int cai_load_plan(cai_context_t* ctx, const char* path) {
    Plan p;
    if (int rc = plan_read(path, &p); rc != OK) {
        logf(LOG_ERROR, "cannot read plan '%s': %s", path, status_str(rc));
        return rc;
    }
    if (p.hdr.topology_hash != topology_hash(ctx->topo)) {
        logf(LOG_ERROR, "plan was compiled for a different topology (hash mismatch)");
        return ERR_TOPOLOGY;
    }
    if (p.hdr.world_size != ctx->topo.world_size) {
        logf(LOG_ERROR, "plan world_size %u != topology world_size %u", p.hdr.world_size, ctx->topo.world_size);
        return ERR_PLAN;
    }
    if (ctx->be && ctx->be->load_plan) {
        if (int rc = ctx->be->load_plan(ctx->be, p, path, ctx->desc.global_rank, ctx->topo.world_size); rc != OK) return rc;
    }
    ctx->plan = std::move(p);
    ctx->plan_path = path;
    ctx->event_time.assign(ctx->plan.hdr.num_events ? ctx->plan.hdr.num_events : 1, 0.0);
    ctx->replay.clear();
    ctx->plan_loaded = true;
    logf(LOG_INFO, "plan loaded: stage %u/%u ops=%u groups=%u arena=%.2f GiB", ctx->plan.hdr.pipeline_stage,
         ctx->plan.hdr.num_stages, ctx->plan.hdr.num_ops, ctx->plan.hdr.num_groups,
         ctx->plan.hdr.arena_bytes / (1024.0 * 1024.0 * 1024.0));
    return OK;
}

int cai_load_checkpoint(cai_context_t* ctx, const char* path) {
    uint32_t step = 0, nsec = 0;
    uint64_t ph = 0;
    char resolved[1024];
    const int rc = cai_ckpt_probe(path, ctx->desc.global_rank, &step, &ph, &nsec, resolved, sizeof resolved);
    if (rc == 1) return OK;  // nothing to resume from
    if (rc != OK) return rc;
    if (ctx->plan_loaded && ph != ctx->plan.hdr.plan_hash) {
        logf(LOG_ERROR, "checkpoint '%s' belongs to a different plan (hash %016llx, plan %016llx)", resolved,
             (unsigned long long)ph, (unsigned long long)ctx->plan.hdr.plan_hash);
        return ERR_PLAN;
    }
    if (ctx->be && ctx->be->restore) {
        for (uint32_t i = 0; i < nsec; ++i) {
            char name[17] = {0};
            uint64_t n = 0;
            if (cai_ckpt_section(resolved, i, name, &n, nullptr, 0) != OK) return ERR_IO;
            std::vector<uint8_t> buf(n);
            if (cai_ckpt_section(resolved, i, name, &n, buf.data(), n) != OK) return ERR_IO;
            if (int rc2 = ctx->be->restore(ctx->be, name, buf.data(), n); rc2 != OK) return rc2;
        }
    }
    ctx->step = step;
    logf(LOG_INFO, "resumed from checkpoint at step %u", ctx->step);
    return OK;
}

int cai_next_batch(cai_context_t* ctx, cai_batch_t* batch) {
    if (ctx->desc.max_steps && ctx->step >= ctx->desc.max_steps) return 1;
    batch->step = ctx->step;
    batch->tokens = ctx->plan_loaded ? ctx->plan.hdr.global_tokens_per_step : 0;
    batch->seed = 0x9E3779B97F4A7C15ull ^ ctx->step;
    return OK;
}

int cai_train_step(cai_context_t* ctx, const cai_batch_t* batch) {
    if (!ctx->plan_loaded) return ERR_PLAN;
    const Plan& p = ctx->plan;
    if (ctx->be && ctx->be->run_step) {
        // executing backend: the whole table runs on the device, statistics are measurements
        StepResult r;
        const uint64_t seed = batch ? batch->seed : (0x9E3779B97F4A7C15ull ^ ctx->step);
        if (int rc = ctx->be->run_step(ctx->be, ctx->step + 1, seed, ctx->trace_on, &r); rc != OK) return rc;
        ctx->trace = std::move(r.trace);
        const double useful = static_cast<double>(p.hdr.global_tokens_per_step) * static_cast<double>(p.hdr.flops_per_token_useful) /
                              p.hdr.world_size;
        cai_step_stats_t& L = ctx->last;
        L = cai_step_stats_t{};
        L.step_time_s = r.step_time_s;
        L.busy_compute_s = std::max(r.stream_busy[ST_COMPUTE_HI], r.stream_busy[ST_COMPUTE_LO]);
        L.bubble_ratio = pipeline_bubble_interleaved(p.hdr.num_stages, p.hdr.num_microbatches, p.hdr.vpp ? p.hdr.vpp : 1);
        L.mfu = r.step_time_s > 0 ? useful / (ctx->topo.gpu_flops_bf16 * r.step_time_s) : 0.0;
        L.tokens_per_s = r.step_time_s > 0 ? p.hdr.global_tokens_per_step / r.step_time_s : 0.0;
        L.tokens_per_s_per_gpu = L.tokens_per_s / p.hdr.world_size;
        L.arena_bytes = p.hdr.arena_bytes;
        for (int s = 0; s < ST_COUNT; ++s) L.stream_busy[s] = r.stream_busy[s];
        L.loss = r.loss;
        L.bubble_measured = r.hi_idle_ratio;
        L.measured = 1;
        ctx->step++;
        return OK;
    }
    if (ctx->replay.empty() && !p.ops.empty()) ctx->replay_status = price_table(ctx);
    if (ctx->replay_status != OK) return ctx->replay_status;
    double clock[ST_COUNT] = {0}, work[ST_COUNT] = {0};
    double sm_work = 0.0;  // sum of duration x share of the SMs, over all streams (backends that know the share)
    double* const event_time = ctx->event_time.data();
    std::fill(ctx->event_time.begin(), ctx->event_time.end(), 0.0);
    ctx->trace.clear();
    if (ctx->trace_on) ctx->trace.reserve(p.ops.size());
    const bool tracing = ctx->trace_on;
    const cai_context::ReplayEntry* const prog = ctx->replay.data();
    const uint32_t n_ops = static_cast<uint32_t>(ctx->replay.size());
    for (uint32_t i = 0; i < n_ops; ++i) {
        const cai_context::ReplayEntry& r = prog[i];
        double& c = clock[r.stream];
        if (r.what == 1) {
            event_time[r.event] = c;
        } else if (r.what == 2) {
            c = std::max(c, event_time[r.event]);
        } else {
            const double start = c;
            c = start + r.dur;
            work[r.stream] += r.dur;
            sm_work += r.sm;
            if (tracing) ctx->trace.push_back({i, p.ops[i].kind, r.stream, start, start + r.dur, p.ops[i].bytes, p.ops[i].flops});
        }
    }

    double busy = 0.0;
    for (double c : clock) busy = std::max(busy, c);
    busy = std::max(busy, sm_work);  // streams overlap only as far as their kernels leave SMs to each other
    const double bubble = pipeline_bubble_interleaved(p.hdr.num_stages, p.hdr.num_microbatches, p.hdr.vpp ? p.hdr.vpp : 1);
    const double step_time = bubble < 1.0 ? busy / (1.0 - bubble) : busy;
    const double useful_per_gpu = static_cast<double>(p.hdr.global_tokens_per_step) *
                                  static_cast<double>(p.hdr.flops_per_token_useful) / p.hdr.world_size;
    const double cap = ctx->topo.gpu_flops_bf16 * step_time;
    cai_step_stats_t& L = ctx->last;
    L = cai_step_stats_t{};
    L.step_time_s = step_time;
    L.busy_compute_s = std::max(clock[ST_COMPUTE_HI], clock[ST_COMPUTE_LO]);
    L.bubble_ratio = bubble;
    L.mfu = cap > 0 ? useful_per_gpu / cap : 0.0;
    L.tokens_per_s = step_time > 0 ? p.hdr.global_tokens_per_step / step_time : 0.0;
    L.tokens_per_s_per_gpu = L.tokens_per_s / p.hdr.world_size;
    L.arena_bytes = p.hdr.arena_bytes;
    for (int s = 0; s < ST_COUNT; ++s) L.stream_busy[s] = work[s];
    ctx->step++;
    return OK;
}

int cai_trace_enable(cai_context_t* ctx, int on) {
    ctx->trace_on = on != 0;
    if (!on) ctx->trace.clear();
    return OK;
}

int cai_trace_dump_csv(cai_context_t* ctx, const char* path) {
    if (ctx->trace.empty()) return ERR_INVALID;
    FILE* f = std::fopen(path, "w");
    if (!f) return ERR_IO;
    std::fprintf(f, "op_index,kind,stream,start_us,end_us,dur_us,bytes,flops\n");
    for (const cai_trace_rec_t& r : ctx->trace)
        std::fprintf(f, "%u,%s,%s,%.4f,%.4f,%.4f,%llu,%llu\n", r.op_index, op_name(r.kind), stream_name(r.stream),
                     r.start_s * 1e6, r.end_s * 1e6, (r.end_s - r.start_s) * 1e6, (unsigned long long)r.bytes,
                     (unsigned long long)r.flops);
    std::fclose(f);
    return OK;
}

// The same timeline in the Trace Event format (chrome://tracing, Perfetto): one complete event per op, one track per
// logical stream. The reference's header promises a "Chrome-trace style" dump (include/cai.h:62) and only has the CSV.
int cai_trace_dump_json(cai_context_t* ctx, const char* path) {
    if (ctx->trace.empty()) return ERR_INVALID;
    FILE* f = std::fopen(path, "w");
    if (!f) return ERR_IO;
    std::fprintf(f, "{\"displayTimeUnit\": \"ms\", \"traceEvents\": [\n");
    for (int s = 0; s < ST_COUNT; ++s)
        std::fprintf(f, "{\"ph\": \"M\", \"pid\": %u, \"tid\": %d, \"name\": \"thread_name\", \"args\": {\"name\": \"%s\"}},\n",
                     ctx->desc.global_rank, s, stream_name(static_cast<uint16_t>(s)));
    for (size_t i = 0; i < ctx->trace.size(); ++i) {
        const cai_trace_rec_t& r = ctx->trace[i];
        std::fprintf(f, "{\"ph\": \"X\", \"pid\": %u, \"tid\": %u, \"name\": \"%s\", \"ts\": %.4f, \"dur\": %.4f, "
                        "\"args\": {\"op\": %u, \"bytes\": %llu, \"flops\": %llu}}%s\n",
                     ctx->desc.global_rank, r.stream, op_name(r.kind), r.start_s * 1e6, (r.end_s - r.start_s) * 1e6, r.op_index,
                     (unsigned long long)r.bytes, (unsigned long long)r.flops, i + 1 < ctx->trace.size() ? "," : "");
    }
    std::fprintf(f, "]}\n");
    std::fclose(f);
    return OK;
}

int cai_should_checkpoint(cai_context_t* ctx) {
    return ctx->desc.checkpoint_every && ctx->step % ctx->desc.checkpoint_every == 0;
}

int cai_save_checkpoint(cai_context_t* ctx, const char* tag) {
    if (ctx->ckpt_path.empty()) return OK;
    const bool emergency = !std::strcmp(tag, "emergency");
    if (ctx->be && ctx->be->snapshot && !emergency) {
        // an executing backend has real state: parameters and optimizer moments travel with the step counter
        std::vector<std::string> names;
        std::vector<std::vector<uint8_t>> data;
        if (int rc = ctx->be->snapshot(ctx->be, &names, &data); rc != OK) return rc;
        std::vector<const char*> n;
        std::vector<const void*> d;
        std::vector<uint64_t> len;
        for (size_t i = 0; i < names.size(); ++i) {
            n.push_back(names[i].c_str());
            d.push_back(data[i].data());
            len.push_back(data[i].size());
        }
        return cai_ckpt_write(ctx->ckpt_path.c_str(), tag, ctx->desc.global_rank, ctx->step, ctx->plan.hdr.plan_hash,
                              static_cast<uint32_t>(n.size()), n.data(), d.data(), len.data());
    }
    if (emergency)   // after a failed step only the step number is recorded, and "latest" keeps the last good state
        return cai_ckpt_write2(ctx->ckpt_path.c_str(), tag, ctx->desc.global_rank, ctx->step, ctx->plan.hdr.plan_hash, 0, nullptr,
                               nullptr, nullptr, ctx->be && ctx->be->snapshot ? 0 : 1);
    return cai_ckpt_write(ctx->ckpt_path.c_str(), tag, ctx->desc.global_rank, ctx->step, ctx->plan.hdr.plan_hash, 0,
                          nullptr, nullptr, nullptr);
}

int cai_last_step_stats(cai_context_t* ctx, cai_step_stats_t* out) {
    if (!ctx->plan_loaded) return ERR_PLAN;
    *out = ctx->last;
    return OK;
}

uint32_t cai_current_step(cai_context_t* ctx) { return ctx->step; }
const char* cai_backend_name(cai_context_t* ctx) { return ctx->be ? ctx->be->name : "none"; }

int cai_finalize(cai_context_t* ctx) {
    delete ctx;
    return OK;
}

// ------------------------------------------------------------------ checkpoint files
namespace {
constexpr uint32_t kCkptMagicV2 = 0x32504B43u;  // 'CKP2': section table without checksums (still readable)
constexpr uint32_t kCkptMagic = 0x33504B43u;    // 'CKP3': every section carries a hash of its bytes
struct SectionHdrV2 { char name[16]; uint64_t nbytes; };
struct SectionHdr { char name[16]; uint64_t nbytes; uint64_t hash; };

// FNV-1a over 64-bit words (the tail byte-wise): a checkpoint of tens of GB is hashed while it is written,
// so the byte-serial form would dominate the write.
uint64_t section_hash(const void* data, uint64_t n) {
    const uint8_t* p = static_cast<const uint8_t*>(data);
    uint64_t h = kFnvInit;
    uint64_t i = 0;
    for (; i + 8 <= n; i += 8) {
        uint64_t w;
        std::memcpy(&w, p + i, 8);
        h = (h ^ w) * 1099511628211ull;
    }
    for (; i < n; ++i) h = (h ^ p[i]) * 1099511628211ull;
    return h;
}

std::string ckpt_name(const char* path, const char* tag, uint32_t rank) {
    char buf[1200];
    std::snprintf(buf, sizeof buf, "%s.%s.rank%06u", path, tag, rank);
    return buf;
}

int write_file(const std::string& file, uint32_t step, uint64_t plan_hash, uint32_t nsec, const char* const* names,
               const void* const* data, const uint64_t* nbytes) {
    const std::string tmp = file + ".tmp";
    FILE* f = std::fopen(tmp.c_str(), "wb");
    if (!f) return ERR_IO;
    bool ok = write_all(f, &step, 4) && write_all(f, &plan_hash, 8) && write_all(f, &kCkptMagic, 4) &&
              write_all(f, &nsec, 4);
    for (uint32_t i = 0; ok && i < nsec; ++i) {
        SectionHdr sh{};
        std::strncpy(sh.name, names[i], sizeof sh.name - 1);
        sh.nbytes = nbytes[i];
        sh.hash = section_hash(data[i], nbytes[i]);
        ok = write_all(f, &sh, sizeof sh);
    }
    for (uint32_t i = 0; ok && i < nsec; ++i) ok = write_all(f, data[i], nbytes[i]);
    ok = (std::fclose(f) == 0) && ok;
    if (!ok || std::rename(tmp.c_str(), file.c_str()) != 0) {
        std::remove(tmp.c_str());
        return ERR_IO;
    }
    return OK;
}
}  // namespace

int cai_ckpt_write(const char* path, const char* tag, uint32_t rank, uint32_t step, uint64_t plan_hash,
                   uint32_t nsec, const char* const* names, const void* const* data, const uint64_t* nbytes) {
    return cai_ckpt_write2(path, tag, rank, step, plan_hash, nsec, names, data, nbytes, 1);
}

int cai_ckpt_write2(const char* path, const char* tag, uint32_t rank, uint32_t step, uint64_t plan_hash,
                    uint32_t nsec, const char* const* names, const void* const* data, const uint64_t* nbytes, int roll_latest) {
    int rc = write_file(ckpt_name(path, tag, rank), step, plan_hash, nsec, names, data, nbytes);
    // roll the "latest" pointer so a resume finds the newest state without knowing the tag; a snapshot taken
    // after a failed step (possibly half-updated state) is kept under its own tag only
    if (rc == OK && roll_latest) rc = write_file(ckpt_name(path, "latest", rank), step, plan_hash, nsec, names, data, nbytes);
    return rc;
}

int cai_ckpt_probe(const char* path, uint32_t rank, uint32_t* step, uint64_t* plan_hash, uint32_t* nsections,
                   char* resolved, size_t resolved_len) {
    std::string file = ckpt_name(path, "latest", rank);
    FILE* f = std::fopen(file.c_str(), "rb");
    if (!f) {
        file = path;
        f = std::fopen(file.c_str(), "rb");
    }
    if (!f) return 1;
    uint32_t st = 0, magic = 0, ns = 0;
    uint64_t ph = 0;
    int rc = OK;
    if (!read_all(f, &st, 4)) rc = ERR_IO;
    else if (!read_all(f, &ph, 8)) ph = 0;               // step-only file: tolerated
    else if (read_all(f, &magic, 4) && (magic == kCkptMagic || magic == kCkptMagicV2)) {
        if (!read_all(f, &ns, 4)) rc = ERR_IO;
    }
    std::fclose(f);
    if (rc != OK) return rc;
    if (step) *step = st;
    if (plan_hash) *plan_hash = ph;
    if (nsections) *nsections = ns;
    if (resolved && resolved_len) std::snprintf(resolved, resolved_len, "%s", file.c_str());
    return OK;
}

int cai_ckpt_section(const char* file, uint32_t index, char name[16], uint64_t* nbytes, void* dst, uint64_t cap) {
    FILE* f = std::fopen(file, "rb");
    if (!f) return ERR_IO;
    uint32_t st, magic = 0, ns = 0;
    uint64_t ph;
    int rc = OK;
    if (!read_all(f, &st, 4) || !read_all(f, &ph, 8) || !read_all(f, &magic, 4) ||
        (magic != kCkptMagic && magic != kCkptMagicV2) || !read_all(f, &ns, 4) || index >= ns)
        rc = ERR_INVALID;
    std::vector<SectionHdr> hdrs(rc == OK ? ns : 0);
    const bool hashed = magic == kCkptMagic;
    if (rc == OK && hashed && !read_all(f, hdrs.data(), ns * sizeof(SectionHdr))) rc = ERR_IO;
    if (rc == OK && !hashed) {
        std::vector<SectionHdrV2> old(ns);
        if (!read_all(f, old.data(), ns * sizeof(SectionHdrV2))) rc = ERR_IO;
        for (uint32_t i = 0; rc == OK && i < ns; ++i) {
            std::memcpy(hdrs[i].name, old[i].name, 16);
            hdrs[i].nbytes = old[i].nbytes;
        }
    }
    if (rc == OK) {
        uint64_t off = 0;
        for (uint32_t i = 0; i < index; ++i) off += hdrs[i].nbytes;
        if (name) std::memcpy(name, hdrs[index].name, 16);
        if (nbytes) *nbytes = hdrs[index].nbytes;
        if (dst) {
            if (cap < hdrs[index].nbytes) rc = ERR_INVALID;
            else if (std::fseek(f, static_cast<long>(off), SEEK_CUR) != 0 || !read_all(f, dst, hdrs[index].nbytes))
                rc = ERR_IO;
            else if (hashed && section_hash(dst, hdrs[index].nbytes) != hdrs[index].hash) {
                logf(LOG_ERROR, "checkpoint '%s': section '%.16s' fails its checksum", file, hdrs[index].name);
                rc = ERR_IO;
            }
        }
    }
    std::fclose(f);
    return rc;
}

uint64_t cai_fnv1a64(const void* data, size_t len, uint64_t seed) { return fnv1a(data, len, seed ? seed : kFnvInit); }

}  // extern "C"
