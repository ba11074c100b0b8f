// trainer <plan.bin> <topology.bin> [--steps N] [--ckpt PATH] [--ckpt-every K] [--trace CSV] [--device | --backend B]
// trainer <plan.bin> <topology.bin> --pipeline [--backend analytic|calibrated] [--calibration FILE] [--trace x.json]
//
// Replays a compiled plan: per-step critical path, pipeline bubble, MFU and tokens/s, per-stream
// occupancy, optional op timeline as CSV, periodic and emergency checkpoints. Same command line and
// table as the reference (tools/trainer.c). The backend is chosen at cai_init: the analytic cost model
// (default, no GPU), or with --device the executor of the kernel library, which runs a single-rank
// executable plan on the GPU and fills the same table with measurements plus a loss column
// (--backend auto takes the device when there is one, like the reference's cai_init). Multi-rank
// jobs run through `python -m cai_b200.trainer`.
//
// --pipeline replays the plans of ALL stages of the pipeline the given plan belongs to (its siblings are looked up in
// the same directory) as one graph in which sends meet their receives, instead of correcting one stage's busy time
// with the closed bubble formula: per-stage finish times and idle shares, step time, and a deadlock report when the
// stages' sends and receives cannot all meet.
#include <cstdio>
#include <cstdlib>
#include <cstring>

#include <string>
#include <vector>

#include "cai.h"
#include "plan.h"

// The plans of all stages of the pipeline `plan_path` belongs to, replayed together.
static int run_pipeline(const char* plan_path, const char* topology_path, uint32_t backend, const char* trace) {
    cai::Plan p;
    if (cai::plan_read(plan_path, &p) != cai::OK) { std::fprintf(stderr, "cannot read plan '%s'\n", plan_path); return 1; }
    const cai::PlanHeader& h = p.hdr;
    const uint32_t stride = h.tp * (h.cp ? h.cp : 1), base = h.global_rank - h.pipeline_stage * stride;
    std::string dir = plan_path;
    const size_t slash = dir.find_last_of('/');
    dir = slash == std::string::npos ? "." : dir.substr(0, slash);
    std::vector<std::string> paths;
    std::vector<const char*> cpaths;
    for (uint32_t s = 0; s < h.num_stages; ++s) {
        char name[64];
        std::snprintf(name, sizeof name, "/plan.rank%06u.bin", base + s * stride);
        paths.push_back(dir + name);
        if (FILE* f = std::fopen(paths.back().c_str(), "rb")) std::fclose(f);
        else {
            std::fprintf(stderr, "stage %u of the pipeline needs %s: compile the plans of all stages (plan_compiler --all, or --rank %u)\n", s,
                         paths.back().c_str(), base + s * stride);
            return 1;
        }
    }
    for (const std::string& q : paths) cpaths.push_back(q.c_str());
    cai_pipeline_stats_t st;
    char err[512] = "";
    const int rc = cai_pipeline_replay(cpaths.data(), h.num_stages, topology_path, backend, std::getenv("CAI_CALIBRATION"), trace, &st, err, sizeof err);
    if (rc != 0) { std::fprintf(stderr, "pipeline replay failed (%s): %s\n", cai_status_str(rc), err); return 1; }
    const bool sm = st.stage_sm_busy_s[0] > 0;   // the calibrated backend knows what share of the SMs a kernel keeps busy
    std::printf("stage |   rank | finish      | compute_hi busy | idle %s\n", sm ? " | SMs busy" : "");
    std::printf("------+--------+-------------+-----------------+-------%s\n", sm ? "+---------" : "");
    for (uint32_t s = 0; s < st.n_stages; ++s) {
        std::printf("%5u | %6u | %8.2f ms | %12.2f ms | %4.1f%%", s, base + s * stride, st.stage_finish_s[s] * 1e3, st.stage_busy_hi_s[s] * 1e3,
                    st.stage_idle_hi[s] * 100.0);
        if (sm) std::printf(" | %6.1f%%", st.step_time_s > 0 ? st.stage_sm_busy_s[s] / st.step_time_s * 100.0 : 0.0);
        std::printf("\n");
    }
    std::printf("\nstep %.2f ms | %.3e tokens/s | MFU %.1f%% | busiest stage idle %.1f%% of the step; pipeline bubble by formula %.1f%%\n",
                st.step_time_s * 1e3, st.tokens_per_s, st.mfu * 100.0, st.bubble_replayed * 100.0, st.bubble_formula * 100.0);
    if (trace) std::printf("wrote the timeline of all stages to %s\n", trace);
    return 0;
}

int main(int argc, char** argv) {
    if (argc < 3) {
        std::fprintf(stderr, "usage: %s <plan.bin> <topology.bin> [--steps N] [--ckpt PATH] [--ckpt-every K] [--trace CSV] [--fail-at STEP] [--device | --backend analytic|calibrated|device|auto] [--calibration FILE] [--pipeline]\n", argv[0]);
        return 2;
    }
    cai_init_desc_t desc;
    std::memset(&desc, 0, sizeof desc);
    desc.plan_path = argv[1];
    desc.topology_path = argv[2];
    desc.max_steps = 10;
    const char* trace = nullptr;
    long fail_at = -1;  // host-side fault injection: report a backend error at this step
    bool pipeline = false;
    if (const char* r = std::getenv("RANK")) desc.global_rank = std::strtoul(r, nullptr, 10);
    if (const char* r = std::getenv("LOCAL_RANK")) desc.local_rank = std::strtoul(r, nullptr, 10);
    for (int i = 3; i < argc; ++i) {
        if (!std::strcmp(argv[i], "--steps") && i + 1 < argc) desc.max_steps = std::strtoul(argv[++i], nullptr, 10);
        else if (!std::strcmp(argv[i], "--ckpt") && i + 1 < argc) { desc.checkpoint_path = argv[++i]; if (!desc.checkpoint_every) desc.checkpoint_every = 5; }
        else if (!std::strcmp(argv[i], "--ckpt-every") && i + 1 < argc) desc.checkpoint_every = std::strtoul(argv[++i], nullptr, 10);
        else if (!std::strcmp(argv[i], "--trace") && i + 1 < argc) trace = argv[++i];
        else if (!std::strcmp(argv[i], "--fail-at") && i + 1 < argc) fail_at = std::strtol(argv[++i], nullptr, 10);
        else if (!std::strcmp(argv[i], "--device")) desc.backend = CAI_BACKEND_DEVICE;
        else if (!std::strcmp(argv[i], "--pipeline")) pipeline = true;
        else if (!std::strcmp(argv[i], "--backend") && i + 1 < argc) {
            const char* b = argv[++i];
            desc.backend = !std::strcmp(b, "device") ? CAI_BACKEND_DEVICE : !std::strcmp(b, "auto") ? CAI_BACKEND_AUTO
                         : !std::strcmp(b, "calibrated") ? CAI_BACKEND_CALIBRATED : CAI_BACKEND_ANALYTIC;
        }
        else if (!std::strcmp(argv[i], "--calibration") && i + 1 < argc) {
            setenv("CAI_CALIBRATION", argv[++i], 1);   // constants of the calibrated backend, key = value
            if (desc.backend == CAI_BACKEND_DEFAULT) desc.backend = CAI_BACKEND_CALIBRATED;
        }
        else { std::fprintf(stderr, "unknown arg: %s\n", argv[i]); return 2; }
    }
    if (pipeline) return run_pipeline(argv[1], argv[2], desc.backend, trace);
    cai_context_t* ctx = nullptr;
    int rc = cai_init(&ctx, &desc);
    if (rc != 0) { std::fprintf(stderr, "init failed: %s\n", cai_status_str(rc)); return 1; }
    if (desc.checkpoint_path && (rc = cai_load_checkpoint(ctx, desc.checkpoint_path)) != 0) {
        std::fprintf(stderr, "checkpoint rejected: %s\n", cai_status_str(rc));
        cai_finalize(ctx);
        return 1;
    }
    if (trace) cai_trace_enable(ctx, 1);
    const bool device = !std::strcmp(cai_backend_name(ctx), "device");
    std::printf("step | step_time | bubble |   MFU  | tokens/s    | tok/s/gpu%s\n", device ? " |   loss" : "");
    std::printf("-----+-----------+--------+--------+-------------+----------%s\n", device ? "+--------" : "");
    double sum_mfu = 0, sum_tps = 0;
    unsigned n = 0;
    cai_step_stats_t st;
    for (;;) {
        cai_batch_t batch;
        if (cai_next_batch(ctx, &batch) != 0) break;
        rc = (static_cast<long>(batch.step) == fail_at) ? -6 : cai_train_step(ctx, &batch);
        if (rc != 0) {
            std::fprintf(stderr, "step %u failed: %s\n", batch.step, cai_status_str(rc));
            cai_save_checkpoint(ctx, "emergency");
            cai_finalize(ctx);
            return 1;
        }
        cai_last_step_stats(ctx, &st);
        std::printf("%4u | %7.2f ms| %5.1f%% | %5.1f%% | %9.2e | %8.1f", batch.step, st.step_time_s * 1e3,
                    st.bubble_ratio * 100.0, st.mfu * 100.0, st.tokens_per_s, st.tokens_per_s_per_gpu);
        if (st.measured) std::printf(" | %7.4f", st.loss);
        std::printf("\n");
        sum_mfu += st.mfu;
        sum_tps += st.tokens_per_s;
        ++n;
        if (cai_should_checkpoint(ctx) && cai_save_checkpoint(ctx, "periodic") != 0)
            std::fprintf(stderr, "warning: checkpoint write failed at step %u\n", batch.step);
    }
    if (n) {
        std::printf("\nsummary: %u steps | avg MFU %.1f%% | avg %.3e tokens/s | arena %.2f GiB/gpu\n", n, sum_mfu / n * 100.0,
                    sum_tps / n, st.arena_bytes / (1024.0 * 1024.0 * 1024.0));
        static const char* names[] = {"compute_hi", "compute_lo", "comm_tp", "comm_pp", "comm_dp", "io"};
        std::printf("per-stream occupancy (ms)%s: ", st.measured ? ", measured" : "");
        for (int s = 0; s < 6; ++s) std::printf("%s=%.1f ", names[s], st.stream_busy[s] * 1e3);
        std::printf("\n");
        if (st.measured) std::printf("compute stream idle %.1f%% of the step (measured); pipeline bubble by formula %.1f%%\n",
                                     st.bubble_measured * 100.0, st.bubble_ratio * 100.0);
    }
    if (trace) {   // *.json: Trace Event format for chrome://tracing / Perfetto; anything else: the reference's CSV
        const size_t n = std::strlen(trace);
        const bool json = n > 5 && !std::strcmp(trace + n - 5, ".json");
        if ((json ? cai_trace_dump_json(ctx, trace) : cai_trace_dump_csv(ctx, trace)) == 0) std::printf("wrote op timeline to %s\n", trace);
    }
    cai_finalize(ctx);
    return 0;
}
