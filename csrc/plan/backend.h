// backend.h - what the runtime asks of a backend.
//
// The runtime (runtime_sim.cc) owns the plan, the step counter, statistics, tracing and checkpoint
// files; a backend turns one step of the op table into times. Three exist:
//   * analytic: prices every op from its FLOPs / bytes and the topology's datasheet figures; the
//     runtime walks the op table over six stream clocks (no GPU);
//   * calibrated: prices every op with costs fitted to this repository's kernels as measured on B200s (no GPU);
//   * device: hands the whole table to the executor in libcai_kernels.so, which launches the real
//     kernels on six CUDA streams, and reports measured times and the loss.
// Same role as the reference's `struct cai_backend {name, impl, op_seconds, sync, destroy}`
// (src/backend.h:16-32), whose CUDA member is a stub (src/backend_cuda.c:13-30); here the device member
// is real, so the vtable also has the entry an executing backend needs (run_step).
#pragma once

#include <string>
#include <vector>

#include "cai.h"
#include "plan.h"

namespace cai {

struct StepResult {
    double step_time_s = 0.0;          // first op start to last op end, measured
    double stream_busy[ST_COUNT] = {};  // summed op durations per logical stream
    double hi_idle_ratio = 0.0;        // share of the step compute_hi had no op in flight
    double loss = 0.0;
    bool has_loss = false;
    std::vector<cai_trace_rec_t> trace;  // filled when the caller asked for a timeline
};

struct Backend {
    const char* name;
    void* impl;
    // Pricing backends: modelled seconds `op` occupies its stream (`g` = its communicator or null).
    double (*op_seconds)(Backend* be, const Topology& topo, const Op& op, const CommGroup* g);
    // Optional for pricing backends: the share of the GPU's SMs the op keeps busy while it runs (0..1). When given,
    // the replayer does not let a step be shorter than the sum of duration x share over all streams.
    double (*op_sm_share)(Backend* be, const Topology& topo, const Op& op, const CommGroup* g) = nullptr;
    // Executing backends: bind a plan (file bytes; the plan is parsed again by the executor) ...
    int (*load_plan)(Backend* be, const Plan& plan, const std::string& path, uint32_t rank, uint32_t world);
    // ... and run one optimizer step of it on a synthetic batch drawn from `seed`.
    int (*run_step)(Backend* be, uint32_t step_1based, uint64_t seed, bool want_trace, StepResult* out);
    // Parameters + optimizer state for checkpoints: section names, host copies (filled by the call).
    int (*snapshot)(Backend* be, std::vector<std::string>* names, std::vector<std::vector<uint8_t>>* data);
    int (*restore)(Backend* be, const std::string& name, const void* data, uint64_t nbytes);
    int (*sync)(Backend* be);
    void (*destroy)(Backend* be);
};

// Joint replay of all stages of one pipeline under a pricing backend (pipeline_sim.cc).
struct PipelineResult {
    struct Stage {
        double finish_s = 0.0;               // when the stage's last op ends on the longest path (streams overlapping freely)
        double stream_busy[ST_COUNT] = {};   // summed op durations per logical stream
        double sm_work_s = 0.0;              // sum of duration x share of the SMs (backends that know the share)
        double idle_hi = 0.0;                // share of the step compute_hi has no op in flight
    };
    struct Rec { uint32_t stage; cai_trace_rec_t rec; };
    double step_time_s = 0.0, bubble_formula = 0.0, tokens_per_s = 0.0, mfu = 0.0;
    std::vector<Stage> stages;
    bool want_trace = false;
    std::vector<Rec> trace;
};
// `stages[s]` is the plan of one rank of stage s (same tensor / data coordinates). ERR_DEPENDENCY (with the op named in
// *err) when the sends and receives of neighbouring stages can never all meet.
int replay_pipeline(const std::vector<const Plan*>& stages, const Topology& topo, Backend* be, PipelineResult* out, std::string* err);

Backend* backend_analytic_create();
// Costs fitted to measurements on B200s (backend_calibrated.cc); `calibration_path` (may be null) overrides constants
// from a key = value file. nullptr (with the reason in *why) when that file cannot be read or names an unknown key.
Backend* backend_calibrated_create(const char* calibration_path, std::string* why);
// nullptr (with the reason in *why) when the kernel library or a CUDA device is missing.
Backend* backend_device_create(uint32_t local_rank, std::string* why);

double analytic_op_seconds(const Topology& topo, const Op& op, const CommGroup* g);

}  // namespace cai
