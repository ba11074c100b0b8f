/* cai.h - public C API of the host library (libcai_host.so).
 *
 * The runtime half mirrors the reference's public API (include/cai.h:29-89): load a compiled
 * plan + topology, replay it step by step, read per-step statistics, trace, checkpoint. Here the
 * replay uses the analytic cost backend ("simulate" mode): it needs no GPU and predicts the step
 * time, pipeline bubble, MFU and tokens/s of a schedule. The device runtime that executes the
 * same op table with real kernels lives in libcai_kernels.so (csrc/runtime).
 *
 * The compiler half exposes the offline tools to other languages: parse a config, decompose,
 * build and write plans, verify a whole cluster. */
#ifndef CAI_PUBLIC_H
#define CAI_PUBLIC_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct cai_context cai_context_t;

typedef struct {
    uint32_t global_rank;
    uint32_t world_size;
    uint32_t local_rank;
    const char* plan_path;
    const char* topology_path;
    const char* checkpoint_path; /* NULL: start from scratch */
    uint32_t checkpoint_every;   /* steps; 0 disables */
    uint32_t max_steps;          /* 0: run until the caller stops */
    uint32_t backend;            /* CAI_BACKEND_*: which backend replays the plan (the CAI_BACKEND environment
                                  * variable, "analytic" / "calibrated" / "device" / "auto", overrides CAI_BACKEND_DEFAULT) */
} cai_init_desc_t;

enum {
    CAI_BACKEND_DEFAULT = 0,  /* analytic unless the environment says otherwise */
    CAI_BACKEND_ANALYTIC = 1, /* cost model, no GPU: predicts step time, bubble, MFU */
    CAI_BACKEND_DEVICE = 2,   /* execute the plan on the GPU of local_rank (needs a version-2 plan); fail if impossible */
    CAI_BACKEND_AUTO = 3,     /* device when a GPU and the kernel library are there, else analytic (the reference's order,
                               * src/runtime.c:32-73) */
    CAI_BACKEND_CALIBRATED = 4 /* cost model fitted to this repository's kernels as measured on B200s, no GPU (needs a
                                * version-2 plan; constants can be overridden from the file named by CAI_CALIBRATION) */
};

typedef struct {
    uint32_t step;
    uint64_t tokens;
    uint64_t seed;
} cai_batch_t;

typedef struct {
    double step_time_s;
    double busy_compute_s;
    double bubble_ratio;
    double mfu;
    double tokens_per_s;
    double tokens_per_s_per_gpu;
    uint64_t arena_bytes;
    double stream_busy[6];
    /* filled by an executing backend (0 under the analytic one) */
    double loss;                 /* mean loss of the step */
    double bubble_measured;      /* share of the step the main compute stream had no op in flight */
    uint32_t measured;           /* 1: times above are measurements, 0: predictions of the cost model */
    uint32_t reserved;
} cai_step_stats_t;

typedef struct {
    uint32_t op_index;
    uint16_t kind;
    uint16_t stream;
    double start_s;
    double end_s;
    uint64_t bytes;
    uint64_t flops;
} cai_trace_rec_t;

/* Result of cai_pipeline_replay: all stages of one pipeline replayed together (sends meet their receives), so fill,
 * drain, uneven stages and transfer times are in step_time_s without the closed bubble formula. */
#define CAI_MAX_PIPELINE_STAGES 64
typedef struct {
    uint32_t n_stages;
    uint32_t reserved;
    double step_time_s;
    double bubble_formula;       /* (pp-1)/(m+pp-1), for comparison */
    double bubble_replayed;      /* share of the step the busiest stage's main compute stream stands still */
    double tokens_per_s;
    double mfu;
    double stage_finish_s[CAI_MAX_PIPELINE_STAGES];  /* end of the stage's longest path, streams overlapping freely */
    double stage_busy_hi_s[CAI_MAX_PIPELINE_STAGES];
    double stage_idle_hi[CAI_MAX_PIPELINE_STAGES];
    double stage_sm_busy_s[CAI_MAX_PIPELINE_STAGES]; /* sum of duration x share of the SMs over all streams (0: the backend does not say) */
} cai_pipeline_stats_t;

const char* cai_status_str(int status);
void cai_log_set_level(int level);   /* 0 error, 1 warn, 2 info (default), 3 debug; CAI_LOG_LEVEL sets the starting level */

int cai_init(cai_context_t** ctx, const cai_init_desc_t* desc);
int cai_load_plan(cai_context_t* ctx, const char* path);
int cai_load_checkpoint(cai_context_t* ctx, const char* path);
int cai_next_batch(cai_context_t* ctx, cai_batch_t* batch);
int cai_train_step(cai_context_t* ctx, const cai_batch_t* batch);
int cai_should_checkpoint(cai_context_t* ctx);
int cai_save_checkpoint(cai_context_t* ctx, const char* tag);
int cai_last_step_stats(cai_context_t* ctx, cai_step_stats_t* out);
int cai_trace_enable(cai_context_t* ctx, int on);
int cai_trace_dump_csv(cai_context_t* ctx, const char* path);
int cai_trace_dump_json(cai_context_t* ctx, const char* path);   /* Trace Event format (chrome://tracing, Perfetto) */
int cai_finalize(cai_context_t* ctx);
/* plan_paths[s]: the plan file of one rank of stage s. backend: CAI_BACKEND_ANALYTIC or CAI_BACKEND_CALIBRATED
 * (calibration_path may be NULL). trace_json_path (may be NULL): Trace Event timeline, one process per stage.
 * CAI_ERR_DEPENDENCY with the op named in err when the stages' sends and receives deadlock. */
int cai_pipeline_replay(const char* const* plan_paths, uint32_t n_stages, const char* topology_path, uint32_t backend,
                        const char* calibration_path, const char* trace_json_path, cai_pipeline_stats_t* out, char* err,
                        size_t errlen);
uint32_t cai_current_step(cai_context_t* ctx);
const char* cai_backend_name(cai_context_t* ctx);   /* "analytic", "calibrated" or "device" */

/* ---- compiler entry points (used by the Python package through ctypes) ---------------- */

/* Compile `config_path` and write topology.bin plus plan.rankNNNNNN.bin for ranks
 * [rank_lo, rank_hi) into outdir. version = 1 (reference-format, cost only) or 2 (executable).
 * Writes plan_hash / topology_hash when the pointers are non-NULL. err receives a message. */
int cai_compile(const char* config_path, const char* outdir, uint32_t rank_lo, uint32_t rank_hi,
                uint32_t version, uint64_t* plan_hash, uint64_t* topology_hash, char* err, size_t errlen);
/* Same, from config text. */
int cai_compile_text(const char* config_text, const char* outdir, uint32_t rank_lo, uint32_t rank_hi,
                     uint32_t version, uint64_t* plan_hash, uint64_t* topology_hash, char* err, size_t errlen);
/* Whole-cluster verification; returns the number of problems (0 = pass), negative on error.
 * The report text is written into `report`. */
int cai_verify(const char* config_path, int check_exec, char* report, size_t report_len);
/* Pre-compile checks of a configuration (memory budget, tensor-parallel placement, rank <-> location round trips,
 * pipeline bubble): "[ok]" / "[warn]" / "[FAIL]" lines in `report`; returns the number of failed checks,
 * negative when the configuration cannot be read. */
int cai_lint(const char* config_path, char* report, size_t report_len);
/* Decomposition summary as "key=value\n" lines. */
int cai_describe(const char* config_text, char* out, size_t out_len, char* err, size_t errlen);
/* Members of a communicator, for building process groups. Returns the count. */
int cai_group_members(const char* config_text, uint16_t kind, uint32_t rank, uint32_t* out, uint32_t cap);
uint64_t cai_fnv1a64(const void* data, size_t len, uint64_t seed);

/* ---- checkpoint files ("<path>.<tag>.rank%06u" + rolling "<path>.latest.rank%06u") ------
 * Layout: u32 step, u64 plan_hash (the reference's 12 bytes), then u32 'CKP3', u32 nsections,
 * then per section {char name[16]; u64 nbytes; u64 hash} followed by the payloads. The hash (FNV-1a over
 * 64-bit words) is checked when a section is read back; files with the older 'CKP2' table (no hash) load. */
int cai_ckpt_write(const char* path, const char* tag, uint32_t rank, uint32_t step, uint64_t plan_hash,
                   uint32_t nsections, const char* const* names, const void* const* data,
                   const uint64_t* nbytes);
/* Same; roll_latest = 0 writes only "<path>.<tag>.rank..." and leaves the rolling "latest" file alone. */
int cai_ckpt_write2(const char* path, const char* tag, uint32_t rank, uint32_t step, uint64_t plan_hash,
                    uint32_t nsections, const char* const* names, const void* const* data,
                    const uint64_t* nbytes, int roll_latest);
/* Reads the header of the newest checkpoint for `rank` (prefers .latest). Returns 0 and fills
 * step / plan_hash / nsections, 1 if no checkpoint exists, negative on error. */
int cai_ckpt_probe(const char* path, uint32_t rank, uint32_t* step, uint64_t* plan_hash, uint32_t* nsections,
                   char* resolved, size_t resolved_len);
int cai_ckpt_section(const char* file, uint32_t index, char name[16], uint64_t* nbytes, void* dst, uint64_t cap);

#ifdef __cplusplus
}
#endif

#endif /* CAI_PUBLIC_H */
