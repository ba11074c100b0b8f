// plan.h - the offline compiler: config -> decomposition -> per-rank plan, plus the helpers the
// tools and runtimes share (logging, hashing, raw IO, formatting, topology math, 1F1B schedule,
// arena packing, plan files, verification).
#pragma once

#include <cstdio>
#include <string>
#include <vector>

#include "formats.h"

namespace cai {

// ---- logging (stderr, "[cai LEVEL] msg") ------------------------------------------------
enum LogLevel { LOG_ERROR = 0, LOG_WARN, LOG_INFO, LOG_DEBUG };
void log_set_level(LogLevel lv);
void logf(LogLevel lv, const char* fmt, ...) __attribute__((format(printf, 2, 3)));

// ---- small utilities -----------------------------------------------------------------
constexpr uint64_t kFnvInit = 1469598103934665603ull;
uint64_t fnv1a(const void* data, size_t len, uint64_t seed = kFnvInit);
bool write_all(FILE* f, const void* buf, size_t n);
bool read_all(FILE* f, void* buf, size_t n);
std::string fmt_bytes(uint64_t bytes);   // "1.82 GiB"
std::string fmt_count(double v);         // "408.03B"
inline uint64_t align_up(uint64_t v, uint64_t a) { return (v + a - 1) & ~(a - 1); }
constexpr uint64_t kArenaAlign = 512;
bool mkdir_p(const std::string& path);

const char* status_str(int status);
size_t dtype_size(uint16_t dt);
const char* dtype_name(uint16_t dt);
const char* tclass_name(uint16_t c);
const char* stream_name(uint16_t s);
const char* op_name(uint16_t k);
const char* kernel_name(uint16_t k);
bool op_is_comm(uint16_t k);
bool op_is_compute(uint16_t k);

// ---- topology ------------------------------------------------------------------------
void topology_default(Topology* t);                      // GB300 NVL72 figures, like the reference
int topology_finalize(Topology* t, std::string* err);    // derives world_size, validates
PhysId phys_of_rank(const Topology& t, uint32_t rank);
uint32_t rank_of(const Topology& t, uint16_t rack, uint8_t tray, uint8_t gpu);
bool same_rack(const Topology& t, uint32_t a, uint32_t b);
int spare_rank(const Topology& t, uint32_t failed_rank, uint32_t* out);
int topology_write(const std::string& path, const Topology& t);
int topology_read(const std::string& path, Topology* t);
uint64_t topology_hash(const Topology& t);

// ---- config ----------------------------------------------------------------------------
void config_defaults(Config* cfg);
int config_load(const std::string& path, Config* cfg, std::string* err);
int config_parse(const std::string& text, Config* cfg, std::string* err);

// ---- decomposition -------------------------------------------------------------------
struct Decomp {
    uint32_t tp, pp, ep, cp, dp, vpp;
    uint32_t model_replica_gpus;
    uint64_t global_batch, global_tokens;
    uint32_t num_microbatches, layers_per_stage;
    double bubble_ratio;
    uint64_t mem_param, mem_grad, mem_opt, mem_act, mem_comm, mem_ws, mem_total;
    double flops_per_token_train, flops_per_token_useful, step_flops;
    uint64_t total_params, active_params;
};
int decompose(const Config& cfg, Decomp* out, std::string* err);
uint64_t mem_budget(const Config& cfg);
bool report_decomp(FILE* f, const Config& cfg, const Decomp& d);  // true if memory fits
uint64_t plan_hash(const Config& cfg, const Decomp& d);
uint64_t layer_params_total(const ModelSpec& m);
uint64_t layer_params_active(const ModelSpec& m);

// ---- pipeline ------------------------------------------------------------------------
struct Tick { uint16_t kind; uint16_t microbatch; };  // kind 0 = forward, 1 = backward
double pipeline_bubble(uint32_t pp, uint32_t m);
double pipeline_bubble_interleaved(uint32_t pp, uint32_t m, uint32_t vpp);
std::vector<Tick> schedule_1f1b(uint32_t stage, uint32_t pp, uint32_t m);

// ---- arena ---------------------------------------------------------------------------
struct Arena { uint64_t seg_off[TC_COUNT], seg_len[TC_COUNT], total; };
void arena_layout(Arena* a, const uint64_t want[TC_COUNT]);
void arena_relocate(const Arena& a, TensorDesc* tensors, uint32_t n);

// ---- plans ---------------------------------------------------------------------------
struct Plan {
    PlanHeader hdr{};
    std::vector<TensorDesc> tensors;
    std::vector<CommGroup> groups;
    std::vector<Op> ops;
    // version 2 only
    ExecHeader xhdr{};
    TrainSpec train{};
    ModelSpec model{};
    std::vector<ExecOp> exec;
    std::vector<NamedTensor> named;
    std::vector<uint32_t> shapes;  // 4 x uint32 per tensor: rows, cols, ld, slot count
};
uint32_t rank_stage(const Decomp& d, uint32_t rank);
std::vector<CommGroup> rank_groups(const Decomp& d, const Topology& topo, bool is_moe, uint32_t rank);
bool rank_group(const Decomp& d, const Topology& topo, bool is_moe, uint16_t kind, uint32_t rank, CommGroup* out);  // false: the rank has no group of this kind
// Members of the communicator of `kind` that `rank` belongs to, in group-rank order.
std::vector<uint32_t> group_members(const Decomp& d, bool is_moe, uint16_t kind, uint32_t rank);

// Version-1 plan: the reference's cost-only schedule, byte for byte.
int build_plan_v1(const Config& cfg, const Decomp& d, uint32_t rank, uint64_t ph, uint64_t th, Plan* out,
                  std::string* err);
// Version-2 plan: an executable schedule with real tensors and kernel records.
int build_plan_v2(const Config& cfg, const Decomp& d, uint32_t rank, uint64_t ph, uint64_t th, Plan* out,
                  std::string* err);
// Bytes every tensor class occupies in a plan's arena (extent from the lowest offset to the highest end of the class's
// tensors, so views and reused workspace count once): what a device really allocates, next to the model the
// decomposition report prints (the reference's formula, which e.g. counts gradients at the parameter width).
void plan_class_bytes(const Plan& p, uint64_t out[TC_COUNT]);
int plan_write(const std::string& path, const Plan& p);
int plan_read(const std::string& path, Plan* p);
void plan_arena_breakdown(const Plan& p, uint64_t out_bytes[TC_COUNT]);

// ---- verification ----------------------------------------------------------------------
struct VerifyReport {
    int problems = 0;
    std::vector<std::string> lines;  // "[ok] ..." / "[FAIL] ..."
};
void verify_tiling(const Decomp& d, const Topology& topo, bool is_moe, uint16_t kind, const char* name,
                   VerifyReport* rep);
// Every WAIT follows its RECORD, event ids in range, stream ids valid.
void verify_event_order(const Plan& p, VerifyReport* rep);
// Happens-before analysis over streams + events: no two ops that touch overlapping arena bytes
// (at least one writing) may be unordered. Needs a version-2 plan.
void verify_hazards(const Plan& p, VerifyReport* rep);
// Cross-rank reuse of the buffers the fused tensor-parallel kernels share between GPUs: every reuse is separated
// from the peers' accesses by an op that orders the whole group. Needs a version-2 plan.
void verify_peer_reuse(const Plan& p, VerifyReport* rep);
// Pairwise send/recv order between adjacent pipeline stages (not just counts).
void verify_pipeline_pairing(const std::vector<Plan>& stage_plans, VerifyReport* rep);

// Pre-compile sanity checks of a configuration; `memory_fits` is what report_decomp returned.
void lint_config(const Config& cfg, const Decomp& d, bool memory_fits, VerifyReport* rep);

// Which tensors an exec record reads / writes (ids into Plan::tensors).
void exec_operands(const ExecOp& x, std::vector<int>* reads, std::vector<int>* writes);

}  // namespace cai
